// The streaming codec decoder behind include/omni_b200_codec.h: the host-side weight folding, the per-stream state
// slots, and the order of a frame's kernels. The folding and the op order are the ones `codec::build` emits
// (crates/omni-qwen3-tts/src/codec.rs:112-448; tap layouts crates/omni-kern/src/weights.rs:98-121); small GEMMs (the
// transformer over one row per stream, the upsamplers' pointwise layers) run on gemm.h, the convs and everything with
// many rows per stream on the implicit conv GEMM of codec_gemm.cu, the glue on codec_kernels.cu.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "../../include/omni_b200_codec.h"
#include "codec.h"
#include "gemm.h"

using namespace omni;

struct omni_codec_stream {
  int32_t line = -1;
  int32_t frames = 0;
  bool live = false;
};

namespace {

constexpr int kGroups = 16, kTaps = 7, kWindow = 72;

struct Snake {
  float *alpha = nullptr, *inv_b = nullptr;
};

struct Unit {
  Snake s1, s2;
  bf16 *in_b, *c1, *c1_b, *c2;
  int64_t hist;
};

struct Block {
  Snake snake;
  bf16 *in_b, *up_w, *up_b;
  int64_t prev;
  Unit units[3];
};

struct Upsampler {
  bf16 *up_w, *zb, *dw_w, *dw_b, *ln_w, *ln_b, *pw1_w, *pw1_b, *pw2_w;
  int64_t hist;
};

struct TLayer {
  bf16 *qkv, *o, *ln2, *gate_up, *down, *next;
  int64_t ring;
};

uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

float bf2f(uint16_t h) {
  const uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

}  // namespace

struct omni_codec {
  omni_codec_config cfg;
  int device = 0, sm_count = 148;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::string error;
  std::vector<void*> allocations;
  int launches = 0, last_launches = 0;
  float last_ms = 0.f;
  int spf = 0;

  // folded weights
  bf16 *books = nullptr, *rvq_out = nullptr, *zeros = nullptr, *pre_w = nullptr, *in_w = nullptr, *in_b = nullptr,
       *ln1_0 = nullptr, *out_w = nullptr, *conv_in_b = nullptr, *conv_in_w = nullptr, *out_in_b = nullptr,
       *conv_out_w = nullptr, *conv_out_b = nullptr;
  Snake snake_out;
  std::vector<TLayer> layers;
  std::vector<Upsampler> ups;
  std::vector<Block> blocks;
  int64_t pre_hist = 0, conv_in_hist = 0, out_hist = 0;

  // per-stream state
  char* state = nullptr;
  int64_t stride = 0;
  std::vector<int32_t> free_lines;
  int pad_line = 0;
  std::vector<std::unique_ptr<omni_codec_stream>> streams;

  // activations (each max_batch * elems_per_stream) and the staged inputs
  size_t elems = 0;
  bf16 *A = nullptr, *B = nullptr, *X = nullptr, *RES = nullptr, *COL = nullptr, *PAD = nullptr;
  float* wav = nullptr;
  int32_t *in_host = nullptr, *in_dev = nullptr;  // [codes n*16 | lines n | pos n]
  float* wav_host = nullptr;
  uint32_t* err = nullptr;
  GemmScratch scratch;
  std::map<std::tuple<const void*, const void*, const void*, int>, TcGemmPlan> plans;
  std::map<std::tuple<const void*, const void*, const void*, int>, RmGemmPlan> rm_plans;
  std::map<std::tuple<const void*, const void*, const void*, int, int>, ConvGemmPlan> conv_plans;
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    int seen = 0, nodes = 0;
  };
  std::map<int, StepGraph> graphs;

  int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    error = buf;
    return code;
  }
};

#define CCUDA(m, expr)                                                                              \
  do {                                                                                              \
    cudaError_t e_ = (expr);                                                                        \
    if (e_ != cudaSuccess) return (m)->fail(OMNI_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)
#define CLAUNCH(m, expr) \
  do {                   \
    CCUDA(m, expr);      \
    ++(m)->launches;     \
  } while (0)
#define CTRY(expr)                  \
  do {                              \
    const int rc_ = (expr);         \
    if (rc_ != OMNI_OK) return rc_; \
  } while (0)

namespace {

template <typename T>
int calloc_dev(omni_codec* m, T** out, size_t count, bool zero = false) {
  void* p = nullptr;
  CCUDA(m, cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T)));
  if (zero) CCUDA(m, cudaMemset(p, 0, std::max<size_t>(count, 1) * sizeof(T)));
  m->allocations.push_back(p);
  *out = static_cast<T*>(p);
  return OMNI_OK;
}

using Index = std::unordered_map<std::string, const omni_tensor*>;
using Vec = std::vector<float>;

// One checkpoint tensor as host f32; the shape must match.
int fetch(omni_codec* m, const Index& idx, const std::string& name, std::initializer_list<int64_t> shape, Vec* out) {
  auto it = idx.find(name);
  if (it == idx.end()) return m->fail(OMNI_ERR_MISSING_TENSOR, "missing tensor %s", name.c_str());
  const omni_tensor* t = it->second;
  if (t->ndim != (int)shape.size()) return m->fail(OMNI_ERR_MISSING_TENSOR, "%s: rank %d", name.c_str(), t->ndim);
  int64_t count = 1;
  int k = 0;
  for (int64_t s : shape) {
    if (t->shape[k] != s)
      return m->fail(OMNI_ERR_MISSING_TENSOR, "%s: dim %d is %lld, expected %lld", name.c_str(), k,
                     (long long)t->shape[k], (long long)s);
    count *= s;
    ++k;
  }
  const size_t bytes = (size_t)count * (t->dtype == OMNI_BF16 ? 2 : 4);
  std::vector<unsigned char> raw(bytes);
  if (t->location == OMNI_DEVICE)
    CCUDA(m, cudaMemcpy(raw.data(), t->data, bytes, cudaMemcpyDeviceToHost));
  else
    memcpy(raw.data(), t->data, bytes);
  out->resize((size_t)count);
  if (t->dtype == OMNI_BF16) {
    const uint16_t* h = reinterpret_cast<const uint16_t*>(raw.data());
    for (int64_t i = 0; i < count; ++i) (*out)[i] = bf2f(h[i]);
  } else {
    memcpy(out->data(), raw.data(), bytes);
  }
  return OMNI_OK;
}

int put(omni_codec* m, const Vec& v, bf16** out) {
  std::vector<uint16_t> h(v.size());
  for (size_t i = 0; i < v.size(); ++i) h[i] = f2bf(v[i]);
  CTRY(calloc_dev(m, out, v.size()));
  CCUDA(m, cudaMemcpy(*out, h.data(), h.size() * 2, cudaMemcpyHostToDevice));
  return OMNI_OK;
}

int put_f32(omni_codec* m, const Vec& v, float** out) {
  CTRY(calloc_dev(m, out, v.size()));
  CCUDA(m, cudaMemcpy(*out, v.data(), v.size() * 4, cudaMemcpyHostToDevice));
  return OMNI_OK;
}

// [out, in, k] -> [out, k * in], tap-major: the matrix the taps of a conv's input rows multiply.
Vec conv_taps(const Vec& w, int o, int i, int k) {
  Vec r((size_t)o * k * i);
  for (int a = 0; a < o; ++a)
    for (int j = 0; j < k; ++j)
      for (int c = 0; c < i; ++c) r[((size_t)a * k + j) * i + c] = w[((size_t)a * i + c) * k + j];
  return r;
}

// [in, out, k] -> [k * out, in]: the matrix whose product with [l, in] rows an overlap-add turns into the transposed conv.
Vec transposed_taps(const Vec& w, int i, int o, int k) {
  Vec r((size_t)k * o * i);
  for (int j = 0; j < k; ++j)
    for (int a = 0; a < o; ++a)
      for (int c = 0; c < i; ++c) r[((size_t)j * o + a) * i + c] = w[((size_t)c * o + a) * k + j];
  return r;
}

Vec scale_rows(const Vec& w, const Vec& s) {
  Vec r(w.size());
  const size_t cols = w.size() / s.size();
  for (size_t i = 0; i < w.size(); ++i) r[i] = w[i] * s[i / cols];
  return r;
}

// w [n, k] . v [k], f32 accumulation in index order
Vec matvec(const Vec& w, const Vec& v) {
  const size_t k = v.size(), n = w.size() / k;
  Vec r(n);
  for (size_t a = 0; a < n; ++a) {
    float acc = 0.f;
    for (size_t c = 0; c < k; ++c) acc += w[a * k + c] * v[c];
    r[a] = acc;
  }
  return r;
}

int snake_weights(omni_codec* m, const Index& idx, const std::string& prefix, int c, Snake* out) {
  Vec alpha, beta;
  CTRY(fetch(m, idx, prefix + ".alpha", {c}, &alpha));
  CTRY(fetch(m, idx, prefix + ".beta", {c}, &beta));
  for (auto& x : alpha) x = expf(x);
  for (auto& x : beta) x = 1.f / (expf(x) + 1e-9f);
  CTRY(put_f32(m, alpha, &out->alpha));
  return put_f32(m, beta, &out->inv_b);
}

int64_t take(int64_t* cursor, int64_t bytes) {
  const int64_t at = *cursor;
  *cursor = (at + bytes + 255) / 256 * 256;
  return at;
}

int load_weights(omni_codec* m, const Index& idx) {
  const omni_codec_config& c = m->cfg;
  const int dim = c.codebook_dim, half = dim / 2, cb = c.codebook_size, lat = c.latent_dim, h = c.hidden_size;
  const int qd = c.num_attention_heads * c.head_dim, inter = c.intermediate_size;
  int64_t cursor = 0;
  // RVQ: [first | sum of the rest] -> one projection
  Vec books;
  for (int g = 0; g < kGroups; ++g) {
    const std::string p = g == 0 ? std::string("decoder.quantizer.rvq_first.vq.layers.0")
                                 : "decoder.quantizer.rvq_rest.vq.layers." + std::to_string(g - 1);
    Vec sum, usage;
    CTRY(fetch(m, idx, p + "._codebook.embedding_sum", {cb, half}, &sum));
    CTRY(fetch(m, idx, p + "._codebook.cluster_usage", {cb}, &usage));
    for (int r = 0; r < cb; ++r)
      for (int k = 0; k < half; ++k) books.push_back(sum[(size_t)r * half + k] / std::max(usage[r], 1e-5f));
  }
  CTRY(put(m, books, &m->books));
  Vec first, rest, rvq((size_t)dim * dim);
  CTRY(fetch(m, idx, "decoder.quantizer.rvq_first.output_proj.weight", {dim, half, 1}, &first));
  CTRY(fetch(m, idx, "decoder.quantizer.rvq_rest.output_proj.weight", {dim, half, 1}, &rest));
  for (int r = 0; r < dim; ++r)
    for (int k = 0; k < half; ++k) {
      rvq[(size_t)r * dim + k] = first[(size_t)r * half + k];
      rvq[(size_t)r * dim + half + k] = rest[(size_t)r * half + k];
    }
  CTRY(put(m, rvq, &m->rvq_out));
  CTRY(put(m, Vec((size_t)std::max(dim, lat), 0.f), &m->zeros));
  Vec w, b, pre_b;
  CTRY(fetch(m, idx, "decoder.pre_conv.conv.weight", {lat, dim, 3}, &w));
  CTRY(fetch(m, idx, "decoder.pre_conv.conv.bias", {lat}, &pre_b));
  CTRY(put(m, conv_taps(w, lat, dim, 3), &m->pre_w));
  m->pre_hist = take(&cursor, 2 * 2 * (int64_t)dim * 2);
  // transformer: pre_conv's bias goes through input_proj
  const std::string pt = "decoder.pre_transformer";
  Vec in_w, in_b;
  CTRY(fetch(m, idx, pt + ".input_proj.weight", {h, lat}, &in_w));
  CTRY(fetch(m, idx, pt + ".input_proj.bias", {h}, &in_b));
  const Vec through = matvec(in_w, pre_b);
  for (int i = 0; i < h; ++i) in_b[i] += through[i];
  CTRY(put(m, in_w, &m->in_w));
  CTRY(put(m, in_b, &m->in_b));
  m->layers.resize(c.num_hidden_layers);
  for (int i = 0; i < c.num_hidden_layers; ++i) {
    const std::string q = pt + ".layers." + std::to_string(i) + ".";
    TLayer& L = m->layers[i];
    Vec ln, wq, wk, wv, wo, sa, sm, ln2, gate, up, down;
    CTRY(fetch(m, idx, q + "input_layernorm.weight", {h}, &ln));
    bf16* ln_dev = nullptr;
    CTRY(put(m, ln, &ln_dev));
    if (i == 0) m->ln1_0 = ln_dev; else m->layers[i - 1].next = ln_dev;
    CTRY(fetch(m, idx, q + "self_attn.q_proj.weight", {qd, h}, &wq));
    CTRY(fetch(m, idx, q + "self_attn.k_proj.weight", {qd, h}, &wk));
    CTRY(fetch(m, idx, q + "self_attn.v_proj.weight", {qd, h}, &wv));
    wq.insert(wq.end(), wk.begin(), wk.end());
    wq.insert(wq.end(), wv.begin(), wv.end());
    CTRY(put(m, wq, &L.qkv));
    CTRY(fetch(m, idx, q + "self_attn.o_proj.weight", {h, qd}, &wo));
    CTRY(fetch(m, idx, q + "self_attn_layer_scale.scale", {h}, &sa));
    CTRY(put(m, scale_rows(wo, sa), &L.o));
    CTRY(fetch(m, idx, q + "post_attention_layernorm.weight", {h}, &ln2));
    CTRY(put(m, ln2, &L.ln2));
    CTRY(fetch(m, idx, q + "mlp.gate_proj.weight", {inter, h}, &gate));
    CTRY(fetch(m, idx, q + "mlp.up_proj.weight", {inter, h}, &up));
    gate.insert(gate.end(), up.begin(), up.end());
    CTRY(put(m, gate, &L.gate_up));
    CTRY(fetch(m, idx, q + "mlp.down_proj.weight", {h, inter}, &down));
    CTRY(fetch(m, idx, q + "mlp_layer_scale.scale", {h}, &sm));
    CTRY(put(m, scale_rows(down, sm), &L.down));
    L.ring = take(&cursor, 2 * (int64_t)kWindow * qd * 2);
  }
  Vec norm, out_w, pending;
  CTRY(fetch(m, idx, pt + ".norm.weight", {h}, &norm));
  CTRY(put(m, norm, &m->layers.back().next));
  CTRY(fetch(m, idx, pt + ".output_proj.weight", {lat, h}, &out_w));
  CTRY(fetch(m, idx, pt + ".output_proj.bias", {lat}, &pending));
  CTRY(put(m, out_w, &m->out_w));
  // upsamplers: the transposed conv folds the bias its input still lacks into its own, per tap
  m->ups.resize(c.n_upsampling_ratios);
  for (int i = 0; i < c.n_upsampling_ratios; ++i) {
    const int r = c.upsampling_ratios[i];
    const std::string p = "decoder.upsample." + std::to_string(i);
    Upsampler& U = m->ups[i];
    Vec upw, upb, dw, dwb, lnw, lnb, pw1, pw1b, gamma, pw2, pw2b;
    CTRY(fetch(m, idx, p + ".0.conv.weight", {lat, lat, r}, &upw));
    CTRY(fetch(m, idx, p + ".0.conv.bias", {lat}, &upb));
    const Vec up = transposed_taps(upw, lat, lat, r);
    Vec zb = matvec(up, pending);
    for (int j = 0; j < r; ++j)
      for (int k = 0; k < lat; ++k) zb[(size_t)j * lat + k] += upb[k];
    CTRY(put(m, up, &U.up_w));
    CTRY(put(m, zb, &U.zb));
    CTRY(fetch(m, idx, p + ".1.dwconv.conv.weight", {lat, 1, kTaps}, &dw));
    Vec dwt((size_t)kTaps * lat);
    for (int ch = 0; ch < lat; ++ch)
      for (int j = 0; j < kTaps; ++j) dwt[(size_t)j * lat + ch] = dw[(size_t)ch * kTaps + j];
    CTRY(put(m, dwt, &U.dw_w));
    CTRY(fetch(m, idx, p + ".1.dwconv.conv.bias", {lat}, &dwb));
    CTRY(put(m, dwb, &U.dw_b));
    CTRY(fetch(m, idx, p + ".1.norm.weight", {lat}, &lnw));
    CTRY(fetch(m, idx, p + ".1.norm.bias", {lat}, &lnb));
    CTRY(put(m, lnw, &U.ln_w));
    CTRY(put(m, lnb, &U.ln_b));
    CTRY(fetch(m, idx, p + ".1.pwconv1.weight", {4 * lat, lat}, &pw1));
    CTRY(fetch(m, idx, p + ".1.pwconv1.bias", {4 * lat}, &pw1b));
    CTRY(put(m, pw1, &U.pw1_w));
    CTRY(put(m, pw1b, &U.pw1_b));
    CTRY(fetch(m, idx, p + ".1.gamma", {lat}, &gamma));
    CTRY(fetch(m, idx, p + ".1.pwconv2.weight", {lat, 4 * lat}, &pw2));
    CTRY(fetch(m, idx, p + ".1.pwconv2.bias", {lat}, &pw2b));
    CTRY(put(m, scale_rows(pw2, gamma), &U.pw2_w));
    pending = scale_rows(pw2b, gamma);
    U.hist = take(&cursor, 2 * (int64_t)(kTaps - 1) * lat * 2);
  }
  CTRY(put(m, pending, &m->conv_in_b));
  CTRY(fetch(m, idx, "decoder.decoder.0.conv.weight", {c.decoder_dim, lat, kTaps}, &w));
  CTRY(fetch(m, idx, "decoder.decoder.0.conv.bias", {c.decoder_dim}, &pending));
  CTRY(put(m, conv_taps(w, c.decoder_dim, lat, kTaps), &m->conv_in_w));
  m->conv_in_hist = take(&cursor, 2 * (int64_t)(kTaps - 1) * lat * 2);
  // decoder blocks: the bias of a conv that feeds a residual stream is carried to the stream's consumers
  m->blocks.resize(c.n_upsample_rates);
  for (int i = 0; i < c.n_upsample_rates; ++i) {
    const int rate = c.upsample_rates[i], cin = c.decoder_dim >> i, cout = c.decoder_dim >> (i + 1);
    const std::string p = "decoder.decoder." + std::to_string(i + 1) + ".block";
    Block& Bk = m->blocks[i];
    CTRY(snake_weights(m, idx, p + ".0", cin, &Bk.snake));
    CTRY(put(m, pending, &Bk.in_b));
    Vec up, upb;
    CTRY(fetch(m, idx, p + ".1.conv.weight", {cin, cout, 2 * rate}, &up));
    CTRY(fetch(m, idx, p + ".1.conv.bias", {cout}, &upb));
    CTRY(put(m, transposed_taps(up, cin, cout, 2 * rate), &Bk.up_w));
    CTRY(put(m, upb, &Bk.up_b));
    Bk.prev = take(&cursor, (int64_t)rate * cout * 2);
    pending.assign((size_t)cout, 0.f);
    const int dilation[3] = {1, 3, 9};
    for (int u = 0; u < 3; ++u) {
      const std::string q = p + "." + std::to_string(u + 2);
      Unit& Un = Bk.units[u];
      Vec c1, c1b, c2, c2b;
      CTRY(snake_weights(m, idx, q + ".act1", cout, &Un.s1));
      CTRY(fetch(m, idx, q + ".conv1.conv.weight", {cout, cout, kTaps}, &c1));
      CTRY(fetch(m, idx, q + ".conv1.conv.bias", {cout}, &c1b));
      CTRY(put(m, conv_taps(c1, cout, cout, kTaps), &Un.c1));
      CTRY(put(m, c1b, &Un.c1_b));
      CTRY(snake_weights(m, idx, q + ".act2", cout, &Un.s2));
      CTRY(fetch(m, idx, q + ".conv2.conv.weight", {cout, cout, 1}, &c2));
      CTRY(fetch(m, idx, q + ".conv2.conv.bias", {cout}, &c2b));
      CTRY(put(m, c2, &Un.c2));
      CTRY(put(m, pending, &Un.in_b));
      for (int k = 0; k < cout; ++k) pending[k] += c2b[k];
      Un.hist = take(&cursor, 2 * (int64_t)(kTaps - 1) * dilation[u] * cout * 2);
    }
  }
  const int n = c.n_upsample_rates + 1, out_dim = c.decoder_dim >> c.n_upsample_rates;
  CTRY(snake_weights(m, idx, "decoder.decoder." + std::to_string(n), out_dim, &m->snake_out));
  CTRY(put(m, pending, &m->out_in_b));
  Vec ow, ob;
  CTRY(fetch(m, idx, "decoder.decoder." + std::to_string(n + 1) + ".conv.weight", {1, out_dim, kTaps}, &ow));
  CTRY(fetch(m, idx, "decoder.decoder." + std::to_string(n + 1) + ".conv.bias", {1}, &ob));
  CTRY(put(m, conv_taps(ow, 1, out_dim, kTaps), &m->conv_out_w));
  CTRY(put(m, ob, &m->conv_out_b));
  m->out_hist = take(&cursor, 2 * (int64_t)(kTaps - 1) * out_dim * 2);
  m->stride = cursor;
  return OMNI_OK;
}

// Elements per stream of the largest activation any op of a frame writes.
size_t elems_per_stream(const omni_codec_config& c) {
  const int qd = c.num_attention_heads * c.head_dim;
  size_t e = std::max({(size_t)3 * c.codebook_dim, (size_t)3 * qd, (size_t)2 * c.intermediate_size, (size_t)c.latent_dim});
  int t = 1;
  for (int i = 0; i < c.n_upsampling_ratios; ++i) {
    t *= c.upsampling_ratios[i];
    e = std::max(e, (size_t)t * 4 * c.latent_dim);
  }
  e = std::max(e, (size_t)(t + kTaps - 1) * c.latent_dim);
  e = std::max(e, (size_t)t * kTaps * c.latent_dim);
  e = std::max(e, (size_t)t * c.decoder_dim);
  for (int i = 0; i < c.n_upsample_rates; ++i) {
    const int rate = c.upsample_rates[i], cout = c.decoder_dim >> (i + 1);
    e = std::max(e, (size_t)t * 2 * rate * cout);
    t *= rate;
    e = std::max(e, (size_t)(t + (kTaps - 1) * 9) * cout);
  }
  return e;
}

// y[rows, N] = x[rows, K] . w[N, K]^T on the library's dense GEMMs (K a multiple of 64).
int dense(omni_codec* m, const bf16* w, int N, int K, const bf16* x, int rows, bf16* y) {
  if (rows <= 8 || !tc_supports(N, K, rows)) {
    CLAUNCH(m, gemv_launch(w, N, K, x, rows, y, N, Epilogue{}, m->sm_count, m->stream));
    return OMNI_OK;
  }
  const auto key = std::make_tuple((const void*)w, (const void*)x, (const void*)y, rows);
  if (rm_supports(N, K, rows)) {
    auto rt = m->rm_plans.find(key);
    if (rt == m->rm_plans.end()) {
      RmGemmPlan plan;
      const int rc = rm_plan(&plan, w, N, K, x, rows, y, N, Epilogue{}, m->sm_count);
      if (rc != 0) return m->fail(OMNI_ERR_CUDA, "tensor-map encode failed (%d) for N=%d K=%d rows=%d", rc, N, K, rows);
      rt = m->rm_plans.emplace(key, plan).first;
    }
    CLAUNCH(m, rm_launch(rt->second, m->err, m->stream));
    return OMNI_OK;
  }
  auto it = m->plans.find(key);
  if (it == m->plans.end()) {
    TcGemmPlan plan;
    const int rc = tc_plan(&plan, w, N, K, x, rows, y, N, Epilogue{}, m->sm_count);
    if (rc != 0) return m->fail(OMNI_ERR_CUDA, "tensor-map encode failed (%d) for N=%d K=%d rows=%d", rc, N, K, rows);
    if (plan.partial_floats() > m->scratch.partial_floats || plan.tiles_n() * plan.row_tiles > m->scratch.counter_slots)
      return m->fail(OMNI_ERR_UNSUPPORTED, "split-K scratch too small for N=%d K=%d rows=%d", N, K, rows);
    it = m->plans.emplace(key, plan).first;
  }
  CLAUNCH(m, tc_launch(it->second, m->scratch, m->err, m->stream));
  return OMNI_OK;
}

// The implicit conv GEMM over `n` streams of T rows: x is the padded activation (taps > 1) or the dense one (taps = 1).
int conv(omni_codec* m, const bf16* w, int N, int C, int taps, int dil, const bf16* x, int T, int n, bf16* y, int kind,
         const bf16* bias = nullptr, const Snake* snake = nullptr) {
  const auto key = std::make_tuple((const void*)w, (const void*)x, (const void*)y, n, kind);
  auto it = m->conv_plans.find(key);
  if (it == m->conv_plans.end()) {
    ConvGemmPlan plan;
    const int rc = conv_plan(&plan, w, N, C, taps, dil, x, T, n, y, kind, bias, snake ? snake->alpha : nullptr,
                             snake ? snake->inv_b : nullptr, m->sm_count);
    if (rc != 0)
      return m->fail(OMNI_ERR_CUDA, "conv plan failed (%d) for N=%d C=%d taps=%d T=%d streams=%d", rc, N, C, taps, T, n);
    it = m->conv_plans.emplace(key, plan).first;
  }
  CLAUNCH(m, conv_launch(it->second, m->err, m->stream));
  return OMNI_OK;
}

// The kernels of one frame for n streams (codes, lines and pos already staged on the device).
int enqueue_frame(omni_codec* m, int n) {
  const omni_codec_config& c = m->cfg;
  const int dim = c.codebook_dim, half = dim / 2, lat = c.latent_dim, h = c.hidden_size;
  const int qd = c.num_attention_heads * c.head_dim, inter = c.intermediate_size;
  const int32_t* codes = m->in_dev;
  const int32_t* lines = m->in_dev + (size_t)m->cfg.max_batch * kGroups;
  const int32_t* pos = lines + m->cfg.max_batch;
  const CodecStateRef st{m->state, lines, pos, m->stride};
  cudaStream_t s = m->stream;
  bf16 *A = m->A, *B = m->B, *X = m->X, *RES = m->RES, *COL = m->COL, *PAD = m->PAD;

  CLAUNCH(m, launch_codec_rvq(codes, m->books, COL, n, half, c.codebook_size, s));
  CTRY(dense(m, m->rvq_out, dim, dim, COL, n, A));
  CLAUNCH(m, launch_codec_stage(A, m->zeros, nullptr, nullptr, st, m->pre_hist, PAD, n, 1, dim, 2, s));
  CLAUNCH(m, launch_codec_gather_taps(PAD, COL, n, 1, dim, 3, 1, s));
  CTRY(dense(m, m->pre_w, lat, 3 * dim, COL, n, B));
  CTRY(dense(m, m->in_w, h, lat, B, n, RES));
  CLAUNCH(m, launch_codec_add_norm(m->in_b, 0, RES, m->ln1_0, X, n, h, c.rms_norm_eps, s));
  for (const TLayer& L : m->layers) {
    CTRY(dense(m, L.qkv, 3 * qd, h, X, n, COL));
    CLAUNCH(m, launch_codec_window_attend(COL, st, L.ring, A, n, c.num_attention_heads, c.rope_theta, s));
    CTRY(dense(m, L.o, h, qd, A, n, X));
    CLAUNCH(m, launch_codec_add_norm(X, h, RES, L.ln2, X, n, h, c.rms_norm_eps, s));
    CTRY(dense(m, L.gate_up, 2 * inter, h, X, n, COL));
    CLAUNCH(m, launch_codec_silu_mul(COL, A, n, inter, s));
    CTRY(dense(m, L.down, h, inter, A, n, X));
    CLAUNCH(m, launch_codec_add_norm(X, h, RES, L.next, X, n, h, c.rms_norm_eps, s));
  }
  CTRY(dense(m, m->out_w, lat, h, X, n, A));
  bf16 *cur = A, *tmp = B;
  int t = 1;
  for (int i = 0; i < c.n_upsampling_ratios; ++i) {
    const int r = c.upsampling_ratios[i];
    const Upsampler& U = m->ups[i];
    CTRY(dense(m, U.up_w, r * lat, lat, cur, n * t, COL));  // kernel = stride: the GEMM rows are the output rows
    t *= r;
    CLAUNCH(m, launch_codec_dwconv_ln(COL, U.zb, U.dw_w, U.dw_b, U.ln_w, U.ln_b, st, U.hist, tmp, X, n, t, r, lat, 1e-6f, s));
    CTRY(dense(m, U.pw1_w, 4 * lat, lat, X, n * t, COL));
    CLAUNCH(m, launch_codec_bias_gelu(COL, U.pw1_b, (int64_t)n * t, 4 * lat, s));
    CTRY(conv(m, U.pw2_w, lat, 4 * lat, 1, 1, COL, t, n, tmp, kConvAccumulate));
    std::swap(cur, tmp);
  }
  CLAUNCH(m, launch_codec_stage(cur, m->conv_in_b, nullptr, nullptr, st, m->conv_in_hist, PAD, n, t, lat, kTaps - 1, s));
  CLAUNCH(m, launch_codec_gather_taps(PAD, COL, n, t, lat, kTaps, 1, s));
  CTRY(dense(m, m->conv_in_w, c.decoder_dim, kTaps * lat, COL, n * t, tmp));
  std::swap(cur, tmp);
  const int dilation[3] = {1, 3, 9};
  for (int i = 0; i < c.n_upsample_rates; ++i) {
    const int rate = c.upsample_rates[i], cin = c.decoder_dim >> i, cout = c.decoder_dim >> (i + 1);
    const Block& Bk = m->blocks[i];
    CLAUNCH(m, launch_codec_bias_snake(cur, Bk.in_b, Bk.snake.alpha, Bk.snake.inv_b, tmp, (int64_t)n * t, cin, s));
    CTRY(conv(m, Bk.up_w, 2 * rate * cout, cin, 1, 1, tmp, t, n, COL, kConvStore));
    CLAUNCH(m, launch_codec_overlap_add(COL, Bk.up_b, st, Bk.prev, cur, n, t, rate, cout, s));
    t *= rate;
    for (int u = 0; u < 3; ++u) {
      const Unit& Un = Bk.units[u];
      const int H = (kTaps - 1) * dilation[u];
      CLAUNCH(m, launch_codec_stage(cur, Un.in_b, Un.s1.alpha, Un.s1.inv_b, st, Un.hist, PAD, n, t, cout, H, s));
      CTRY(conv(m, Un.c1, cout, cout, kTaps, dilation[u], PAD, t, n, X, kConvBiasSnake, Un.c1_b, &Un.s2));
      CTRY(conv(m, Un.c2, cout, cout, 1, 1, X, t, n, cur, kConvAccumulate));
    }
  }
  const int out_dim = c.decoder_dim >> c.n_upsample_rates;
  CLAUNCH(m, launch_codec_out_conv(cur, m->out_in_b, m->snake_out.alpha, m->snake_out.inv_b, m->conv_out_w,
                                   m->conv_out_b, st, m->out_hist, m->wav, n, t, out_dim, s));
  return OMNI_OK;
}

int bucket_of(const omni_codec* m, int n) {
  int b = 1;
  while (b < n) b <<= 1;
  return std::min(b, m->cfg.max_batch);
}

// One frame of n live streams padded to bucket b (rows n..b-1 on the padding slot).
int decode_rows(omni_codec* m, int n, int b, omni_codec_stream* const* streams, const int32_t* codes, float* wav) {
  CCUDA(m, cudaSetDevice(m->device));
  const int mb = m->cfg.max_batch;
  int32_t* hc = m->in_host;
  int32_t* hl = hc + (size_t)mb * kGroups;
  int32_t* hp = hl + mb;
  for (int i = 0; i < b; ++i) {
    if (i < n) {
      memcpy(hc + (size_t)i * kGroups, codes + (size_t)i * kGroups, kGroups * sizeof(int32_t));
      hl[i] = streams[i]->line;
      hp[i] = streams[i]->frames;
    } else {
      memset(hc + (size_t)i * kGroups, 0, kGroups * sizeof(int32_t));
      hl[i] = m->pad_line;
      hp[i] = 0;
    }
  }
  m->launches = 0;
  CCUDA(m, cudaMemcpyAsync(m->in_dev, m->in_host, ((size_t)mb * (kGroups + 2)) * sizeof(int32_t), cudaMemcpyHostToDevice,
                           m->stream));
  CCUDA(m, cudaEventRecord(m->ev0, m->stream));
  omni_codec::StepGraph& sg = m->graphs[b];
  if (!m->cfg.use_graphs || sg.seen == 0) {
    CTRY(enqueue_frame(m, b));
    sg.seen = 1;
  } else {
    if (!sg.exec) {
      CCUDA(m, cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
      const int rc = enqueue_frame(m, b);
      cudaGraph_t graph = nullptr;
      const cudaError_t end = cudaStreamEndCapture(m->stream, &graph);  // always ends the capture, also after a failure
      if (rc != OMNI_OK || end != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return rc != OMNI_OK ? rc : m->fail(OMNI_ERR_CUDA, "frame capture: %s", cudaGetErrorString(end));
      }
      const cudaError_t inst = cudaGraphInstantiate(&sg.exec, graph, 0);
      cudaGraphDestroy(graph);
      if (inst != cudaSuccess) {
        sg.exec = nullptr;
        return m->fail(OMNI_ERR_CUDA, "frame graph: %s", cudaGetErrorString(inst));
      }
      sg.nodes = m->launches;
    }
    CCUDA(m, cudaGraphLaunch(sg.exec, m->stream));
    m->launches = sg.nodes;
  }
  CCUDA(m, cudaEventRecord(m->ev1, m->stream));
  if (n > 0)
    CCUDA(m, cudaMemcpyAsync(m->wav_host, m->wav, (size_t)n * m->spf * sizeof(float), cudaMemcpyDeviceToHost, m->stream));
  uint32_t err_host = 0;
  CCUDA(m, cudaMemcpyAsync(&err_host, m->err, sizeof(err_host), cudaMemcpyDeviceToHost, m->stream));
  CCUDA(m, cudaStreamSynchronize(m->stream));
  CCUDA(m, cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
  m->last_launches = m->launches;
  if (err_host != 0) {
    cudaMemsetAsync(m->err, 0, sizeof(uint32_t), m->stream);
    return m->fail(OMNI_ERR_DEVICE, "device error word 0x%x (a bounded wait ran out)", err_host);
  }
  if (n > 0) memcpy(wav, m->wav_host, (size_t)n * m->spf * sizeof(float));
  for (int i = 0; i < n; ++i) ++streams[i]->frames;
  return OMNI_OK;
}

int check_config(omni_codec* m) {
  const omni_codec_config& c = m->cfg;
  if (c.num_quantizers != kGroups) return m->fail(OMNI_ERR_UNSUPPORTED, "%d quantizers, the decoder is built for 16", c.num_quantizers);
  if (c.head_dim != 64) return m->fail(OMNI_ERR_UNSUPPORTED, "head_dim %d unsupported (attention is built for 64)", c.head_dim);
  if (c.sliding_window != kWindow) return m->fail(OMNI_ERR_UNSUPPORTED, "window %d unsupported (the ring is built for 72)", c.sliding_window);
  if (c.hidden_size % 256 || c.hidden_size > 1024) return m->fail(OMNI_ERR_UNSUPPORTED, "hidden size %d unsupported (256 | h <= 1024)", c.hidden_size);
  if (c.latent_dim % 64 || c.latent_dim > 8192) return m->fail(OMNI_ERR_UNSUPPORTED, "latent dim %d unsupported (64 | d <= 8192)", c.latent_dim);
  if (c.codebook_dim % 64 || c.intermediate_size % 64 || (c.num_attention_heads * 64) % 64)
    return m->fail(OMNI_ERR_UNSUPPORTED, "codebook_dim and intermediate_size must be multiples of 64");
  if (c.n_upsampling_ratios < 0 || c.n_upsampling_ratios > 4 || c.n_upsample_rates < 1 || c.n_upsample_rates > 8)
    return m->fail(OMNI_ERR_INVALID, "rate counts out of range");
  const int out_dim = c.decoder_dim >> c.n_upsample_rates;
  if (out_dim % 32 || out_dim > 128 || out_dim < 32) return m->fail(OMNI_ERR_UNSUPPORTED, "output conv width %d unsupported (32 | c <= 128)", out_dim);
  int spf = 1;
  for (int i = 0; i < c.n_upsampling_ratios; ++i) spf *= c.upsampling_ratios[i];
  for (int i = 0; i < c.n_upsample_rates; ++i) spf *= c.upsample_rates[i];
  if (spf % 64) return m->fail(OMNI_ERR_UNSUPPORTED, "the output conv needs whole 64-row tiles, got %d rows per frame", spf);
  if (c.max_batch < 1 || c.max_streams < 1) return m->fail(OMNI_ERR_INVALID, "max_batch and max_streams must be positive");
  m->spf = spf;
  return OMNI_OK;
}

int create_impl(omni_codec* m, const omni_tensor* tensors, int n_tensors) {
  CTRY(check_config(m));
  CCUDA(m, cudaSetDevice(m->device));
  cudaDeviceProp prop;
  CCUDA(m, cudaGetDeviceProperties(&prop, m->device));
  if (prop.major != 10) return m->fail(OMNI_ERR_UNSUPPORTED, "compute capability %d.%d: this library is built for sm_100a", prop.major, prop.minor);
  m->sm_count = prop.multiProcessorCount;
  if (tc_init() != 0) return m->fail(OMNI_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  tc_configure();
  conv_configure();
  CCUDA(m, cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
  CCUDA(m, cudaEventCreate(&m->ev0));
  CCUDA(m, cudaEventCreate(&m->ev1));
  Index idx;
  for (int i = 0; i < n_tensors; ++i) idx[tensors[i].name] = &tensors[i];
  CTRY(load_weights(m, idx));
  const int slots = m->cfg.max_streams + 1;  // the last one pads a call up to its bucket
  CTRY(calloc_dev(m, &m->state, (size_t)slots * m->stride, true));
  m->pad_line = slots - 1;
  for (int i = m->cfg.max_streams - 1; i >= 0; --i) m->free_lines.push_back(i);
  m->elems = elems_per_stream(m->cfg);
  const size_t cap = m->elems * m->cfg.max_batch;
  for (bf16** buf : {&m->A, &m->B, &m->X, &m->RES, &m->COL, &m->PAD}) CTRY(calloc_dev(m, buf, cap, true));
  CTRY(calloc_dev(m, &m->wav, (size_t)m->cfg.max_batch * m->spf));
  CTRY(calloc_dev(m, &m->in_dev, (size_t)m->cfg.max_batch * (kGroups + 2)));
  CTRY(calloc_dev(m, &m->err, 1, true));
  CCUDA(m, cudaMallocHost(&m->in_host, (size_t)m->cfg.max_batch * (kGroups + 2) * sizeof(int32_t)));
  CCUDA(m, cudaMallocHost(&m->wav_host, (size_t)m->cfg.max_batch * m->spf * sizeof(float)));
  m->scratch.partial_floats = (size_t)32 << 20;
  m->scratch.counter_slots = 1 << 16;
  CTRY(calloc_dev(m, &m->scratch.partials, m->scratch.partial_floats));
  CTRY(calloc_dev(m, &m->scratch.counters, (size_t)m->scratch.counter_slots, true));
  CCUDA(m, cudaDeviceSynchronize());
  return OMNI_OK;
}

}  // namespace

extern "C" {

int32_t omni_codec_create(const omni_codec_config* config, const omni_tensor* tensors, int32_t n_tensors, int32_t device,
                          omni_codec** out) {
  if (!config || !out || (!tensors && n_tensors > 0)) return OMNI_ERR_INVALID;
  omni_codec* m = new omni_codec();
  m->cfg = *config;
  m->device = device;
  *out = m;  // kept on failure so that the caller can read the error, then destroy
  return create_impl(m, tensors, n_tensors);
}

void omni_codec_destroy(omni_codec* m) {
  if (!m) return;
  cudaSetDevice(m->device);
  if (m->stream) cudaStreamSynchronize(m->stream);
  for (auto& g : m->graphs)
    if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
  for (void* p : m->allocations) cudaFree(p);
  if (m->in_host) cudaFreeHost(m->in_host);
  if (m->wav_host) cudaFreeHost(m->wav_host);
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

const char* omni_codec_last_error(const omni_codec* m) { return m ? m->error.c_str() : "null model"; }

int32_t omni_codec_open(omni_codec* m, omni_codec_stream** out) {
  if (!m || !out) return OMNI_ERR_INVALID;
  if (m->free_lines.empty()) return m->fail(OMNI_DENIED_BUSY, "every state slot is taken");
  CCUDA(m, cudaSetDevice(m->device));
  const int line = m->free_lines.back();
  // a fresh slot reads as zero: the convs' causal padding
  CCUDA(m, cudaMemsetAsync(m->state + (int64_t)line * m->stride, 0, (size_t)m->stride, m->stream));
  m->free_lines.pop_back();
  m->streams.emplace_back(new omni_codec_stream());
  omni_codec_stream* s = m->streams.back().get();
  s->line = line;
  s->frames = 0;
  s->live = true;
  *out = s;
  return OMNI_OK;
}

int32_t omni_codec_close(omni_codec* m, omni_codec_stream* s) {
  if (!m || !s || !s->live) return OMNI_ERR_INVALID;
  s->live = false;
  m->free_lines.push_back(s->line);
  for (auto it = m->streams.begin(); it != m->streams.end(); ++it)
    if (it->get() == s) {
      m->streams.erase(it);
      break;
    }
  return OMNI_OK;
}

int32_t omni_codec_stream_frames(const omni_codec_stream* s) { return s ? s->frames : -1; }

int32_t omni_codec_samples_per_frame(const omni_codec* m) { return m ? m->spf : -1; }

int32_t omni_codec_warmup(omni_codec* m) {
  if (!m) return OMNI_ERR_INVALID;
  std::vector<int> buckets;
  for (int b = 1; b < m->cfg.max_batch; b <<= 1) buckets.push_back(b);
  buckets.push_back(m->cfg.max_batch);
  for (int b : buckets)
    for (int pass = 0; pass < (m->cfg.use_graphs ? 2 : 1); ++pass) CTRY(decode_rows(m, 0, b, nullptr, nullptr, nullptr));
  // the padding slot starts from silence again (its audio is never read; this only keeps its values bounded)
  CCUDA(m, cudaMemsetAsync(m->state + (int64_t)m->pad_line * m->stride, 0, (size_t)m->stride, m->stream));
  return OMNI_OK;
}

int32_t omni_codec_decode(omni_codec* m, int32_t n, omni_codec_stream* const* streams, const int32_t* codes, float* wav) {
  if (!m || !streams || !codes || !wav) return OMNI_ERR_INVALID;
  if (n < 1 || n > m->cfg.max_batch) return m->fail(OMNI_ERR_INVALID, "%d streams, the model takes 1..%d per call", n, m->cfg.max_batch);
  for (int i = 0; i < n; ++i) {
    if (!streams[i] || !streams[i]->live) return m->fail(OMNI_ERR_INVALID, "stream %d is not open", i);
    for (int j = 0; j < i; ++j)
      if (streams[j] == streams[i]) return m->fail(OMNI_ERR_INVALID, "stream %d is given twice", i);
    for (int g = 1; g < kGroups; ++g) {
      const int32_t code = codes[(size_t)i * kGroups + g];
      if (code < 0 || code >= m->cfg.codebook_size)
        return m->fail(OMNI_ERR_INVALID, "stream %d: code %d of codebook %d is outside the book", i, code, g);
    }
    if (codes[(size_t)i * kGroups] < 0) return m->fail(OMNI_ERR_INVALID, "stream %d: negative code", i);
  }
  return decode_rows(m, n, bucket_of(m, n), streams, codes, wav);
}

int32_t omni_codec_stats(const omni_codec* m, float* last_call_gpu_ms, int32_t* last_call_launches) {
  if (!m) return OMNI_ERR_INVALID;
  if (last_call_gpu_ms) *last_call_gpu_ms = m->last_ms;
  if (last_call_launches) *last_call_launches = m->last_launches;
  return OMNI_OK;
}

}  // extern "C"
