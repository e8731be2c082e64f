// CPU oracle for the codec-frame token loop of the Qwen3-TTS talker.
//
// TEST INFRASTRUCTURE ONLY. This file restates, on the CPU, the arithmetic the
// reference performs on the GPU for one talker frame: the decoder stack, the
// talker/code-predictor glue and the fused sampler. It exists so the CUDA path
// can be checked against something that follows the reference's op order and
// rounding points. Nothing in the shipped library links, loads or calls it;
// only the tests, the smoke check and the CPU-baseline leg of the benchmark do.
//
// Parity status: the stack arithmetic (q/k norm, half-rotation RoPE, GQA,
// SwiGLU, RMSNorm) is pinned against the `transformers` Qwen3 model on CPU
// (the same model the reference's Higgs recorder uses as truth,
// tools/higgs_audio/golden.py:44-69); those vectors live in tests/golden/.
// The reference's real-checkpoint golden files are not available, so parity
// against recorded official outputs is unpinned.
//
// Every activation that the reference stores to memory as bf16 is rounded to
// bf16 here at the same point; accumulation is f32. Sections cite the
// reference file:line they follow (paths relative to the reference root).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

typedef uint16_t bf16_t;

inline float bf2f(bf16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

// Round-to-nearest-even f32 -> bf16, the rounding of `half::bf16::from_f32`
// (crates/omni-kern/src/lib.rs:62-66) and of `__float2bfloat16`
// (crates/omni-kern/kernels/common.cuh:10).
inline bf16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (bf16_t)((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return (bf16_t)(u >> 16);
}

inline float rbf(float f) { return bf2f(f2bf(f)); }

struct Tensor {
  std::vector<bf16_t> v;
  std::vector<int64_t> shape;
  int64_t rows() const { return shape.empty() ? 0 : shape[0]; }
  int64_t cols() const { return shape.size() < 2 ? 1 : shape[1]; }
};

extern "C" {
struct orc_tensor {
  const char* name;
  const void* data;
  int32_t dtype;  // 0 = bf16, 1 = f32
  int32_t ndim;
  int64_t shape[4];
  int32_t location;  // must be 0 (host)
};

struct orc_stack {
  int32_t hidden, inter, layers, q_heads, kv_heads, head_dim, vocab;
  float rms_eps, rope_theta;
};

struct orc_config {
  orc_stack talker, predictor;
  int32_t groups;
  int32_t tts_pad_token_id, codec_eos_token_id;
  float temperature;
  int32_t top_k;
  float repetition_penalty;
  float sub_temperature;
  int32_t sub_top_k;
  float top_p;       // 1.0 = the reference's behaviour
  int32_t sampler;   // 0 = host uniforms (reference), 1 = Philox per session
  int32_t min_frames, control_tokens;
};
}

struct LayerW {
  const Tensor *ln1, *q, *k, *v, *q_norm, *k_norm, *o, *ln2, *gate, *up, *down;
};

struct StackW {
  orc_stack cfg;
  std::vector<LayerW> layers;
  const Tensor* norm;
};

// y[rows, n] = bf16( x[rows, k] . w[n, k]^T ), f32 accumulation: the GEMM op of
// crates/omni-kern/src/lib.rs:144-179 (`extern:cublaslt_bf16_tn`), all operands
// bf16 row-major, one rounding of the f32 accumulator to bf16.
// (round_out = false keeps the f32 sum: only the two head GEMMs use it, and only when a test asked for the logits
// before their bf16 store, to measure how far either GPU path is from them)
void gemm(const float* x, int rows, const bf16_t* w, int n, int k, float* y, int ldy, int col0 = 0, bool round_out = true) {
#pragma omp parallel for schedule(static)
  for (int j = 0; j < n; ++j) {
    const bf16_t* wr = w + (int64_t)j * k;
    // widen the weight row once, reuse it for every input row
    float wf[8192 + 4096];
    float* wp = wf;
    std::unique_ptr<float[]> big;
    if (k > (int)(sizeof(wf) / sizeof(float))) {
      big.reset(new float[k]);
      wp = big.get();
    }
    for (int c = 0; c < k; ++c) wp[c] = bf2f(wr[c]);
    for (int r = 0; r < rows; ++r) {
      const float* xr = x + (int64_t)r * k;
      float acc[16] = {0};
      int c = 0;
      for (; c + 16 <= k; c += 16)
        for (int e = 0; e < 16; ++e) acc[e] += xr[c + e] * wp[c + e];
      float s = 0.f;
      for (; c < k; ++c) s += xr[c] * wp[c];
      for (int e = 0; e < 16; ++e) s += acc[e];
      y[(int64_t)r * ldy + col0 + j] = round_out ? rbf(s) : s;
    }
  }
}

// Test aid: 0 = the head GEMMs keep their f32 sums (every other rounding point stays), 1 = the reference's behaviour.
bool g_round_logits = true;

// crates/omni-qwen3/kernels/qwen3.cu:18-31 (`qwen3_norm_copy`): res = x,
// out = bf16(x * rsqrt(mean(x^2) + eps) * w).
void norm_copy(const float* x, const bf16_t* w, float* out, float* res, int rows, int dim, float eps) {
  for (int r = 0; r < rows; ++r) {
    const float* xr = x + (int64_t)r * dim;
    float ss = 0.f;
    for (int c = 0; c < dim; ++c) ss += xr[c] * xr[c];
    const float rs = 1.f / sqrtf(ss / dim + eps);
    for (int c = 0; c < dim; ++c) {
      const float v = xr[c];
      res[(int64_t)r * dim + c] = v;
      out[(int64_t)r * dim + c] = rbf(v * rs * bf2f(w[c]));
    }
  }
}

// crates/omni-qwen3/kernels/qwen3.cu:37-57 (`qwen3_add_norm`): res += x stored
// as bf16; the norm runs over the UNROUNDED f32 sum; row n is kept as
// out[n / every] when n % every == which.
void add_norm(const float* x, float* res, const bf16_t* w, float* out, int rows, int dim, float eps, int every,
              int which) {
  std::vector<float> v(dim);
  for (int r = 0; r < rows; ++r) {
    float ss = 0.f;
    for (int c = 0; c < dim; ++c) {
      v[c] = x[(int64_t)r * dim + c] + res[(int64_t)r * dim + c];
      ss += v[c] * v[c];
    }
    const float rs = 1.f / sqrtf(ss / dim + eps);
    for (int c = 0; c < dim; ++c) res[(int64_t)r * dim + c] = rbf(v[c]);
    if (r % every != which) continue;
    for (int c = 0; c < dim; ++c) out[(int64_t)(r / every) * dim + c] = rbf(v[c] * rs * bf2f(w[c]));
  }
}

// crates/omni-kern/kernels/common.cuh:66-76 (`silu_mul`): bf16(SiLU(g)) * u,
// the product rounded once more on store.
void silu_mul(const float* gate_up, float* act, int rows, int inter) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < inter; ++c) {
      const float g = gate_up[(int64_t)r * 2 * inter + c];
      const float u = gate_up[(int64_t)r * 2 * inter + inter + c];
      act[(int64_t)r * inter + c] = rbf(rbf(g / (1.f + expf(-g))) * u);
    }
}

// crates/omni-qwen3/kernels/qwen3.cu:66-107 (`rope_kv`): per-head RMSNorm of
// q and k (the normalised value is rounded to bf16 BEFORE the gain, :92-93),
// half-rotation rotary embedding with inv_freq = theta^(-2i/d), K and V to the
// row's KV slot, Q in place.
void rope_head(float* head, const bf16_t* w, int d, int pos, float eps, float theta) {
  float ss = 0.f;
  for (int i = 0; i < d; ++i) ss += head[i] * head[i];
  const float r = 1.f / sqrtf(ss / d + eps);
  const int half = d / 2;
  for (int i = 0; i < half; ++i) {
    const float a = rbf(head[i] * r) * bf2f(w[i]);
    const float b = rbf(head[half + i] * r) * bf2f(w[half + i]);
    const float inv_freq = 1.f / powf(theta, (float)(2 * i) / d);
    const float ang = (float)pos * inv_freq;
    const float sn = sinf(ang), cs = cosf(ang);
    head[i] = rbf(a * cs - b * sn);
    head[half + i] = rbf(b * cs + a * sn);
  }
}

// A sequence's K/V of one stack, dense by position: [layer][pos][K heads | V heads][d].
struct Kv {
  int layers = 0, width = 0;  // width = 2 * hk * d
  std::vector<std::vector<bf16_t>> data;
  void init(int l, int w, int cap) {
    layers = l;
    width = w;
    data.assign(l, std::vector<bf16_t>((size_t)cap * w));
  }
  bf16_t* at(int layer, int pos) { return data[layer].data() + (size_t)pos * width; }
};

// crates/omni-qwen3/kernels/qwen3.cu:123-207 (`attend`): scores over positions
// 0..pos, softmax in f32, output rounded to bf16. (The reference merges per-tile
// online-softmax states; the value is the same softmax up to f32 rounding.)
void attend_row(const float* q, Kv& kv, int layer, int len, int hq, int hk, int d, float scale, float* out) {
  const int G = hq / hk;
  std::vector<float> sc(len);
  for (int h = 0; h < hq; ++h) {
    const int kh = h / G;
    const float* qh = q + (int64_t)h * d;
    float m = -INFINITY;
    for (int t = 0; t < len; ++t) {
      const bf16_t* k = kv.at(layer, t) + kh * d;
      float s = 0.f;
      for (int c = 0; c < d; ++c) s += qh[c] * bf2f(k[c]);
      sc[t] = s * scale;
      m = std::max(m, sc[t]);
    }
    float l = 0.f;
    std::vector<float> acc(d, 0.f);
    for (int t = 0; t < len; ++t) {
      const float p = expf(sc[t] - m);
      l += p;
      const bf16_t* v = kv.at(layer, t) + (hk + kh) * d;
      for (int c = 0; c < d; ++c) acc[c] += p * bf2f(v[c]);
    }
    for (int c = 0; c < d; ++c) out[(int64_t)h * d + c] = rbf(acc[c] / l);
  }
}

struct Row {
  Kv* kv;
  int pos;
};

// One pass of a decoder stack over `rows` rows, op order of
// crates/omni-qwen3/src/stack.rs:152-203 (`Stack::forward`) and :207-241
// (`Stack::attention`). Row r writes its K/V at rows[r].pos of rows[r].kv and
// attends positions 0..pos of it. All K/V of the call are written before any
// row attends (the `rope` launch precedes the `attn` launch), which is what
// makes a ragged prompt causal.
void stack_forward(const StackW& S, const float* input, const std::vector<Row>& rows, float* keep_out, int every,
                   int which) {
  const orc_stack& c = S.cfg;
  const int n = (int)rows.size(), h = c.hidden, d = c.head_dim, hq = c.q_heads, hk = c.kv_heads, I = c.inter;
  const int qw = (hq + 2 * hk) * d;
  std::vector<float> x((size_t)n * h), res((size_t)n * h), qkv((size_t)n * qw), attn((size_t)n * hq * d),
      gu((size_t)n * 2 * I), act((size_t)n * I);
  norm_copy(input, S.layers[0].ln1->v.data(), x.data(), res.data(), n, h, c.rms_eps);
  const float scale = 1.f / sqrtf((float)d);
  for (int li = 0; li < c.layers; ++li) {
    const LayerW& L = S.layers[li];
    gemm(x.data(), n, L.q->v.data(), hq * d, h, qkv.data(), qw, 0);
    gemm(x.data(), n, L.k->v.data(), hk * d, h, qkv.data(), qw, hq * d);
    gemm(x.data(), n, L.v->v.data(), hk * d, h, qkv.data(), qw, (hq + hk) * d);
    for (int r = 0; r < n; ++r) {
      float* row = qkv.data() + (size_t)r * qw;
      for (int hd = 0; hd < hq; ++hd) rope_head(row + hd * d, L.q_norm->v.data(), d, rows[r].pos, c.rms_eps, c.rope_theta);
      for (int hd = 0; hd < hk; ++hd)
        rope_head(row + (hq + hd) * d, L.k_norm->v.data(), d, rows[r].pos, c.rms_eps, c.rope_theta);
      bf16_t* dst = rows[r].kv->at(li, rows[r].pos);
      for (int i = 0; i < 2 * hk * d; ++i) dst[i] = f2bf(row[hq * d + i]);
    }
#pragma omp parallel for schedule(dynamic)
    for (int r = 0; r < n; ++r)
      attend_row(qkv.data() + (size_t)r * qw, *rows[r].kv, li, rows[r].pos + 1, hq, hk, d, scale,
                 attn.data() + (size_t)r * hq * d);
    gemm(attn.data(), n, L.o->v.data(), h, hq * d, x.data(), h);
    add_norm(x.data(), res.data(), L.ln2->v.data(), x.data(), n, h, c.rms_eps, 1, 0);
    gemm(x.data(), n, L.gate->v.data(), I, h, gu.data(), 2 * I, 0);
    gemm(x.data(), n, L.up->v.data(), I, h, gu.data(), 2 * I, I);
    silu_mul(gu.data(), act.data(), n, I);
    gemm(act.data(), n, L.down->v.data(), h, I, x.data(), h);
    if (li + 1 < c.layers)
      add_norm(x.data(), res.data(), S.layers[li + 1].ln1->v.data(), x.data(), n, h, c.rms_eps, 1, 0);
    else
      add_norm(x.data(), res.data(), S.norm->v.data(), keep_out, n, h, c.rms_eps, every, which);
  }
}

// ---------------------------------------------------------------------------
// Token selection: crates/omni-qwen3-tts/kernels/talker.cu:108-293.
// The reference runs one 1024-thread block per row, four consecutive logits
// per thread. The probabilities are summed by a block scan whose association
// order decides which token a uniform lands on, so the scan tree is reproduced
// here lane by lane (`block_scan`, talker.cu:136-169). The one thing a CPU
// cannot reproduce bit for bit is `__expf`; `expf` is used instead.

inline uint32_t order_key(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

const int kSampleThreads = 1024, kPer = 4;

// Philox4x32-10 (Salmon et al., SC'11), counter = (frame, group, 0, 0),
// key = the session's 64-bit seed; the first output word becomes a uniform in
// [0, 1) with 24 bits. Used only by the native sampler mode.
inline void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1, n3 = (uint32_t)p0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

inline float philox_uniform(uint64_t seed, uint32_t frame, uint32_t group) {
  uint32_t c[4] = {frame, group, 0u, 0u};
  philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
  return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

// `draw` (talker.cu:171-257). v: processed logits, padded to 4096 with -inf.
// top_p < 1 adds nucleus filtering after top-k (not in the reference): tokens
// are ranked by descending probability (ties: lower index first) and a token
// is dropped when the probability mass ranked strictly before it is >= top_p.
int draw(const float* v, int vocab, float temperature, int top_k, float top_p, float u) {
  const int N = kSampleThreads * kPer;
  if (temperature <= 0.f) {  // talker.cu:177-188: argmax, lowest index on ties
    uint64_t best = 0;
    for (int i = 0; i < vocab; ++i) best = std::max(best, (uint64_t)order_key(v[i]) << 32 | (uint32_t)(4095 - i));
    return 4095 - (int)(best & 0xffffffffu);
  }
  std::vector<float> x(N, -INFINITY);
  std::vector<uint32_t> key(N);
  for (int i = 0; i < N; ++i) {
    x[i] = v[i] / temperature;
    key[i] = order_key(x[i]);
  }
  const int k_keep = top_k > 0 && top_k < vocab ? top_k : vocab;
  uint32_t prefix = 0;
  if (k_keep < vocab) {  // talker.cu:199-233: the k-th largest key, ties kept
    std::vector<uint32_t> s(key.begin(), key.begin() + vocab);
    std::nth_element(s.begin(), s.begin() + (k_keep - 1), s.end(), std::greater<uint32_t>());
    prefix = s[k_keep - 1];
  }
  float m = -INFINITY;
  for (int i = 0; i < N; ++i) m = std::max(m, x[i]);
  std::vector<float> p(N, 0.f);
  for (int i = 0; i < vocab; ++i) p[i] = key[i] >= prefix ? expf(x[i] - m) : 0.f;
  if (top_p < 1.f) {
    std::vector<int> idx;
    for (int i = 0; i < vocab; ++i)
      if (p[i] > 0.f) idx.push_back(i);
    std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return p[a] > p[b]; });
    float tot = 0.f;
    for (int i : idx) tot += p[i];
    float before = 0.f;
    for (size_t r = 0; r < idx.size(); ++r) {
      const float mine = p[idx[r]];
      if (r > 0 && before >= top_p * tot) p[idx[r]] = 0.f;
      before += mine;
    }
  }
  // block_scan (talker.cu:136-169): per-thread sum, Hillis-Steele inclusive
  // scan inside each warp, then the same scan over the 32 warp totals.
  std::vector<float> own(kSampleThreads), incl(kSampleThreads), wtot(32);
  for (int t = 0; t < kSampleThreads; ++t) {
    float o = 0.f;
    for (int k = 0; k < kPer; ++k) o += p[t * kPer + k];
    own[t] = o;
  }
  for (int w = 0; w < 32; ++w) {
    float xs[32];
    for (int l = 0; l < 32; ++l) xs[l] = own[w * 32 + l];
    for (int o = 1; o < 32; o <<= 1) {
      float y[32];
      for (int l = 0; l < 32; ++l) y[l] = l >= o ? xs[l - o] : 0.f;
      for (int l = 0; l < 32; ++l)
        if (l >= o) xs[l] += y[l];
    }
    for (int l = 0; l < 32; ++l) incl[w * 32 + l] = xs[l];
    wtot[w] = xs[31];
  }
  {
    float xs[32];
    for (int l = 0; l < 32; ++l) xs[l] = wtot[l];
    for (int o = 1; o < 32; o <<= 1) {
      float y[32];
      for (int l = 0; l < 32; ++l) y[l] = l >= o ? xs[l - o] : 0.f;
      for (int l = 0; l < 32; ++l)
        if (l >= o) xs[l] += y[l];
    }
    for (int l = 0; l < 32; ++l) wtot[l] = xs[l];
  }
  const float total = wtot[31];
  const float target = u * total;
  int token = -1, last = 0;
  for (int t = 0; t < kSampleThreads; ++t) {
    const int w = t >> 5;
    const float before = w > 0 ? wtot[w - 1] : 0.f;
    float run = before + incl[t] - own[t];
    for (int k = 0; k < kPer; ++k) {
      const float pk = p[t * kPer + k];
      if (pk > 0.f) {
        last = std::max(last, t * kPer + k);
        if (run <= target && target < run + pk) token = t * kPer + k;
      }
      run += pk;
    }
  }
  return token >= 0 ? token : last;
}

// The per-sequence state slot: the last frame and the repetition bitmap
// (crates/omni-qwen3-tts/src/talker.rs:104; talker.cu:265-266).
struct SeqState {
  int32_t last_frame[16];
  std::vector<uint32_t> seen;
};

// `talker_sample` (talker.cu:259-293): repetition penalty on seen codes,
// suppression of [lo, hi) except `exempt`, `exempt` blocked before
// `min_frames`, then `draw`; the result goes to the frame, the slot and (when
// penalising) the bitmap.
int sample_row(const float* logits, int vocab, float temperature, int top_k, float top_p, float penalty,
               int suppress_lo, int suppress_hi, int exempt, int min_frames, int frame, float u, int forced,
               SeqState& st, bool penalize, int group) {
  int token = forced;
  if (forced < 0) {
    std::vector<float> v(kSampleThreads * kPer, -INFINITY);
    const bool exempt_blocked = frame < min_frames;
    for (int i = 0; i < vocab; ++i) {
      float x = logits[i];
      if (penalize && (st.seen[i / 32] >> (i % 32) & 1u)) x = x > 0.f ? x / penalty : x * penalty;
      const bool in_range = i >= suppress_lo && i < suppress_hi;
      if ((in_range && i != exempt) || (i == exempt && exempt_blocked)) x = -INFINITY;
      v[i] = x;
    }
    token = std::min(std::max(draw(v.data(), vocab, temperature, top_k, top_p, u), 0), vocab - 1);
  }
  st.last_frame[group] = token;
  if (penalize) st.seen[token / 32] |= 1u << (token % 32);
  return token;
}

struct Session {
  bool live = false;
  int prompt = 0, frames = 0, cap = 0;
  uint64_t seed = 0;
  Kv kv;
  SeqState st;
  std::vector<float> hidden;  // the talker's last hidden state, bf16 values
};

struct Model {
  orc_config cfg;
  std::map<std::string, Tensor> t;
  StackW talker, pred;
  std::vector<float> pad_embed;
  std::vector<Session> sessions;
  // debug outputs of the last call (crates/omni-qwen3-tts/src/model.rs:241-262)
  std::vector<float> logits, p_logits, embeds, hidden_out;
  int last_n = 0;

  const Tensor* get(const std::string& n) const {
    auto it = t.find(n);
    if (it == t.end()) {
      fprintf(stderr, "oracle: missing tensor %s\n", n.c_str());
      return nullptr;
    }
    return &it->second;
  }
};

bool bind_stack(Model& m, StackW& S, const orc_stack& cfg, const std::string& prefix) {
  S.cfg = cfg;
  S.layers.resize(cfg.layers);
  bool ok = true;
  for (int i = 0; i < cfg.layers; ++i) {
    const std::string p = prefix + ".layers." + std::to_string(i) + ".";
    LayerW& L = S.layers[i];
    ok &= (L.ln1 = m.get(p + "input_layernorm.weight")) != nullptr;
    ok &= (L.q = m.get(p + "self_attn.q_proj.weight")) != nullptr;
    ok &= (L.k = m.get(p + "self_attn.k_proj.weight")) != nullptr;
    ok &= (L.v = m.get(p + "self_attn.v_proj.weight")) != nullptr;
    ok &= (L.q_norm = m.get(p + "self_attn.q_norm.weight")) != nullptr;
    ok &= (L.k_norm = m.get(p + "self_attn.k_norm.weight")) != nullptr;
    ok &= (L.o = m.get(p + "self_attn.o_proj.weight")) != nullptr;
    ok &= (L.ln2 = m.get(p + "post_attention_layernorm.weight")) != nullptr;
    ok &= (L.gate = m.get(p + "mlp.gate_proj.weight")) != nullptr;
    ok &= (L.up = m.get(p + "mlp.up_proj.weight")) != nullptr;
    ok &= (L.down = m.get(p + "mlp.down_proj.weight")) != nullptr;
  }
  ok &= (S.norm = m.get(prefix + ".norm.weight")) != nullptr;
  return ok;
}

std::vector<float> row_of(const Tensor* t, int64_t r) {
  const int64_t c = t->cols();
  std::vector<float> out(c);
  for (int64_t i = 0; i < c; ++i) out[i] = bf2f(t->v[r * c + i]);
  return out;
}

// x = bf16(x + b), optionally SiLU after the rounding
// (`bias_act`, crates/omni-qwen3-tts/kernels/talker.cu:28-43).
void bias_act(float* x, const bf16_t* b, int rows, int cols, bool silu) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      float v = rbf(x[(int64_t)r * cols + c] + bf2f(b[c]));
      if (silu) v = v / (1.f + expf(-v));
      x[(int64_t)r * cols + c] = rbf(v);
    }
}

// `Talker::init` (crates/omni-qwen3-tts/src/talker.rs:169-183): the <tts_pad>
// embedding through the text projection, once.
void init_pad(Model& m) {
  const int h = m.cfg.talker.hidden;
  std::vector<float> e = row_of(m.get("talker.model.text_embedding.weight"), m.cfg.tts_pad_token_id), p(h);
  gemm(e.data(), 1, m.get("talker.text_projection.linear_fc1.weight")->v.data(), h, h, p.data(), h);
  bias_act(p.data(), m.get("talker.text_projection.linear_fc1.bias")->v.data(), 1, h, true);
  m.pad_embed.assign(h, 0.f);
  gemm(p.data(), 1, m.get("talker.text_projection.linear_fc2.weight")->v.data(), h, h, m.pad_embed.data(), h);
  bias_act(m.pad_embed.data(), m.get("talker.text_projection.linear_fc2.bias")->v.data(), 1, h, false);
}

float session_uniform(const Model& m, const Session& s, const float* uniforms, int row, int group, int frame) {
  if (m.cfg.sampler == 1) return philox_uniform(s.seed, (uint32_t)frame, (uint32_t)group);
  return uniforms[row * 16 + group];
}

// `Talker::sample` (crates/omni-qwen3-tts/src/talker.rs:254-290): group 0 uses
// the talker's sampling constants, the repetition penalty, the control-token
// suppression and the end-token gate; groups 1.. the sub-talker constants.
int sample_group(Model& m, Session& s, const float* logits, int group, float u, int forced, int frame) {
  const orc_config& c = m.cfg;
  if (group == 0) {
    const int v = c.talker.vocab;
    return sample_row(logits, v, c.temperature, c.top_k, c.top_p, c.repetition_penalty, v - c.control_tokens, v,
                      c.codec_eos_token_id, c.min_frames, frame, u, forced, s.st, true, 0);
  }
  return sample_row(logits, c.predictor.vocab, c.sub_temperature, c.sub_top_k, c.top_p, 1.0f, 0, 0, -1, 0, frame, u,
                    forced, s.st, false, group);
}

// `Talker::tail` (crates/omni-qwen3-tts/src/talker.rs:293-356): codec head and
// the codebook-0 draw, then groups-1 code-predictor passes over a dense
// per-frame KV of `groups` slots; pass 1 runs two rows per sequence (the hidden
// state, then the embedding of the code just drawn) and keeps the second.
void tail(Model& m, const std::vector<int>& sids, const float* uniforms, const int32_t* force, int32_t* codes) {
  const orc_config& c = m.cfg;
  const int n = (int)sids.size(), h = c.talker.hidden, p = c.predictor.hidden, V = c.talker.vocab,
            PV = c.predictor.vocab, G = c.groups;
  m.last_n = n;
  std::vector<float> hidden((size_t)n * h);
  for (int s = 0; s < n; ++s) memcpy(&hidden[(size_t)s * h], m.sessions[sids[s]].hidden.data(), h * sizeof(float));
  m.hidden_out = hidden;
  m.logits.assign((size_t)n * V, 0.f);
  gemm(hidden.data(), n, m.get("talker.codec_head.weight")->v.data(), V, h, m.logits.data(), V, 0, g_round_logits);
  for (int s = 0; s < n; ++s) {
    Session& S = m.sessions[sids[s]];
    codes[s * 16 + 0] = sample_group(m, S, &m.logits[(size_t)s * V], 0,
                                     session_uniform(m, S, uniforms, s, 0, S.frames), force[s * 16 + 0], S.frames);
  }
  m.p_logits.assign((size_t)(G - 1) * n * PV, 0.f);
  std::vector<Kv> pkv(n);
  for (auto& k : pkv) k.init(c.predictor.layers, 2 * c.predictor.kv_heads * c.predictor.head_dim, G);
  const Tensor* codec_emb = m.get("talker.model.codec_embedding.weight");
  const Tensor* mtp_w = m.get("talker.code_predictor.small_to_mtp_projection.weight");
  const Tensor* mtp_b = m.get("talker.code_predictor.small_to_mtp_projection.bias");
  std::vector<float> last((size_t)n * p);
  for (int g = 1; g < G; ++g) {
    const int per = g == 1 ? 2 : 1, rows = n * per;
    std::vector<float> in((size_t)rows * h), ph((size_t)rows * p);
    std::vector<Row> rr(rows);
    for (int s = 0; s < n; ++s) {
      if (g == 1) {  // `talker_pred_input`, talker.cu:100-106
        memcpy(&in[(size_t)(2 * s) * h], &hidden[(size_t)s * h], h * sizeof(float));
        std::vector<float> e = row_of(codec_emb, codes[s * 16]);
        memcpy(&in[(size_t)(2 * s + 1) * h], e.data(), h * sizeof(float));
        rr[2 * s] = Row{&pkv[s], 0};
        rr[2 * s + 1] = Row{&pkv[s], 1};
      } else {  // `talker_gather` over table g-2 of the stacked predictor embeddings, talker.rs:328-342
        const Tensor* tab =
            m.get("talker.code_predictor.model.codec_embedding." + std::to_string(g - 2) + ".weight");
        std::vector<float> e = row_of(tab, codes[s * 16 + g - 1]);
        memcpy(&in[(size_t)s * h], e.data(), h * sizeof(float));
        rr[s] = Row{&pkv[s], g};
      }
    }
    gemm(in.data(), rows, mtp_w->v.data(), p, h, ph.data(), p);
    bias_act(ph.data(), mtp_b->v.data(), rows, p, false);
    stack_forward(m.pred, ph.data(), rr, last.data(), per, per - 1);
    const Tensor* head = m.get("talker.code_predictor.lm_head." + std::to_string(g - 1) + ".weight");
    float* lg = &m.p_logits[(size_t)(g - 1) * n * PV];
    gemm(last.data(), n, head->v.data(), PV, p, lg, PV, 0, g_round_logits);
    for (int s = 0; s < n; ++s) {
      Session& S = m.sessions[sids[s]];
      codes[s * 16 + g] = sample_group(m, S, lg + (size_t)s * PV, g, session_uniform(m, S, uniforms, s, g, S.frames),
                                       force[s * 16 + g], S.frames);
    }
  }
  for (int s = 0; s < n; ++s)
    for (int g = G; g < 16; ++g) codes[s * 16 + g] = 0;
}

}  // namespace

extern "C" {

void* orc_create(const orc_config* cfg, const orc_tensor* tensors, int n) {
  auto m = std::make_unique<Model>();
  m->cfg = *cfg;
  for (int i = 0; i < n; ++i) {
    const orc_tensor& src = tensors[i];
    if (src.location != 0) return nullptr;
    Tensor t;
    int64_t count = 1;
    for (int d = 0; d < src.ndim; ++d) {
      t.shape.push_back(src.shape[d]);
      count *= src.shape[d];
    }
    t.v.resize(count);
    if (src.dtype == 0)
      memcpy(t.v.data(), src.data, count * 2);
    else
      for (int64_t e = 0; e < count; ++e) t.v[e] = f2bf(((const float*)src.data)[e]);
    m->t.emplace(src.name, std::move(t));
  }
  if (!bind_stack(*m, m->talker, cfg->talker, "talker.model")) return nullptr;
  if (!bind_stack(*m, m->pred, cfg->predictor, "talker.code_predictor.model")) return nullptr;
  init_pad(*m);
  return m.release();
}

void orc_destroy(void* h) { delete (Model*)h; }

void orc_round_logits(int on) { g_round_logits = on != 0; }

void orc_set_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int orc_max_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// `Model::open` (crates/omni-qwen3-tts/src/model.rs:135-146): a sequence of a
// `prompt`-token prompt and up to `frames` frames; its state slot starts zeroed.
int orc_open(void* h, int prompt, int frames, uint64_t seed) {
  Model& m = *(Model*)h;
  int id = -1;
  for (size_t i = 0; i < m.sessions.size(); ++i)
    if (!m.sessions[i].live) id = (int)i;
  if (id < 0) {
    m.sessions.emplace_back();
    id = (int)m.sessions.size() - 1;
  }
  Session& s = m.sessions[id];
  s = Session();
  s.live = true;
  s.prompt = prompt;
  s.cap = prompt + frames;
  s.seed = seed;
  s.kv.init(m.cfg.talker.layers, 2 * m.cfg.talker.kv_heads * m.cfg.talker.head_dim, s.cap);
  memset(s.st.last_frame, 0, sizeof(s.st.last_frame));
  s.st.seen.assign((m.cfg.talker.vocab + 31) / 32, 0u);
  s.hidden.assign(m.cfg.talker.hidden, 0.f);
  return id;
}

void orc_close(void* h, int sid) { ((Model*)h)->sessions[sid] = Session(); }

// `Model::start` (model.rs:153-177) = `Talker::prefill` (talker.rs:186-221)
// then the `first` program (the tail on the prompt's last hidden state).
int orc_start(void* h, int n, const int32_t* sids, const int32_t* text_ids, const int32_t* codec_ids,
              const int32_t* prompt_lens, const float* uniforms, const int32_t* force, int32_t* codes) {
  Model& m = *(Model*)h;
  const int hd = m.cfg.talker.hidden;
  int tokens = 0;
  for (int s = 0; s < n; ++s) tokens += prompt_lens[s];
  const Tensor* text_emb = m.get("talker.model.text_embedding.weight");
  const Tensor* codec_emb = m.get("talker.model.codec_embedding.weight");
  std::vector<float> e((size_t)tokens * hd), p((size_t)tokens * hd);
  for (int r = 0; r < tokens; ++r) {
    if (text_ids[r] < 0 || text_ids[r] >= text_emb->rows()) return 1;
    std::vector<float> row = row_of(text_emb, text_ids[r]);
    memcpy(&e[(size_t)r * hd], row.data(), hd * sizeof(float));
  }
  gemm(e.data(), tokens, m.get("talker.text_projection.linear_fc1.weight")->v.data(), hd, hd, p.data(), hd);
  bias_act(p.data(), m.get("talker.text_projection.linear_fc1.bias")->v.data(), tokens, hd, true);
  m.embeds.assign((size_t)tokens * hd, 0.f);
  gemm(p.data(), tokens, m.get("talker.text_projection.linear_fc2.weight")->v.data(), hd, hd, m.embeds.data(), hd);
  // `talker_prompt_codec` (talker.cu:55-71): x + bias (+ codec embedding), one rounding
  const bf16_t* b2 = m.get("talker.text_projection.linear_fc2.bias")->v.data();
  for (int r = 0; r < tokens; ++r)
    for (int c = 0; c < hd; ++c) {
      float v = m.embeds[(size_t)r * hd + c] + bf2f(b2[c]);
      if (codec_ids[r] >= 0) v += bf2f(codec_emb->v[(size_t)codec_ids[r] * hd + c]);
      m.embeds[(size_t)r * hd + c] = rbf(v);
    }
  std::vector<Row> rows;
  std::vector<int> last_row, ids;
  for (int s = 0; s < n; ++s) {
    Session& S = m.sessions[sids[s]];
    if (!S.live || S.frames != 0 || S.prompt != prompt_lens[s]) return 2;
    for (int t = 0; t < prompt_lens[s]; ++t) rows.push_back(Row{&S.kv, t});
    last_row.push_back((int)rows.size() - 1);
    ids.push_back(sids[s]);
  }
  std::vector<float> out((size_t)tokens * hd);
  stack_forward(m.talker, m.embeds.data(), rows, out.data(), 1, 0);
  for (int s = 0; s < n; ++s)
    memcpy(m.sessions[sids[s]].hidden.data(), &out[(size_t)last_row[s] * hd], hd * sizeof(float));
  tail(m, ids, uniforms, force, codes);
  for (int s = 0; s < n; ++s) m.sessions[sids[s]].frames = 1;
  return 0;
}

// `Model::step` (model.rs:180-192) = `Talker::advance` (talker.rs:224-251) then
// the tail. The talker row of a sequence sits at position prompt + frames - 1;
// the sampler sees the frame index.
int orc_step(void* h, int n, const int32_t* sids, const float* uniforms, const int32_t* force, int32_t* codes) {
  Model& m = *(Model*)h;
  const orc_config& c = m.cfg;
  const int hd = c.talker.hidden, PV = c.predictor.vocab;
  std::vector<float> in((size_t)n * hd);
  std::vector<Row> rows(n);
  std::vector<int> ids;
  const Tensor* codec_emb = m.get("talker.model.codec_embedding.weight");
  for (int s = 0; s < n; ++s) {
    Session& S = m.sessions[sids[s]];
    if (!S.live || S.frames == 0) return 2;
    if (S.prompt + S.frames - 1 >= S.cap) return 3;
    // `talker_frame_embed` (talker.cu:76-96): pad + codebook-0 embedding + the
    // predictor tables' embeddings of codes 1.., f32 sum, one rounding
    std::vector<const Tensor*> tabs(c.groups, nullptr);
    for (int g = 1; g < c.groups; ++g)
      tabs[g] = m.get("talker.code_predictor.model.codec_embedding." + std::to_string(g - 1) + ".weight");
    for (int col = 0; col < hd; ++col) {
      float acc = 0.f;
      acc += m.pad_embed[col];
      acc += bf2f(codec_emb->v[(size_t)S.st.last_frame[0] * hd + col]);
      for (int g = 1; g < c.groups; ++g) acc += bf2f(tabs[g]->v[(size_t)S.st.last_frame[g] * hd + col]);
      in[(size_t)s * hd + col] = rbf(acc);
    }
    rows[s] = Row{&S.kv, S.prompt + S.frames - 1};
    ids.push_back(sids[s]);
  }
  (void)PV;
  std::vector<float> out((size_t)n * hd);
  stack_forward(m.talker, in.data(), rows, out.data(), 1, 0);
  for (int s = 0; s < n; ++s) memcpy(m.sessions[sids[s]].hidden.data(), &out[(size_t)s * hd], hd * sizeof(float));
  tail(m, ids, uniforms, force, codes);
  for (int s = 0; s < n; ++s) m.sessions[sids[s]].frames += 1;
  return 0;
}

// Debug reads of the last call, rows indexed by the call's sequence order.
int orc_read(void* h, int what, int s, float* dst, int64_t count) {
  Model& m = *(Model*)h;
  const orc_config& c = m.cfg;
  switch (what) {
    case 0:  // codebook-0 logits [vocab]
      if (count != c.talker.vocab) return 1;
      memcpy(dst, &m.logits[(size_t)s * c.talker.vocab], count * 4);
      return 0;
    case 1: {  // predictor logits [groups-1, p_vocab]
      const int PV = c.predictor.vocab;
      if (count != (int64_t)(c.groups - 1) * PV) return 1;
      for (int g = 0; g < c.groups - 1; ++g)
        memcpy(dst + (size_t)g * PV, &m.p_logits[((size_t)g * m.last_n + s) * PV], PV * 4);
      return 0;
    }
    case 2:  // prompt embeddings, `count` leading values
      if (count > (int64_t)m.embeds.size()) return 1;
      memcpy(dst, m.embeds.data(), count * 4);
      return 0;
    case 3:  // talker hidden state of row s
      if (count != c.talker.hidden) return 1;
      memcpy(dst, &m.hidden_out[(size_t)s * c.talker.hidden], count * 4);
      return 0;
    case 4:  // pad embedding
      if (count != c.talker.hidden) return 1;
      memcpy(dst, m.pad_embed.data(), count * 4);
      return 0;
  }
  return 1;
}

// Operator-level entry points for kernel parity tests.

void orc_gemm(const float* x, int rows, const uint16_t* w, int n, int k, float* y) { gemm(x, rows, w, n, k, y, n); }

void orc_add_norm(const float* x, float* res, const uint16_t* w, float* out, int rows, int dim, float eps, int every,
                  int which) {
  add_norm(x, res, w, out, rows, dim, eps, every, which);
}

void orc_norm_copy(const float* x, const uint16_t* w, float* out, float* res, int rows, int dim, float eps) {
  norm_copy(x, w, out, res, rows, dim, eps);
}

void orc_silu_mul(const float* gate_up, float* act, int rows, int inter) { silu_mul(gate_up, act, rows, inter); }

void orc_rope_head(float* head, const uint16_t* w, int d, int pos, float eps, float theta) {
  rope_head(head, w, d, pos, eps, theta);
}

// Attention of one row over a dense K/V [len][2*hk*d] (bf16 bits).
void orc_attend(const float* q, const uint16_t* kv, int len, int hq, int hk, int d, float* out) {
  Kv k;
  k.init(1, 2 * hk * d, len);
  memcpy(k.data[0].data(), kv, (size_t)len * 2 * hk * d * 2);
  attend_row(q, k, 0, len, hq, hk, d, 1.f / sqrtf((float)d), out);
}

// One sampler row on explicit state: `last_frame` [16] and `seen` bitmap are
// updated in place exactly as the slot would be.
int orc_sample(const float* logits, int vocab, float temperature, int top_k, float top_p, float penalty,
               int suppress_lo, int suppress_hi, int exempt, int min_frames, int frame, float u, int forced,
               int32_t* last_frame, uint32_t* seen, int penalize, int group) {
  SeqState st;
  memcpy(st.last_frame, last_frame, sizeof(st.last_frame));
  st.seen.assign(seen, seen + (vocab + 31) / 32);
  const int tok = sample_row(logits, vocab, temperature, top_k, top_p, penalty, suppress_lo, suppress_hi, exempt,
                             min_frames, frame, u, forced, st, penalize != 0, group);
  memcpy(last_frame, st.last_frame, sizeof(st.last_frame));
  memcpy(seen, st.seen.data(), st.seen.size() * 4);
  return tok;
}

float orc_philox_uniform(uint64_t seed, uint32_t frame, uint32_t group) { return philox_uniform(seed, frame, group); }

uint16_t orc_f2bf(float f) { return f2bf(f); }

}  // extern "C"
