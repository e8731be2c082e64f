// The Higgs-style speech model shell behind include/omni_b200_higgs.h: weights, the paged-KV lease pool, input staging
// and the op order of prefill, first draw and decode step. The op order is the one the reference's manifest emits
// (crates/omni-higgs-audio/src/model.rs:339-405 around `Stack::forward`, crates/omni-qwen3/src/stack.rs:152-203);
// GEMMs run on gemm.h, the stack's other ops on kernels.h, the glue on higgs_kernels.cu.
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

#include "../../include/omni_b200_higgs.h"
#include "../../include/omni_b200_ops.h"
#include "gemm.h"
#include "kernels.h"

using namespace omni;

struct omni_higgs_seq {
  std::vector<int32_t> pages;
  int32_t line = -1;
  int32_t prompt = 0, rows = 0, cap = 0;
  omni_higgs_delay delay{0, 0, 0};
  bool live = false;
};

namespace {

struct Layer {
  bf16 *ln1, *qkv, *q_norm, *k_norm, *o, *ln2, *gate_up, *down;
  // with the audio-FFN adapter: the MLP of an audio position, text and audio branch fused along the channel axis:
  // [gate_text; gate_audio; up_text; up_audio] (4I x h) and [down_text | down_audio] (h x 2I)
  bf16 *gate_up_audio = nullptr, *down_audio = nullptr;
};

uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

}  // namespace

struct omni_higgs {
  omni_higgs_config cfg;
  int device = 0, sm_count = 148;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::string error;
  std::vector<void*> allocations;
  int launches = 0, last_launches = 0;
  float last_ms = 0.f;

  std::vector<Layer> layers;
  bf16 *norm = nullptr, *text_emb = nullptr, *fused = nullptr;

  int pages_total = 0, page_table = 0;
  std::vector<bf16*> kv;  // per layer: [page][kv_head][K | V][16][head_dim]
  std::vector<int32_t> free_pages, free_lines;
  char* state = nullptr;
  int64_t stride = 256;
  std::vector<std::unique_ptr<omni_higgs_seq>> seqs;

  int max_rows = 0;
  bf16 *embeds = nullptr, *x = nullptr, *res = nullptr, *qkv = nullptr, *attn = nullptr, *gate_up = nullptr,
       *act = nullptr, *hidden = nullptr, *logits = nullptr;
  int32_t* codes = nullptr;

  char *in_host = nullptr, *in_dev = nullptr;
  size_t in_bytes = 0;
  int32_t* out_host = nullptr;
  uint32_t* err = nullptr;
  GemmScratch scratch;
  std::map<std::tuple<const void*, const void*, const void*, int>, TcGemmPlan> plans;
  std::map<std::tuple<const void*, const void*, const void*, int>, RmGemmPlan> rm_plans;
  // the padding lease: one page and one state line for the rows between the live sequences and the step's bucket
  int pad_page = 0, pad_line = 0;
  // one CUDA graph of the decode step's kernels per bucket (sequence counts are padded up to 1, 2, 4, ... or max_batch)
  struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    int seen = 0, nodes = 0;
  };
  std::map<int, StepGraph> step_graphs;
  bool use_graphs = true;

  int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    error = buf;
    return code;
  }
  int qkv_width() const { return (cfg.body.q_heads + 2 * cfg.body.kv_heads) * cfg.body.head_dim; }
};

#define HCUDA(m, expr)                                                                              \
  do {                                                                                              \
    cudaError_t e_ = (expr);                                                                        \
    if (e_ != cudaSuccess) return (m)->fail(OMNI_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)
#define HLAUNCH(m, expr) \
  do {                   \
    HCUDA(m, expr);      \
    ++(m)->launches;     \
  } while (0)
#define HTRY(expr)                  \
  do {                              \
    const int rc_ = (expr);         \
    if (rc_ != OMNI_OK) return rc_; \
  } while (0)

namespace {

template <typename T>
int halloc(omni_higgs* m, T** out, size_t count, bool zero = false) {
  void* p = nullptr;
  HCUDA(m, cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T)));
  if (zero) HCUDA(m, cudaMemset(p, 0, std::max<size_t>(count, 1) * sizeof(T)));
  m->allocations.push_back(p);
  *out = static_cast<T*>(p);
  return OMNI_OK;
}

__global__ void higgs_f32_to_bf16(const float* __restrict__ src, bf16* __restrict__ dst, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2bfloat16(src[i]);
}

using Index = std::unordered_map<std::string, const omni_tensor*>;

// Copies one checkpoint tensor (rounded to bf16) to `dst`; the shape must match.
int upload(omni_higgs* m, const Index& idx, const std::string& name, std::initializer_list<int64_t> shape, bf16* dst) {
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
  if (t->location == OMNI_DEVICE) {
    if (t->dtype == OMNI_BF16) {
      HCUDA(m, cudaMemcpy(dst, t->data, count * 2, cudaMemcpyDeviceToDevice));
    } else {
      higgs_f32_to_bf16<<<(unsigned)((count + 255) / 256), 256>>>((const float*)t->data, dst, count);
      HCUDA(m, cudaGetLastError());
      HCUDA(m, cudaDeviceSynchronize());
    }
  } else if (t->dtype == OMNI_BF16) {
    HCUDA(m, cudaMemcpy(dst, t->data, count * 2, cudaMemcpyHostToDevice));
  } else {
    std::vector<uint16_t> tmp((size_t)count);
    const float* src = (const float*)t->data;
    for (int64_t i = 0; i < count; ++i) tmp[i] = f2bf(src[i]);
    HCUDA(m, cudaMemcpy(dst, tmp.data(), count * 2, cudaMemcpyHostToDevice));
  }
  return OMNI_OK;
}

int gemm(omni_higgs* m, const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy) {
  if (rows <= 8 || !tc_supports(N, K, rows)) {
    HLAUNCH(m, gemv_launch(w, N, K, x, rows, y, ldy, Epilogue{}, m->sm_count, m->stream));
    return OMNI_OK;
  }
  const auto key = std::make_tuple((const void*)w, (const void*)x, (const void*)y, rows);
  if (rm_supports(N, K, rows)) {  // decode-sized: input rows on the MMA M dimension, no split and no reduction
    auto rt = m->rm_plans.find(key);
    if (rt == m->rm_plans.end()) {
      RmGemmPlan plan;
      const int rc = rm_plan(&plan, w, N, K, x, rows, y, ldy, Epilogue{}, m->sm_count);
      if (rc != 0) return m->fail(OMNI_ERR_CUDA, "tensor-map encode failed (%d) for N=%d K=%d rows=%d", rc, N, K, rows);
      rt = m->rm_plans.emplace(key, plan).first;
    }
    HLAUNCH(m, rm_launch(rt->second, m->err, m->stream));
    return OMNI_OK;
  }
  auto it = m->plans.find(key);
  if (it == m->plans.end()) {
    TcGemmPlan plan;
    const int rc = tc_plan(&plan, w, N, K, x, rows, y, ldy, Epilogue{}, m->sm_count);
    if (rc != 0) return m->fail(OMNI_ERR_CUDA, "tensor-map encode failed (%d) for N=%d K=%d rows=%d", rc, N, K, rows);
    if (plan.partial_floats() > m->scratch.partial_floats || plan.tiles_n() * plan.row_tiles > m->scratch.counter_slots)
      return m->fail(OMNI_ERR_UNSUPPORTED, "split-K scratch too small for N=%d K=%d rows=%d", N, K, rows);
    it = m->plans.emplace(key, plan).first;
  }
  HLAUNCH(m, tc_launch(it->second, m->scratch, m->err, m->stream));
  return OMNI_OK;
}

// One pass of the body over `rows` rows of `input`: `Stack::forward` (stack.rs:152-203); the final norm's rows go to out.
// `audio`: every row is an audio position. With the audio-FFN adapter such a row's MLP is the text branch and the audio
// branch side by side — one gate|up GEMM over both branches' channels, SwiGLU, one down GEMM whose K runs over both
// branches' activations, so the two branches' outputs are summed in f32 before the one bf16 rounding.
int body_forward(omni_higgs* m, const bf16* input, int rows, const RowMap& map, bf16* out, bool audio) {
  const omni_stack_config& c = m->cfg.body;
  const bool both = audio && m->cfg.audio_adapter != 0;
  const int h = c.hidden, I = both ? 2 * c.inter : c.inter, qd = c.q_heads * c.head_dim, qw = m->qkv_width();
  const AttnShape a{c.q_heads, c.kv_heads, c.head_dim, c.rms_eps, c.rope_theta};
  HLAUNCH(m, launch_norm_copy(input, m->layers[0].ln1, m->x, m->res, rows, h, c.rms_eps, m->stream));
  for (int i = 0; i < c.layers; ++i) {
    const Layer& L = m->layers[i];
    HTRY(gemm(m, L.qkv, qw, h, m->x, rows, m->qkv, qw));
    HLAUNCH(m, launch_rope_kv(m->qkv, L.q_norm, L.k_norm, m->kv[i], map, rows, a, m->pages_total, m->err, m->stream));
    HLAUNCH(m, launch_attend(m->qkv, m->kv[i], m->attn, map, rows, a, m->err, m->stream));
    HTRY(gemm(m, L.o, h, qd, m->attn, rows, m->x, h));
    HLAUNCH(m, launch_add_norm(m->x, m->res, L.ln2, m->x, rows, h, c.rms_eps, 1, 0, m->stream));
    HTRY(gemm(m, both ? L.gate_up_audio : L.gate_up, 2 * I, h, m->x, rows, m->gate_up, 2 * I));
    HLAUNCH(m, launch_silu_mul(m->gate_up, m->act, rows, I, 0, m->stream));
    HTRY(gemm(m, both ? L.down_audio : L.down, h, I, m->act, rows, m->x, h));
    const bf16* next = i + 1 < c.layers ? m->layers[i + 1].ln1 : m->norm;
    HLAUNCH(m, launch_add_norm(m->x, m->res, next, i + 1 < c.layers ? m->x : out, rows, h, c.rms_eps, 1, 0, m->stream));
  }
  return OMNI_OK;
}

struct Staging {
  omni_higgs* m;
  size_t used = 0;
  template <typename T>
  T* take(size_t count) {
    T* p = reinterpret_cast<T*>(m->in_host + used);
    used += (count * sizeof(T) + 255) & ~(size_t)255;
    return used <= m->in_bytes ? p : nullptr;
  }
  template <typename T>
  const T* dev(const T* host) const {
    return reinterpret_cast<const T*>(m->in_dev + (reinterpret_cast<const char*>(host) - m->in_host));
  }
};

// The `force` row of a step (`step`, model.rs:262-265): the draw's own, else the delay pattern's ramp.
void force_row(const omni_higgs_seq* s, const omni_higgs_draw& d, int32_t* out) {
  const int from = omni_higgs_delay_forced_from(&s->delay);
  for (int b = 0; b < OMNI_HIGGS_CODEBOOKS; ++b) out[b] = d.has_force ? d.force[b] : (b >= from ? OMNI_HIGGS_BOC : -1);
}

// head GEMM + the eight draws (`first` / the tail of `decode`, model.rs:381-404)
int tail_kernels(omni_higgs* m, int n, const float* uniforms_dev, const int32_t* force_dev, const int32_t* lines_dev) {
  const omni_higgs_config& c = m->cfg;
  const int head = OMNI_HIGGS_CODEBOOKS * c.code_vocab;
  HTRY(gemm(m, m->fused, head, c.body.hidden, m->hidden, n, m->logits, head));
  HLAUNCH(m, launch_higgs_sample(m->logits, c.code_vocab, c.temperature, c.top_k, uniforms_dev, force_dev,
                                 SlotState{m->state, lines_dev, m->stride}, m->codes, n, m->stream));
  return OMNI_OK;
}

// The tail's kernels (unless a replayed graph already ran them) + read-back (`run`, model.rs:226-240; `finish`, :267-272)
int tail(omni_higgs* m, int n, omni_higgs_seq* const* seqs, const float* uniforms_dev, const int32_t* force_dev,
         const int32_t* lines_dev, int32_t* rows_out, int32_t* ended_out, bool kernels_done = false) {
  if (!kernels_done) HTRY(tail_kernels(m, n, uniforms_dev, force_dev, lines_dev));
  const size_t ints = (size_t)n * OMNI_HIGGS_CODEBOOKS;
  HCUDA(m, cudaMemcpyAsync(m->out_host, m->codes, ints * 4, cudaMemcpyDeviceToHost, m->stream));
  HCUDA(m, cudaMemcpyAsync(m->out_host + ints, m->err, 4, cudaMemcpyDeviceToHost, m->stream));
  HCUDA(m, cudaEventRecord(m->ev1, m->stream));
  HCUDA(m, cudaStreamSynchronize(m->stream));
  cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1);
  m->last_launches = m->launches;
  const uint32_t word = (uint32_t)m->out_host[ints];
  if (word != 0) {
    cudaMemsetAsync(m->err, 0, 4, m->stream);
    cudaStreamSynchronize(m->stream);
    return m->fail(OMNI_ERR_DEVICE, "device error word 0x%x (1: barrier wait ran out, 2: index out of range)", word);
  }
  memcpy(rows_out, m->out_host, ints * 4);
  for (int s = 0; s < n; ++s) {
    seqs[s]->rows += 1;
    const int ended = omni_higgs_delay_advance(&seqs[s]->delay, rows_out[s * OMNI_HIGGS_CODEBOOKS]);
    if (ended_out) ended_out[s] = ended;
  }
  return OMNI_OK;
}

int check_rows(omni_higgs* m, int n, omni_higgs_seq* const* seqs, const omni_higgs_draw* draws) {
  if (n < 1 || n > m->cfg.max_batch) return m->fail(OMNI_ERR_INVALID, "%d sequences in one call", n);
  for (int i = 0; i < n; ++i) {
    if (!seqs[i] || !seqs[i]->live) return m->fail(OMNI_ERR_INVALID, "sequence %d is not open", i);
    for (int j = 0; j < i; ++j)
      if (seqs[j] == seqs[i]) return m->fail(OMNI_ERR_INVALID, "sequence %d appears twice", i);
    if (draws[i].has_force)
      for (int b = 0; b < OMNI_HIGGS_CODEBOOKS; ++b)
        if (draws[i].force[b] >= m->cfg.code_vocab) return m->fail(OMNI_ERR_INVALID, "forced code outside the codebook");
  }
  return OMNI_OK;
}

}  // namespace

extern "C" {

int32_t omni_higgs_create(const omni_higgs_config* config, const omni_tensor* tensors, int32_t n_tensors, int32_t device,
                          omni_higgs** out) {
  if (!config || !out || (!tensors && n_tensors > 0)) return OMNI_ERR_INVALID;
  omni_higgs* m = new omni_higgs();
  *out = m;
  m->cfg = *config;
  m->device = device;
  const omni_higgs_config& c = m->cfg;
  const omni_stack_config& b = c.body;
  const bool shape_ok = b.hidden % 64 == 0 && b.hidden >= 256 && b.hidden / 8 <= 1024 && b.inter % 64 == 0 &&
                        (b.head_dim == 64 || b.head_dim == 128) && b.kv_heads >= 1 && b.q_heads % b.kv_heads == 0 &&
                        b.layers >= 1 && b.vocab >= 1 && c.code_vocab >= 2 && c.code_vocab <= 4096 && c.max_batch >= 1 &&
                        c.max_tokens >= 1 && c.kv_gib > 0;
  const int g = b.kv_heads > 0 ? b.q_heads / b.kv_heads : 0;
  if (!shape_ok || !(g == 1 || g == 2 || g == 4 || g == 5 || g == 8))
    return m->fail(OMNI_ERR_INVALID, "higgs config outside the supported shapes");
  HCUDA(m, cudaSetDevice(device));
  cudaDeviceProp prop;
  HCUDA(m, cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return m->fail(OMNI_ERR_UNSUPPORTED, "device is sm_%d%d; this library is sm_100a only", prop.major, prop.minor);
  m->sm_count = prop.multiProcessorCount;
  m->use_graphs = c.use_graphs != 0;
  HCUDA(m, cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
  HCUDA(m, cudaEventCreate(&m->ev0));
  HCUDA(m, cudaEventCreate(&m->ev1));
  if (tc_init() != 0) return m->fail(OMNI_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  tc_configure();

  Index idx;
  for (int i = 0; i < n_tensors; ++i)
    if (tensors[i].name) idx[tensors[i].name] = &tensors[i];
  const int64_t h = b.hidden, d = b.head_dim, q = (int64_t)b.q_heads * d, kvw = (int64_t)b.kv_heads * d, I = b.inter;
  m->layers.resize(b.layers);
  bf16* adapter_tmp = nullptr;  // staging for the audio branch's down projection (stays allocated with the model)
  for (int i = 0; i < b.layers; ++i) {  // `Stack::load` (stack.rs:93-141): Q|K|V rows and gate|up rows fused
    const std::string p = "body.layers." + std::to_string(i) + ".";
    Layer& L = m->layers[i];
    HTRY(halloc(m, &L.ln1, h));
    HTRY(halloc(m, &L.qkv, (q + 2 * kvw) * h));
    HTRY(halloc(m, &L.q_norm, d));
    HTRY(halloc(m, &L.k_norm, d));
    HTRY(halloc(m, &L.o, h * q));
    HTRY(halloc(m, &L.ln2, h));
    HTRY(halloc(m, &L.gate_up, 2 * I * h));
    HTRY(halloc(m, &L.down, h * I));
    HTRY(upload(m, idx, p + "input_layernorm.weight", {h}, L.ln1));
    HTRY(upload(m, idx, p + "self_attn.q_proj.weight", {q, h}, L.qkv));
    HTRY(upload(m, idx, p + "self_attn.k_proj.weight", {kvw, h}, L.qkv + q * h));
    HTRY(upload(m, idx, p + "self_attn.v_proj.weight", {kvw, h}, L.qkv + (q + kvw) * h));
    HTRY(upload(m, idx, p + "self_attn.q_norm.weight", {d}, L.q_norm));
    HTRY(upload(m, idx, p + "self_attn.k_norm.weight", {d}, L.k_norm));
    HTRY(upload(m, idx, p + "self_attn.o_proj.weight", {h, q}, L.o));
    HTRY(upload(m, idx, p + "post_attention_layernorm.weight", {h}, L.ln2));
    HTRY(upload(m, idx, p + "mlp.gate_proj.weight", {I, h}, L.gate_up));
    HTRY(upload(m, idx, p + "mlp.up_proj.weight", {I, h}, L.gate_up + I * h));
    HTRY(upload(m, idx, p + "mlp.down_proj.weight", {h, I}, L.down));
    if (c.audio_adapter) {
      HTRY(halloc(m, &L.gate_up_audio, 4 * I * h));
      HTRY(halloc(m, &L.down_audio, h * 2 * I));
      HCUDA(m, cudaMemcpy(L.gate_up_audio, L.gate_up, I * h * 2, cudaMemcpyDeviceToDevice));
      HTRY(upload(m, idx, p + "audio_mlp.gate_proj.weight", {I, h}, L.gate_up_audio + I * h));
      HCUDA(m, cudaMemcpy(L.gate_up_audio + 2 * I * h, L.gate_up + I * h, I * h * 2, cudaMemcpyDeviceToDevice));
      HTRY(upload(m, idx, p + "audio_mlp.up_proj.weight", {I, h}, L.gate_up_audio + 3 * I * h));
      if (!adapter_tmp) HTRY(halloc(m, &adapter_tmp, h * I));
      HTRY(upload(m, idx, p + "audio_mlp.down_proj.weight", {h, I}, adapter_tmp));
      HCUDA(m, cudaMemcpy2D(L.down_audio, 2 * I * 2, L.down, I * 2, I * 2, h, cudaMemcpyDeviceToDevice));
      HCUDA(m, cudaMemcpy2D(L.down_audio + I, 2 * I * 2, adapter_tmp, I * 2, I * 2, h, cudaMemcpyDeviceToDevice));
    }
  }
  HTRY(halloc(m, &m->norm, h));
  HTRY(upload(m, idx, "body.norm.weight", {h}, m->norm));
  HTRY(halloc(m, &m->text_emb, (size_t)b.vocab * h));
  HTRY(upload(m, idx, "tied.embedding.text_embedding.weight", {b.vocab, h}, m->text_emb));
  const int64_t head = (int64_t)OMNI_HIGGS_CODEBOOKS * c.code_vocab;
  HTRY(halloc(m, &m->fused, (size_t)head * h));
  HTRY(upload(m, idx, "tied.embedding.modality_embeddings.0.embedding.weight", {head, h}, m->fused));

  // pools: pages of 16 tokens, bytes per token and layer = 2 * kv_heads * head_dim * 2 (`Stack::kv_bytes`)
  const double per_page = 16.0 * b.layers * 2.0 * kvw * 2.0;
  m->pages_total = std::max(2, (int)(c.kv_gib * 1073741824.0 / per_page));
  m->kv.resize(b.layers);
  for (int i = 0; i < b.layers; ++i) HTRY(halloc(m, &m->kv[i], (size_t)m->pages_total * 16 * 2 * kvw, true));
  for (int p = m->pages_total - 1; p >= 0; --p) m->free_pages.push_back(p);
  m->pad_page = m->free_pages.back();  // the padding lease keeps one page and the state line behind the sequences' lines
  m->free_pages.pop_back();
  m->pad_line = c.max_batch;
  HTRY(halloc(m, &m->state, (size_t)(c.max_batch + 1) * m->stride, true));
  for (int i = c.max_batch - 1; i >= 0; --i) m->free_lines.push_back(i);

  m->max_rows = std::max(c.max_tokens, c.max_batch);
  const size_t R = m->max_rows;
  HTRY(halloc(m, &m->embeds, R * h));
  HTRY(halloc(m, &m->x, R * h));
  HTRY(halloc(m, &m->res, R * h));
  HTRY(halloc(m, &m->qkv, R * (q + 2 * kvw)));
  HTRY(halloc(m, &m->attn, R * q));
  const size_t Iw = c.audio_adapter ? 2 * I : I;  // widest MLP a row goes through
  HTRY(halloc(m, &m->gate_up, R * 2 * Iw));
  HTRY(halloc(m, &m->act, R * Iw));
  HTRY(halloc(m, &m->hidden, (size_t)c.max_batch * h, true));
  HTRY(halloc(m, &m->logits, (size_t)c.max_batch * head, true));
  HTRY(halloc(m, &m->codes, (size_t)c.max_batch * OMNI_HIGGS_CODEBOOKS, true));
  HTRY(halloc(m, &m->err, 64, true));
  m->page_table = m->pages_total;
  m->in_bytes = (R * 5 + (size_t)c.max_batch * 24 + (size_t)m->page_table + 64 * 64) * 4;
  HCUDA(m, cudaMallocHost((void**)&m->in_host, m->in_bytes));
  HTRY(halloc(m, &m->in_dev, m->in_bytes));
  HCUDA(m, cudaMallocHost((void**)&m->out_host, ((size_t)c.max_batch * OMNI_HIGGS_CODEBOOKS + 1) * 4));
  m->scratch.partial_floats = (size_t)32 << 20;
  m->scratch.counter_slots = 1 << 16;
  HTRY(halloc(m, &m->scratch.partials, m->scratch.partial_floats));
  HTRY(halloc(m, &m->scratch.counters, (size_t)m->scratch.counter_slots, true));
  return OMNI_OK;
}

void omni_higgs_destroy(omni_higgs* m) {
  if (!m) return;
  cudaSetDevice(m->device);
  if (m->stream) cudaStreamSynchronize(m->stream);
  for (auto& g : m->step_graphs)
    if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
  for (void* p : m->allocations) cudaFree(p);
  if (m->in_host) cudaFreeHost(m->in_host);
  if (m->out_host) cudaFreeHost(m->out_host);
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

const char* omni_higgs_last_error(const omni_higgs* m) { return m ? m->error.c_str() : "null model"; }

int32_t omni_higgs_open(omni_higgs* m, int32_t prompt, int32_t rows, omni_higgs_seq** out) {
  if (!m || !out || prompt < 1 || rows < 1) return OMNI_ERR_INVALID;
  *out = nullptr;
  const int need = (prompt + rows + 15) / 16;
  if (need > m->pages_total - 1) return OMNI_DENIED_EXCEEDS_POOL;  // (one page belongs to the padding lease)
  if (need > (int)m->free_pages.size() || m->free_lines.empty()) return OMNI_DENIED_BUSY;
  auto s = std::make_unique<omni_higgs_seq>();
  for (int i = 0; i < need; ++i) {
    s->pages.push_back(m->free_pages.back());
    m->free_pages.pop_back();
  }
  s->line = m->free_lines.back();
  m->free_lines.pop_back();
  s->prompt = prompt;
  s->cap = rows;
  s->live = true;
  cudaSetDevice(m->device);
  HCUDA(m, cudaMemsetAsync(m->state + (int64_t)s->line * m->stride, 0, m->stride, m->stream));
  *out = s.get();
  m->seqs.push_back(std::move(s));
  return OMNI_OK;
}

int32_t omni_higgs_close(omni_higgs* m, omni_higgs_seq* seq) {
  if (!m || !seq) return OMNI_ERR_INVALID;
  for (size_t i = 0; i < m->seqs.size(); ++i) {
    if (m->seqs[i].get() != seq) continue;
    for (int32_t p : seq->pages) m->free_pages.push_back(p);
    m->free_lines.push_back(seq->line);
    m->seqs.erase(m->seqs.begin() + i);
    return OMNI_OK;
  }
  return m->fail(OMNI_ERR_INVALID, "close of a sequence this model does not own");
}

int32_t omni_higgs_seq_rows(const omni_higgs_seq* seq) { return seq ? seq->rows : OMNI_ERR_INVALID; }

int32_t omni_higgs_start(omni_higgs* m, int32_t n, omni_higgs_seq* const* seqs, const int32_t* ids,
                         const int32_t* prompt_lens, const omni_higgs_draw* draws, int32_t* rows_out,
                         int32_t* ended_out) {
  if (!m || !seqs || !ids || !prompt_lens || !draws || !rows_out) return OMNI_ERR_INVALID;
  HTRY(check_rows(m, n, seqs, draws));
  const omni_higgs_config& c = m->cfg;
  int total = 0;
  for (int i = 0; i < n; ++i) {
    if (seqs[i]->rows != 0 || prompt_lens[i] != seqs[i]->prompt) return m->fail(OMNI_ERR_INVALID, "sequence %d is not fresh", i);
    total += prompt_lens[i];
  }
  if (total > c.max_tokens) return m->fail(OMNI_ERR_INVALID, "%d prompt tokens exceed %d", total, c.max_tokens);
  for (int r = 0; r < total; ++r)
    if (ids[r] < 0 || ids[r] >= c.body.vocab) return m->fail(OMNI_ERR_INVALID, "token id %d outside the vocabulary", ids[r]);
  HCUDA(m, cudaSetDevice(m->device));
  Staging st{m};
  int32_t *t_ids = st.take<int32_t>(total), *pos = st.take<int32_t>(total), *slot = st.take<int32_t>(total);
  int32_t *seq = st.take<int32_t>(total), *last = st.take<int32_t>(n), *indptr = st.take<int32_t>(n + 1);
  size_t page_count = 0;
  for (int i = 0; i < n; ++i) page_count += seqs[i]->pages.size();
  int32_t *pages = st.take<int32_t>(page_count), *lines = st.take<int32_t>(n);
  float* uniforms = st.take<float>((size_t)n * OMNI_HIGGS_CODEBOOKS);
  int32_t* force = st.take<int32_t>((size_t)n * OMNI_HIGGS_CODEBOOKS);
  if (!force) return m->fail(OMNI_ERR_INVALID, "staging block too small");
  memcpy(t_ids, ids, (size_t)total * 4);
  int r = 0;
  indptr[0] = 0;
  for (int i = 0; i < n; ++i) {
    const omni_higgs_seq* s = seqs[i];
    for (int p = 0; p < prompt_lens[i]; ++p, ++r) {
      pos[r] = p;
      slot[r] = s->pages[p >> 4] * 16 + (p & 15);
      seq[r] = i;
    }
    last[i] = r - 1;
    memcpy(pages + indptr[i], s->pages.data(), s->pages.size() * 4);
    indptr[i + 1] = indptr[i] + (int)s->pages.size();
    lines[i] = s->line;
    memcpy(uniforms + i * OMNI_HIGGS_CODEBOOKS, draws[i].uniforms, sizeof(draws[i].uniforms));
    force_row(s, draws[i], force + i * OMNI_HIGGS_CODEBOOKS);
  }
  m->launches = 0;
  HCUDA(m, cudaEventRecord(m->ev0, m->stream));
  HCUDA(m, cudaMemcpyAsync(m->in_dev, m->in_host, st.used, cudaMemcpyHostToDevice, m->stream));
  // `prefill` (model.rs:339-367): text embeddings, the body over every prompt row, each sequence's last row
  HLAUNCH(m, launch_gather(st.dev(t_ids), 1, m->text_emb, c.body.vocab, m->embeds, total, c.body.hidden, m->err, m->stream));
  RowMap map;
  map.pos = st.dev(pos);
  map.slot = st.dev(slot);
  map.seq = st.dev(seq);
  map.indptr = st.dev(indptr);
  map.pages = st.dev(pages);
  HTRY(body_forward(m, m->embeds, total, map, m->x, false));  // prompt rows are text positions
  HLAUNCH(m, launch_gather(st.dev(last), 1, m->x, total, m->hidden, n, c.body.hidden, m->err, m->stream));
  return tail(m, n, seqs, st.dev(uniforms), st.dev(force), st.dev(lines), rows_out, ended_out);
}

}  // extern "C"

namespace {

int step_bucket(const omni_higgs* m, int n) {  // `bucket` (crates/omni-kern/src/lib.rs:97-101), capped at max_batch
  int b = 1;
  while (b < n) b <<= 1;
  return std::min(b, m->cfg.max_batch);
}

// One decode step of n live sequences padded to bucket b (n = 0: the warm-up's step, every row on the padding lease).
int step_rows(omni_higgs* m, int n, int b, omni_higgs_seq* const* seqs, const omni_higgs_draw* draws, int32_t* rows_out,
              int32_t* ended_out) {
  const omni_higgs_config& c = m->cfg;
  HCUDA(m, cudaSetDevice(m->device));
  Staging st{m};
  // every array but the page list has a size b fixes, and the page list comes last: the device addresses the step's
  // kernels get depend on b alone, which is what lets the step be replayed as a CUDA graph
  int32_t *pos = st.take<int32_t>(b), *slot = st.take<int32_t>(b), *indptr = st.take<int32_t>(b + 1);
  int32_t* lines = st.take<int32_t>(b);
  float* uniforms = st.take<float>((size_t)b * OMNI_HIGGS_CODEBOOKS);
  int32_t* force = st.take<int32_t>((size_t)b * OMNI_HIGGS_CODEBOOKS);
  size_t page_count = (size_t)(b - n);
  for (int i = 0; i < n; ++i) page_count += seqs[i]->pages.size();
  int32_t* pages = st.take<int32_t>(page_count);
  if (!pages || !force) return m->fail(OMNI_ERR_INVALID, "staging block too small");
  indptr[0] = 0;
  for (int i = 0; i < n; ++i) {
    const omni_higgs_seq* s = seqs[i];
    const int p = s->prompt + s->rows - 1;  // model.rs:194
    pos[i] = p;
    slot[i] = s->pages[p >> 4] * 16 + (p & 15);
    memcpy(pages + indptr[i], s->pages.data(), s->pages.size() * 4);
    indptr[i + 1] = indptr[i] + (int)s->pages.size();
    lines[i] = s->line;
    memcpy(uniforms + i * OMNI_HIGGS_CODEBOOKS, draws[i].uniforms, sizeof(draws[i].uniforms));
    force_row(s, draws[i], force + i * OMNI_HIGGS_CODEBOOKS);
  }
  for (int i = n; i < b; ++i) {  // padding rows: position 0 of the padding lease, uniform 0.5, nothing forced
    pos[i] = 0;
    slot[i] = m->pad_page * 16;
    pages[indptr[i]] = m->pad_page;
    indptr[i + 1] = indptr[i] + 1;
    lines[i] = m->pad_line;
    for (int k = 0; k < OMNI_HIGGS_CODEBOOKS; ++k) uniforms[i * OMNI_HIGGS_CODEBOOKS + k] = 0.5f, force[i * OMNI_HIGGS_CODEBOOKS + k] = -1;
  }
  m->launches = 0;
  HCUDA(m, cudaEventRecord(m->ev0, m->stream));
  HCUDA(m, cudaMemcpyAsync(m->in_dev, m->in_host, st.used, cudaMemcpyHostToDevice, m->stream));
  // `decode` (model.rs:369-380): the last row's eight codes embedded, the body over one row per sequence, the head and
  // the draws. Captured once per bucket (the first step of a bucket runs eagerly and creates the GEMM plans;
  // omni_higgs_warmup does both for every bucket before live traffic).
  auto body = [&]() -> int {
    HLAUNCH(m, launch_higgs_frame_embed(SlotState{m->state, st.dev(lines), m->stride}, m->fused, m->embeds, b,
                                        c.body.hidden, c.code_vocab, m->err, m->stream));
    RowMap map;
    map.pos = st.dev(pos);
    map.slot = st.dev(slot);
    map.seq = nullptr;
    map.indptr = st.dev(indptr);
    map.pages = st.dev(pages);
    HTRY(body_forward(m, m->embeds, b, map, m->hidden, true));  // frame rows are audio positions
    return tail_kernels(m, b, st.dev(uniforms), st.dev(force), st.dev(lines));
  };
  omni_higgs::StepGraph& sg = m->step_graphs[b];
  if (!m->use_graphs || sg.seen == 0) {
    HTRY(body());
    sg.seen = 1;
  } else {
    if (!sg.exec) {
      HCUDA(m, cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
      const int rc = body();
      cudaGraph_t graph = nullptr;
      const cudaError_t end = cudaStreamEndCapture(m->stream, &graph);  // always ends the capture, also after a failure
      if (rc != OMNI_OK || end != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return rc != OMNI_OK ? rc : m->fail(OMNI_ERR_CUDA, "step capture: %s", cudaGetErrorString(end));
      }
      const cudaError_t inst = cudaGraphInstantiate(&sg.exec, graph, 0);
      cudaGraphDestroy(graph);
      if (inst != cudaSuccess) {
        sg.exec = nullptr;
        return m->fail(OMNI_ERR_CUDA, "step graph: %s", cudaGetErrorString(inst));
      }
      sg.nodes = m->launches;
    }
    HCUDA(m, cudaGraphLaunch(sg.exec, m->stream));
    m->launches = sg.nodes;
  }
  return tail(m, n, seqs, st.dev(uniforms), st.dev(force), st.dev(lines), rows_out, ended_out, true);
}

}  // namespace

extern "C" {

int32_t omni_higgs_step(omni_higgs* m, int32_t n, omni_higgs_seq* const* seqs, const omni_higgs_draw* draws,
                        int32_t* rows_out, int32_t* ended_out) {
  if (!m || !seqs || !draws || !rows_out) return OMNI_ERR_INVALID;
  HTRY(check_rows(m, n, seqs, draws));
  for (int i = 0; i < n; ++i) {
    if (seqs[i]->rows <= 0) return m->fail(OMNI_ERR_INVALID, "a sequence that has not started");
    if (seqs[i]->rows >= seqs[i]->cap) return m->fail(OMNI_ERR_INVALID, "sequence %d is past the rows it leased", i);
  }
  return step_rows(m, n, step_bucket(m, n), seqs, draws, rows_out, ended_out);
}

// Every bucket's decode step on the padding lease, twice (plans, then the captured graph), so that no live step pays
// for a graph capture: what `Model::warmup` does for the duplex model (crates/omni-personaplex/src/model.rs:202-240).
int32_t omni_higgs_warmup(omni_higgs* m) {
  if (!m) return OMNI_ERR_INVALID;
  std::vector<int> buckets;
  for (int b = 1; b < m->cfg.max_batch; b <<= 1) buckets.push_back(b);
  buckets.push_back(m->cfg.max_batch);
  int32_t none = 0;
  for (int b : buckets)
    for (int pass = 0; pass < (m->use_graphs ? 2 : 1); ++pass) HTRY(step_rows(m, 0, b, nullptr, nullptr, &none, nullptr));
  return OMNI_OK;
}

int32_t omni_higgs_read_logits(omni_higgs* m, int32_t s, void* dst, size_t bytes) {
  if (!m || !dst || s < 0 || s >= m->cfg.max_batch) return OMNI_ERR_INVALID;
  const size_t row = (size_t)OMNI_HIGGS_CODEBOOKS * m->cfg.code_vocab;
  if (bytes > row * 2) return m->fail(OMNI_ERR_INVALID, "read past the buffer");
  HCUDA(m, cudaSetDevice(m->device));
  HCUDA(m, cudaStreamSynchronize(m->stream));
  HCUDA(m, cudaMemcpy(dst, m->logits + (size_t)s * row, bytes, cudaMemcpyDeviceToHost));
  return OMNI_OK;
}

int32_t omni_higgs_stats(const omni_higgs* m, float* last_call_gpu_ms, int32_t* last_call_launches) {
  if (!m) return OMNI_ERR_INVALID;
  if (last_call_gpu_ms) *last_call_gpu_ms = m->last_ms;
  if (last_call_launches) *last_call_launches = m->last_launches;
  return OMNI_OK;
}

}  // extern "C"
