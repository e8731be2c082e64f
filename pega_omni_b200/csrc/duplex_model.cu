// The duplex (PersonaPlex) model shell behind include/omni_b200_duplex.h: weights, the ring-KV lease pool, input
// staging and the op order of one prefill and one tick. The op order is the one `Helium::step` / `Helium::forward`
// (crates/omni-personaplex/src/helium.rs:189-284) and `Depformer::step` (depformer.rs:137-259) emit; GEMMs run on this
// library's tensor-core / vector kernels (gemm.h), everything else on duplex_kernels.cu.
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

#include "../../include/omni_b200_duplex.h"
#include "duplex.h"
#include "gemm.h"
#include "kernels.h"

using namespace omni;

struct omni_duplex_session {
  std::vector<int32_t> pages;
  int32_t line = -1;
  int32_t pos = 0;
  int64_t frame = 0;
  int32_t first_force[OMNI_DUPLEX_DRAWN];
  bool live = false;
};

namespace {

constexpr int kCacheSlots = 8;     // PREFIX_CACHE_SLOTS (model.rs:68)
constexpr int kCacheMaxLen = 256;  // PREFIX_CACHE_MAX_LEN (model.rs:70)

struct HeliumLayer {
  bf16 *norm1, *qkv, *o, *norm2, *gate_up, *down;
};
struct DepLayer {
  bf16 *norm1, *qkv, *out, *norm2, *gate_in, *gate_out;
};

uint16_t host_f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

}  // namespace

struct omni_duplex {
  omni_duplex_config cfg;
  int device = 0, sm_count = 148;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::string error;
  std::vector<void*> allocations;
  int launches = 0, last_launches = 0;
  float last_ms = 0.f;

  // weights
  bf16 *text_emb = nullptr, *audio_emb = nullptr, *out_norm = nullptr, *text_linear = nullptr, *voices = nullptr;
  std::vector<HeliumLayer> h;
  bf16 *d_input = nullptr, *d_text_emb = nullptr, *d_emb = nullptr, *d_heads = nullptr;
  std::vector<DepLayer> d;

  // tensor-parallel pair (tp > 1): this rank holds heads / tp attention heads and hidden / tp MLP channels of Helium;
  // the depformer, the embeddings, the norms and the heads are replicated
  int tp = 1, tp_rank = 0;
  char* tp_region = nullptr;       // [256 B of words | exchange buffer 0 | exchange buffer 1]
  char* tp_peer_region = nullptr;  // the other rank's region, mapped by omni_duplex_tp_connect
  size_t tp_buf_bytes = 0;
  int local_heads() const { return cfg.heads / tp; }
  int local_hidden() const { return cfg.hidden / tp; }
  bf16* tp_buf(int which) const { return reinterpret_cast<bf16*>(tp_region + 256 + (size_t)which * tp_buf_bytes); }
  const bf16* tp_peer_buf(int which) const {
    return reinterpret_cast<const bf16*>(tp_peer_region + 256 + (size_t)which * tp_buf_bytes);
  }
  TpLink tp_link() const {
    TpLink l;
    l.my_flag = reinterpret_cast<uint32_t*>(tp_region);
    l.counter = reinterpret_cast<uint32_t*>(tp_region + 64);
    l.finished = reinterpret_cast<uint32_t*>(tp_region + 128);
    l.peer_flag = reinterpret_cast<uint32_t*>(tp_peer_region);
    return l;
  }

  // pools
  int pages_per_session = 0, kv_pages = 0;
  std::vector<uint8_t*> kv;  // per layer
  std::vector<bf16*> dkv;    // per depformer layer: [max_sessions][8][K | V][dep_dim]
  char* state = nullptr;
  int64_t stride = 256;
  std::vector<int32_t> free_leases;  // lease i owns pages [i * pages_per_session, ..) and state line i
  // prefix cache (model.rs:67-70, :242-259): up to kCacheSlots prefilled prompts of at most kCacheMaxLen rows, each in
  // its own pages behind the sessions' rings; a prompt is identified by its rows (ids and voice rows), not by a hash
  struct CachedPrefix {
    std::vector<int32_t> ids, voice, pages;
    int rows = 0;
  };
  std::vector<CachedPrefix> cache;
  int cache_first_page = 0;
  std::vector<std::unique_ptr<omni_duplex_session>> sessions;

  // activations (max_rows = max(max_prefill, max_sessions))
  int max_rows = 0;
  bf16 *x = nullptr, *xn = nullptr, *qkv = nullptr, *attn = nullptr, *y = nullptr, *gu = nullptr, *act = nullptr;
  bf16 *text_logits = nullptr, *audio_logits = nullptr;  // [max_sessions, text_vocab], [8][max_sessions][card]
  bf16 *dproj = nullptr, *dx = nullptr, *dxn = nullptr, *dqkv = nullptr, *dattn = nullptr, *dy = nullptr,
       *dgu = nullptr, *dact = nullptr;
  int32_t *rows_buf = nullptr, *drawn = nullptr, *emitted = nullptr;

  // staged inputs: one pinned block mirrored on the device
  char *in_host = nullptr, *in_dev = nullptr;
  size_t in_bytes = 0;
  int32_t* out_host = nullptr;  // emitted + error word
  uint32_t* err = nullptr;

  // the padding lease (model.rs:151,189): one page and one state line that the rows between the live sessions and the
  // tick's bucket run on
  int pad_page = 0, pad_line = 0;
  // one CUDA graph of the tick's kernels per bucket (session counts are padded up to 1, 2, 4, ... or max_sessions)
  struct TickGraph {
    cudaGraphExec_t exec = nullptr;
    int seen = 0, nodes = 0;
  };
  std::map<int, TickGraph> tick_graphs;
  bool use_graphs = true;

  GemmScratch scratch;
  std::map<std::tuple<const void*, const void*, const void*, int>, TcGemmPlan> plans;
  std::map<std::tuple<const void*, const void*, const void*, int>, RmGemmPlan> rm_plans;

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

#define DCUDA(m, expr)                                                                              \
  do {                                                                                              \
    cudaError_t e_ = (expr);                                                                        \
    if (e_ != cudaSuccess) return (m)->fail(OMNI_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)
#define DLAUNCH(m, expr) \
  do {                   \
    DCUDA(m, expr);      \
    ++(m)->launches;     \
  } while (0)
#define DTRY(expr)                  \
  do {                              \
    const int rc_ = (expr);         \
    if (rc_ != OMNI_OK) return rc_; \
  } while (0)

namespace {

template <typename T>
int dalloc(omni_duplex* m, T** out, size_t count, bool zero = false) {
  void* p = nullptr;
  DCUDA(m, cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T)));
  if (zero) DCUDA(m, cudaMemset(p, 0, std::max<size_t>(count, 1) * sizeof(T)));
  m->allocations.push_back(p);
  *out = static_cast<T*>(p);
  return OMNI_OK;
}

__global__ void duplex_f32_to_bf16(const float* __restrict__ src, bf16* __restrict__ dst, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2bfloat16(src[i]);
}

using Index = std::unordered_map<std::string, const omni_tensor*>;

// Allocates and fills one weight from the checkpoint tensor of that name; the shape must match.
int weight(omni_duplex* m, const Index& idx, const std::string& name, std::initializer_list<int64_t> shape, bf16** out) {
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
  DTRY(dalloc(m, out, (size_t)count));
  if (t->location == OMNI_DEVICE) {
    if (t->dtype == OMNI_BF16) {
      DCUDA(m, cudaMemcpy(*out, t->data, count * 2, cudaMemcpyDeviceToDevice));
    } else {
      duplex_f32_to_bf16<<<(unsigned)((count + 255) / 256), 256>>>((const float*)t->data, *out, count);
      DCUDA(m, cudaGetLastError());
      DCUDA(m, cudaDeviceSynchronize());
    }
  } else if (t->dtype == OMNI_BF16) {
    DCUDA(m, cudaMemcpy(*out, t->data, count * 2, cudaMemcpyHostToDevice));
  } else {
    std::vector<uint16_t> tmp((size_t)count);
    const float* src = (const float*)t->data;
    for (int64_t i = 0; i < count; ++i) tmp[i] = host_f2bf(src[i]);
    DCUDA(m, cudaMemcpy(*out, tmp.data(), count * 2, cudaMemcpyHostToDevice));
  }
  return OMNI_OK;
}

// y[rows, N] = x[rows, K] . w[N, K]^T on the path the row count calls for.
int gemm(omni_duplex* m, const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy) {
  if (rows <= 8 || !tc_supports(N, K, rows)) {
    DLAUNCH(m, gemv_launch(w, N, K, x, rows, y, ldy, Epilogue{}, m->sm_count, m->stream));
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
    DLAUNCH(m, rm_launch(rt->second, m->err, m->stream));
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
  DLAUNCH(m, tc_launch(it->second, m->scratch, m->err, m->stream));
  return OMNI_OK;
}

// The staged inputs of one call: i32 arrays carved from the pinned block, same offsets on the device.
struct Staging {
  omni_duplex* m;
  size_t used = 0;
  int32_t* take(size_t count) {
    int32_t* p = reinterpret_cast<int32_t*>(m->in_host + used);
    used += (count * 4 + 255) & ~(size_t)255;
    return used <= m->in_bytes ? p : nullptr;
  }
  template <typename T>
  const T* dev(const T* host) const {
    return reinterpret_cast<const T*>(m->in_dev + (reinterpret_cast<const char*>(host) - m->in_host));
  }
};

DuplexTables tables(const omni_duplex* m) {
  return DuplexTables{m->text_emb, m->audio_emb, m->cfg.text_vocab + 1, m->cfg.card + 1};
}

float rope_coef(const omni_duplex_config& c) {  // helium.rs:79-81
  return (float)(-std::log((double)c.rope_period) * 2.0 / (double)kHeliumHeadDim);
}

// Every Helium layer over `rows` rows of m->x; the output norm's rows end in m->xn (helium.rs:225-284). In a
// tensor-parallel pair the projections run on this rank's heads and channels, and the o and down projections' partial
// rows are summed over the pair inside the add + norm kernel that follows them.
int helium_forward(omni_duplex* m, int rows, const int32_t* pos, const int32_t* slot, const int32_t* seq,
                   const int32_t* indptr, const int32_t* pages) {
  const omni_duplex_config& c = m->cfg;
  const int D = c.dim, Dl = m->local_heads() * kHeliumHeadDim, Hl = m->local_hidden();
  const bool pair = m->tp > 1;
  if (pair && !m->tp_peer_region) return m->fail(OMNI_ERR_INVALID, "tensor-parallel pair not connected (omni_duplex_tp_connect)");
  const float scale = 1.f / std::sqrt((float)kHeliumHeadDim);
  DLAUNCH(m, launch_lm_norm(m->x, m->h[0].norm1, m->xn, rows, D, c.norm_eps, m->stream));
  for (int i = 0; i < c.layers; ++i) {
    const HeliumLayer& L = m->h[i];
    DTRY(gemm(m, L.qkv, 3 * Dl, D, m->xn, rows, m->qkv, 3 * Dl));
    DLAUNCH(m, launch_lm_rope_kv(m->qkv, pos, slot, m->kv[i], rows, m->local_heads(), rope_coef(c), m->kv_pages, m->err, m->stream));
    DLAUNCH(m, launch_lm_attend(m->qkv, m->kv[i], pos, seq, indptr, pages, m->attn, rows, m->local_heads(), scale, c.context,
                                m->kv_pages, m->err, m->stream));
    bf16* y_o = pair ? m->tp_buf(0) : m->y;
    DTRY(gemm(m, L.o, D, Dl, m->attn, rows, y_o, D));
    if (pair)
      DLAUNCH(m, launch_lm_tp_add_norm(y_o, m->tp_peer_buf(0), m->x, L.norm2, m->xn, rows, D, c.norm_eps, m->tp_link(), m->err, m->stream));
    else
      DLAUNCH(m, launch_lm_add_norm(m->y, m->x, L.norm2, m->xn, rows, D, c.norm_eps, m->stream));
    DTRY(gemm(m, L.gate_up, 2 * Hl, D, m->xn, rows, m->gu, 2 * Hl));
    DLAUNCH(m, launch_silu_mul(m->gu, m->act, rows, Hl, 0, m->stream));
    bf16* y_d = pair ? m->tp_buf(1) : m->y;
    DTRY(gemm(m, L.down, D, Hl, m->act, rows, y_d, D));
    const bf16* next = i + 1 < c.layers ? m->h[i + 1].norm1 : m->out_norm;
    if (pair)
      DLAUNCH(m, launch_lm_tp_add_norm(y_d, m->tp_peer_buf(1), m->x, next, m->xn, rows, D, c.norm_eps, m->tp_link(), m->err, m->stream));
    else
      DLAUNCH(m, launch_lm_add_norm(m->y, m->x, next, m->xn, rows, D, c.norm_eps, m->stream));
  }
  return OMNI_OK;
}

// The eight depformer passes of a tick (depformer.rs:137-259): m->xn and drawn[:, 0] in, drawn[:, 1..9] out.
int depformer_step(omni_duplex* m, int n, const int32_t* force, const int32_t* seeds) {
  const omni_duplex_config& c = m->cfg;
  const int D = c.dep_dim, H = c.dep_hidden, S = c.max_sessions;
  const float scale = 1.f / std::sqrt((float)kDepHeadDim);
  DTRY(gemm(m, m->d_input, kDepSteps * D, c.dim, m->xn, n, m->dproj, kDepSteps * D));
  for (int k = 0; k < kDepSteps; ++k) {
    const bf16* table = k == 0 ? m->d_text_emb : m->d_emb + (size_t)(k - 1) * (c.card + 1) * D;
    const int table_rows = k == 0 ? c.text_vocab + 1 : c.card + 1;
    DLAUNCH(m, launch_lm_dep_embed_norm(m->dproj, k, table, table_rows, m->drawn, m->d[0].norm1, m->dx, m->dxn, n, D,
                                        c.norm_eps, m->err, m->stream));
    for (int i = 0; i < c.dep_layers; ++i) {
      const DepLayer& L = m->d[i];
      DTRY(gemm(m, L.qkv + (size_t)k * 3 * D * D, 3 * D, D, m->dxn, n, m->dqkv, 3 * D));
      DLAUNCH(m, launch_lm_dep_kv_attend(m->dqkv, m->dkv[i], k, m->dattn, n, c.dep_heads, scale, m->stream));
      DTRY(gemm(m, L.out + (size_t)k * D * D, D, D, m->dattn, n, m->dy, D));
      DLAUNCH(m, launch_lm_add_norm(m->dy, m->dx, L.norm2, m->dxn, n, D, c.norm_eps, m->stream));
      DTRY(gemm(m, L.gate_in + (size_t)k * 2 * H * D, 2 * H, D, m->dxn, n, m->dgu, 2 * H));
      DLAUNCH(m, launch_silu_mul(m->dgu, m->dact, n, H, 0, m->stream));
      DTRY(gemm(m, L.gate_out + (size_t)k * D * H, D, H, m->dact, n, m->dy, D));
      if (i + 1 < c.dep_layers)
        DLAUNCH(m, launch_lm_add_norm(m->dy, m->dx, m->d[i + 1].norm1, m->dxn, n, D, c.norm_eps, m->stream));
      else
        DLAUNCH(m, launch_lm_add_norm(m->dy, m->dx, nullptr, nullptr, n, D, c.norm_eps, m->stream));
    }
    bf16* logits = m->audio_logits + (size_t)k * S * c.card;
    DTRY(gemm(m, m->d_heads + (size_t)k * c.card * D, c.card, D, m->dx, n, logits, c.card));
    DLAUNCH(m, launch_lm_sample(logits, c.card, c.card, c.audio_temperature, c.audio_top_k, force, seeds, 1 + k,
                                m->drawn, n, m->stream));
  }
  return OMNI_OK;
}

int finish(omni_duplex* m, size_t d2h_ints) {
  DCUDA(m, cudaMemcpyAsync(m->out_host + d2h_ints, m->err, 4, cudaMemcpyDeviceToHost, m->stream));
  DCUDA(m, cudaEventRecord(m->ev1, m->stream));
  DCUDA(m, cudaStreamSynchronize(m->stream));
  cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1);
  m->last_launches = m->launches;
  const uint32_t word = (uint32_t)m->out_host[d2h_ints];
  if (word != 0) {
    cudaMemsetAsync(m->err, 0, 4, m->stream);
    cudaStreamSynchronize(m->stream);
    return m->fail(OMNI_ERR_DEVICE, "device error word 0x%x (1: barrier wait ran out, 2: index out of range)", word);
  }
  return OMNI_OK;
}

bool valid_config(const omni_duplex_config& c) {
  auto row = [](int d) { return d >= 256 && d % 64 == 0 && d <= 8192; };
  return row(c.dim) && row(c.dep_dim) && c.dim == c.heads * kHeliumHeadDim && c.dep_dim == c.dep_heads * kDepHeadDim &&
         c.layers >= 1 && c.dep_layers >= 1 && c.hidden % 64 == 0 && c.dep_hidden % 64 == 0 && c.hidden > 0 &&
         c.dep_hidden > 0 && c.context >= 1 && c.text_vocab >= 1 && c.card >= 1 && c.max_sessions >= 1 &&
         c.max_prefill >= 1 && c.voice_rows >= 0 && c.tp_size >= 0 && c.tp_size <= 2 && c.tp_rank >= 0 &&
         c.tp_rank < std::max(c.tp_size, 1) && (c.tp_size < 2 || (c.heads % 2 == 0 && c.hidden % 128 == 0));
}

}  // namespace

extern "C" {

int32_t omni_duplex_create(const omni_duplex_config* config, const omni_tensor* tensors, int32_t n_tensors,
                           int32_t device, omni_duplex** out) {
  if (!config || !out || (!tensors && n_tensors > 0)) return OMNI_ERR_INVALID;
  omni_duplex* m = new omni_duplex();
  *out = m;
  m->cfg = *config;
  m->device = device;
  const omni_duplex_config& c = m->cfg;
  if (!valid_config(c)) return m->fail(OMNI_ERR_INVALID, "duplex config outside the supported shapes");
  DCUDA(m, cudaSetDevice(device));
  cudaDeviceProp prop;
  DCUDA(m, cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return m->fail(OMNI_ERR_UNSUPPORTED, "device is sm_%d%d; this library is sm_100a only", prop.major, prop.minor);
  m->sm_count = prop.multiProcessorCount;
  m->use_graphs = c.use_graphs != 0;
  m->tp = c.tp_size >= 2 ? c.tp_size : 1;
  m->tp_rank = c.tp_rank;
  DCUDA(m, cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
  DCUDA(m, cudaEventCreate(&m->ev0));
  DCUDA(m, cudaEventCreate(&m->ev1));
  if (tc_init() != 0) return m->fail(OMNI_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  tc_configure();

  Index idx;
  for (int i = 0; i < n_tensors; ++i)
    if (tensors[i].name) idx[tensors[i].name] = &tensors[i];
  const int64_t D = c.dim, H = c.hidden, DD = c.dep_dim, DH = c.dep_hidden, card1 = c.card + 1;
  const int64_t Dl = (int64_t)m->local_heads() * kHeliumHeadDim, Hl = m->local_hidden();
  DTRY(weight(m, idx, "h.text_emb", {c.text_vocab + 1, D}, &m->text_emb));
  DTRY(weight(m, idx, "h.audio_emb", {16 * card1, D}, &m->audio_emb));
  DTRY(weight(m, idx, "h.out_norm", {D}, &m->out_norm));
  DTRY(weight(m, idx, "h.text_linear", {c.text_vocab, D}, &m->text_linear));
  if (c.voice_rows > 0) DTRY(weight(m, idx, "voices", {c.voice_rows, D}, &m->voices));
  m->h.resize(c.layers);
  for (int i = 0; i < c.layers; ++i) {
    const std::string p = "h.l" + std::to_string(i) + ".";
    HeliumLayer& L = m->h[i];
    DTRY(weight(m, idx, p + "norm1", {D}, &L.norm1));
    // a rank of a tensor-parallel pair is given its own rows / columns of the four projections (header)
    DTRY(weight(m, idx, p + "qkv", {3 * Dl, D}, &L.qkv));
    DTRY(weight(m, idx, p + "o", {D, Dl}, &L.o));
    DTRY(weight(m, idx, p + "norm2", {D}, &L.norm2));
    DTRY(weight(m, idx, p + "gate_up", {2 * Hl, D}, &L.gate_up));
    DTRY(weight(m, idx, p + "down", {D, Hl}, &L.down));
  }
  DTRY(weight(m, idx, "d.input", {kDepSteps * DD, D}, &m->d_input));
  DTRY(weight(m, idx, "d.text_emb", {c.text_vocab + 1, DD}, &m->d_text_emb));
  DTRY(weight(m, idx, "d.emb", {(kDepSteps - 1) * card1, DD}, &m->d_emb));
  DTRY(weight(m, idx, "d.heads", {(int64_t)kDepSteps * c.card, DD}, &m->d_heads));
  m->d.resize(c.dep_layers);
  for (int i = 0; i < c.dep_layers; ++i) {
    const std::string p = "d.l" + std::to_string(i) + ".";
    DepLayer& L = m->d[i];
    DTRY(weight(m, idx, p + "norm1", {DD}, &L.norm1));
    DTRY(weight(m, idx, p + "qkv", {kDepSteps * 3 * DD, DD}, &L.qkv));
    DTRY(weight(m, idx, p + "out", {kDepSteps * DD, DD}, &L.out));
    DTRY(weight(m, idx, p + "norm2", {DD}, &L.norm2));
    DTRY(weight(m, idx, p + "gate_in", {kDepSteps * 2 * DH, DD}, &L.gate_in));
    DTRY(weight(m, idx, p + "gate_out", {kDepSteps * DD, DH}, &L.gate_out));
  }

  // pools: every lease is a ring of `context` positions (model.rs:67) and one state line
  const int S = c.max_sessions;
  m->pages_per_session = (c.context + 15) / 16;
  m->cache_first_page = S * m->pages_per_session;
  m->kv_pages = m->cache_first_page + kCacheSlots * ((kCacheMaxLen + 15) / 16) + 1;
  m->pad_page = m->kv_pages - 1;
  m->pad_line = S;
  m->kv.resize(c.layers);
  for (int i = 0; i < c.layers; ++i)
    DTRY(dalloc(m, &m->kv[i], (size_t)m->kv_pages * m->local_heads() * kDuplexPageHeadBytes, true));
  m->dkv.resize(c.dep_layers);
  for (int i = 0; i < c.dep_layers; ++i) DTRY(dalloc(m, &m->dkv[i], (size_t)S * kDepSteps * 2 * DD, true));
  DTRY(dalloc(m, &m->state, (size_t)(S + 1) * m->stride, true));
  for (int i = S - 1; i >= 0; --i) m->free_leases.push_back(i);

  m->max_rows = std::max(c.max_prefill, S);
  const size_t R = m->max_rows;
  DTRY(dalloc(m, &m->x, R * D));
  DTRY(dalloc(m, &m->xn, R * D));
  DTRY(dalloc(m, &m->qkv, R * 3 * D));
  DTRY(dalloc(m, &m->attn, R * D));
  DTRY(dalloc(m, &m->y, R * D));
  if (m->tp > 1) {  // the pair's exchange region: words, then two buffers of max_rows x dim partial rows
    m->tp_buf_bytes = (R * D * sizeof(bf16) + 255) & ~(size_t)255;
    DTRY(dalloc(m, &m->tp_region, 256 + 2 * m->tp_buf_bytes, true));
  }
  DTRY(dalloc(m, &m->gu, R * 2 * H));
  DTRY(dalloc(m, &m->act, R * H));
  DTRY(dalloc(m, &m->text_logits, (size_t)S * c.text_vocab, true));
  DTRY(dalloc(m, &m->audio_logits, (size_t)kDepSteps * S * c.card, true));
  DTRY(dalloc(m, &m->dproj, (size_t)S * kDepSteps * DD));
  DTRY(dalloc(m, &m->dx, (size_t)S * DD));
  DTRY(dalloc(m, &m->dxn, (size_t)S * DD));
  DTRY(dalloc(m, &m->dqkv, (size_t)S * 3 * DD));
  DTRY(dalloc(m, &m->dattn, (size_t)S * DD));
  DTRY(dalloc(m, &m->dy, (size_t)S * DD));
  DTRY(dalloc(m, &m->dgu, (size_t)S * 2 * DH));
  DTRY(dalloc(m, &m->dact, (size_t)S * DH));
  DTRY(dalloc(m, &m->rows_buf, (size_t)S * kDuplexStreams, true));
  DTRY(dalloc(m, &m->drawn, (size_t)S * kDuplexDrawn, true));
  DTRY(dalloc(m, &m->emitted, (size_t)S * kDuplexDrawn, true));
  DTRY(dalloc(m, &m->err, 64, true));

  // staged inputs: per row pos, slot, seq, voice, 17 ids; per session lines, indptr, pages, init, force, ...
  m->in_bytes = (R * (6 + kDuplexStreams) + (size_t)S * (8 + m->pages_per_session + OMNI_DUPLEX_STATE + 40)) * 4 + 64 * 256;
  DCUDA(m, cudaMallocHost((void**)&m->in_host, m->in_bytes));
  DTRY(dalloc(m, &m->in_dev, m->in_bytes));
  DCUDA(m, cudaMallocHost((void**)&m->out_host, ((size_t)S * kDuplexDrawn + 1) * 4));

  // split-K scratch of the tensor-core GEMM: the largest plan over the shapes above at max_rows rows
  m->scratch.partial_floats = (size_t)32 << 20;
  m->scratch.counter_slots = 1 << 16;
  DTRY(dalloc(m, &m->scratch.partials, m->scratch.partial_floats));
  DTRY(dalloc(m, &m->scratch.counters, (size_t)m->scratch.counter_slots, true));
  return OMNI_OK;
}

void omni_duplex_destroy(omni_duplex* m) {
  if (!m) return;
  cudaSetDevice(m->device);
  if (m->stream) cudaStreamSynchronize(m->stream);
  for (auto& g : m->tick_graphs)
    if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
  if (m->tp_peer_region) cudaIpcCloseMemHandle(m->tp_peer_region);
  for (void* p : m->allocations) cudaFree(p);
  if (m->in_host) cudaFreeHost(m->in_host);
  if (m->out_host) cudaFreeHost(m->out_host);
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

const char* omni_duplex_last_error(const omni_duplex* m) { return m ? m->error.c_str() : "null model"; }

int32_t omni_duplex_tp_export(omni_duplex* m, void* handle, size_t bytes) {
  if (!m || !handle) return OMNI_ERR_INVALID;
  if (m->tp < 2) return m->fail(OMNI_ERR_INVALID, "the model is not a rank of a tensor-parallel pair");
  if (bytes < sizeof(cudaIpcMemHandle_t)) return m->fail(OMNI_ERR_INVALID, "handle buffer below %zu bytes", sizeof(cudaIpcMemHandle_t));
  DCUDA(m, cudaSetDevice(m->device));
  cudaIpcMemHandle_t h;
  DCUDA(m, cudaIpcGetMemHandle(&h, m->tp_region));
  memcpy(handle, &h, sizeof(h));
  return OMNI_OK;
}

int32_t omni_duplex_tp_connect(omni_duplex* m, const void* peer_handle, size_t bytes) {
  if (!m || !peer_handle) return OMNI_ERR_INVALID;
  if (m->tp < 2) return m->fail(OMNI_ERR_INVALID, "the model is not a rank of a tensor-parallel pair");
  if (bytes < sizeof(cudaIpcMemHandle_t)) return m->fail(OMNI_ERR_INVALID, "handle below %zu bytes", sizeof(cudaIpcMemHandle_t));
  if (m->tp_peer_region) return m->fail(OMNI_ERR_INVALID, "the pair is connected already");
  DCUDA(m, cudaSetDevice(m->device));
  cudaIpcMemHandle_t h;
  memcpy(&h, peer_handle, sizeof(h));
  void* p = nullptr;
  DCUDA(m, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  m->tp_peer_region = static_cast<char*>(p);
  return OMNI_OK;
}

int32_t omni_duplex_open(omni_duplex* m, omni_duplex_session** out) {
  if (!m || !out) return OMNI_ERR_INVALID;
  *out = nullptr;
  if (m->free_leases.empty()) return OMNI_DENIED_BUSY;
  const int lease = m->free_leases.back();
  m->free_leases.pop_back();
  auto s = std::make_unique<omni_duplex_session>();
  s->line = lease;
  s->pages.resize(m->pages_per_session);
  for (int i = 0; i < m->pages_per_session; ++i) s->pages[i] = lease * m->pages_per_session + i;
  for (int k = 0; k < OMNI_DUPLEX_DRAWN; ++k) s->first_force[k] = -1;
  s->live = true;
  cudaSetDevice(m->device);
  DCUDA(m, cudaMemsetAsync(m->state + (int64_t)lease * m->stride, 0, m->stride, m->stream));
  *out = s.get();
  m->sessions.push_back(std::move(s));
  return OMNI_OK;
}

int32_t omni_duplex_close(omni_duplex* m, omni_duplex_session* session) {
  if (!m || !session) return OMNI_ERR_INVALID;
  for (size_t i = 0; i < m->sessions.size(); ++i) {
    if (m->sessions[i].get() != session) continue;
    if (session->live) m->free_leases.push_back(session->line);
    m->sessions.erase(m->sessions.begin() + i);
    return OMNI_OK;
  }
  return m->fail(OMNI_ERR_INVALID, "close of a session this model does not own");
}

int32_t omni_duplex_position(const omni_duplex_session* session, int32_t* pos, int64_t* frame) {
  if (!session) return OMNI_ERR_INVALID;
  if (pos) *pos = session->pos;
  if (frame) *frame = session->frame;
  return OMNI_OK;
}

namespace {

// One prompt as the caller gave it: `rows` rows of 17 ids and (optionally) voice rows.
struct PromptView {
  const int32_t* ids;
  const int32_t* voice;  // may be null
  int rows;
};

int find_cached(const omni_duplex* m, const PromptView& p) {
  for (size_t i = 0; i < m->cache.size(); ++i) {
    const auto& c = m->cache[i];
    if (c.rows != p.rows || memcmp(c.ids.data(), p.ids, (size_t)p.rows * kDuplexStreams * 4) != 0) continue;
    bool same = true;
    for (int r = 0; r < p.rows && same; ++r) same = c.voice[r] == (p.voice ? p.voice[r] : -1);
    if (same) return (int)i;
  }
  return -1;
}

// Helium prefill of `n` prompts into the given page lists (`prefill_leases`, model.rs:298-320); lines/init may be null
// (a cache fill has no token state).
int prefill(omni_duplex* m, int n, const PromptView* prompts, const std::vector<int32_t>* const* page_lists,
            const int32_t* lines_in, const int32_t* init) {
  const omni_duplex_config& c = m->cfg;
  int total = 0;
  for (int i = 0; i < n; ++i) total += prompts[i].rows;
  Staging st{m};
  int32_t *pos = st.take(total), *slot = st.take(total), *seq = st.take(total), *vrow = st.take(total);
  int32_t* tok = st.take((size_t)total * kDuplexStreams);
  size_t page_count = 0;
  for (int i = 0; i < n; ++i) page_count += page_lists[i]->size();
  int32_t *lines = st.take(n), *indptr = st.take(n + 1), *pages = st.take(page_count);
  int32_t* ini = st.take((size_t)n * OMNI_DUPLEX_STATE);
  if (!ini) return m->fail(OMNI_ERR_INVALID, "staging block too small");
  int r = 0;
  indptr[0] = 0;
  for (int i = 0; i < n; ++i) {
    const std::vector<int32_t>& pl = *page_lists[i];
    for (int p = 0; p < prompts[i].rows; ++p, ++r) {
      pos[r] = p;
      slot[r] = pl[(p % c.context) >> 4] * 16 + ((p % c.context) & 15);
      seq[r] = i;
      vrow[r] = prompts[i].voice ? prompts[i].voice[p] : -1;
    }
    memcpy(tok + (size_t)(r - prompts[i].rows) * kDuplexStreams, prompts[i].ids, (size_t)prompts[i].rows * kDuplexStreams * 4);
    if (lines_in) lines[i] = lines_in[i];
    memcpy(pages + indptr[i], pl.data(), pl.size() * 4);
    indptr[i + 1] = indptr[i] + (int)pl.size();
  }
  if (init) memcpy(ini, init, (size_t)n * OMNI_DUPLEX_STATE * 4);
  DCUDA(m, cudaMemcpyAsync(m->in_dev, m->in_host, st.used, cudaMemcpyHostToDevice, m->stream));
  DLAUNCH(m, launch_lm_embed_ids(st.dev(tok), st.dev(vrow), m->voices, c.voice_rows, tables(m), m->x, total, c.dim,
                                 m->err, m->stream));
  DTRY(helium_forward(m, total, st.dev(pos), st.dev(slot), st.dev(seq), st.dev(indptr), st.dev(pages)));
  if (lines_in && init) DLAUNCH(m, launch_lm_init(m->state, st.dev(lines), m->stride, st.dev(ini), n, m->stream));
  // the staging block is reused by the next call of this function: wait for this one's copy and kernels
  DCUDA(m, cudaStreamSynchronize(m->stream));
  return OMNI_OK;
}

// `warm_prefix` (model.rs:248-259): prefill into a cache slot if the prompt is short enough and a slot is free.
int warm(omni_duplex* m, const PromptView& p, bool* cached_now) {
  *cached_now = find_cached(m, p) >= 0;
  if (*cached_now || (int)m->cache.size() >= kCacheSlots || p.rows > kCacheMaxLen) return OMNI_OK;
  omni_duplex::CachedPrefix e;
  e.rows = p.rows;
  e.ids.assign(p.ids, p.ids + (size_t)p.rows * kDuplexStreams);
  e.voice.resize(p.rows);
  for (int r = 0; r < p.rows; ++r) e.voice[r] = p.voice ? p.voice[r] : -1;
  const int per = (kCacheMaxLen + 15) / 16, first = m->cache_first_page + (int)m->cache.size() * per;
  for (int i = 0; i < (p.rows + 15) / 16; ++i) e.pages.push_back(first + i);
  const std::vector<int32_t>* pl = &e.pages;
  DTRY(prefill(m, 1, &p, &pl, nullptr, nullptr));
  m->cache.push_back(std::move(e));
  *cached_now = true;
  return OMNI_OK;
}

int check_prompt_args(omni_duplex* m, const int32_t* ids, const int32_t* voice, int rows) {
  if (!m || !ids || rows < 1) return OMNI_ERR_INVALID;
  if (rows >= m->cfg.context) return m->fail(OMNI_ERR_INVALID, "a prompt of %d steps does not fit the %d-step context", rows, m->cfg.context);
  if (rows > m->cfg.max_prefill) return m->fail(OMNI_ERR_INVALID, "%d prompt rows exceed max_prefill %d", rows, m->cfg.max_prefill);
  if (voice && m->cfg.voice_rows == 0)
    for (int r = 0; r < rows; ++r)
      if (voice[r] >= 0) return m->fail(OMNI_ERR_INVALID, "row %d names a voice but the model has none", r);
  return OMNI_OK;
}

}  // namespace

int32_t omni_duplex_is_cached(omni_duplex* m, int32_t rows, const int32_t* ids, const int32_t* voice) {
  if (!m || !ids || rows < 1) return 0;
  return find_cached(m, PromptView{ids, voice, rows}) >= 0 ? 1 : 0;
}

int32_t omni_duplex_warm_prefix(omni_duplex* m, int32_t rows, const int32_t* ids, const int32_t* voice) {
  DTRY(check_prompt_args(m, ids, voice, rows));
  DCUDA(m, cudaSetDevice(m->device));
  m->launches = 0;
  DCUDA(m, cudaEventRecord(m->ev0, m->stream));
  bool cached = false;
  DTRY(warm(m, PromptView{ids, voice, rows}, &cached));
  return finish(m, 0);
}

int32_t omni_duplex_start(omni_duplex* m, int32_t n, omni_duplex_session* const* sessions, const int32_t* row_counts,
                          const int32_t* ids, const int32_t* voice, const int32_t* init, const int32_t* first_force) {
  if (!m || !sessions || !row_counts || !ids || !init) return OMNI_ERR_INVALID;
  const omni_duplex_config& c = m->cfg;
  if (n < 1 || n > c.max_sessions) return m->fail(OMNI_ERR_INVALID, "%d sessions in one start", n);
  int total = 0;
  std::vector<PromptView> prompts(n);
  for (int i = 0; i < n; ++i) {
    if (!sessions[i] || !sessions[i]->live) return m->fail(OMNI_ERR_INVALID, "session %d is not open", i);
    if (sessions[i]->pos != 0) return m->fail(OMNI_ERR_INVALID, "session %d was already started", i);
    for (int j = 0; j < i; ++j)
      if (sessions[j] == sessions[i]) return m->fail(OMNI_ERR_INVALID, "session %d appears twice", i);
    prompts[i] = PromptView{ids + (size_t)total * kDuplexStreams, voice ? voice + total : nullptr, row_counts[i]};
    DTRY(check_prompt_args(m, prompts[i].ids, prompts[i].voice, row_counts[i]));
    total += std::max(row_counts[i], 0);
  }
  if (total > c.max_prefill) return m->fail(OMNI_ERR_INVALID, "%d prompt rows exceed max_prefill %d", total, c.max_prefill);
  DCUDA(m, cudaSetDevice(m->device));
  m->launches = 0;
  DCUDA(m, cudaEventRecord(m->ev0, m->stream));
  // `Model::start` (model.rs:325-370): fill the cache once per eligible prompt, copy the cached ones, prefill the rest
  std::vector<int> cached_slot(n, -1);
  for (int i = 0; i < n; ++i) {
    bool cached = false;
    DTRY(warm(m, prompts[i], &cached));
    if (cached) cached_slot[i] = find_cached(m, prompts[i]);
  }
  {
    Staging st{m};
    int copies = 0, copied_sessions = 0;
    for (int i = 0; i < n; ++i)
      if (cached_slot[i] >= 0) copies += prompts[i].rows, ++copied_sessions;
    if (copies > 0) {
      int32_t *src = st.take(copies), *dst = st.take(copies), *lines = st.take(copied_sessions);
      int32_t* ini = st.take((size_t)copied_sessions * OMNI_DUPLEX_STATE);
      if (!ini) return m->fail(OMNI_ERR_INVALID, "staging block too small");
      int r = 0, k = 0;
      for (int i = 0; i < n; ++i) {
        if (cached_slot[i] < 0) continue;
        const auto& e = m->cache[cached_slot[i]];
        for (int p = 0; p < prompts[i].rows; ++p, ++r) {
          src[r] = e.pages[p >> 4] * 16 + (p & 15);
          dst[r] = sessions[i]->pages[(p % c.context) >> 4] * 16 + ((p % c.context) & 15);
        }
        lines[k] = sessions[i]->line;
        memcpy(ini + (size_t)k * OMNI_DUPLEX_STATE, init + (size_t)i * OMNI_DUPLEX_STATE, OMNI_DUPLEX_STATE * 4);
        ++k;
      }
      DCUDA(m, cudaMemcpyAsync(m->in_dev, m->in_host, st.used, cudaMemcpyHostToDevice, m->stream));
      for (int l = 0; l < c.layers; ++l)
        DLAUNCH(m, launch_lm_copy_kv(m->kv[l], st.dev(src), st.dev(dst), copies, m->local_heads(), m->kv_pages, m->err, m->stream));
      DLAUNCH(m, launch_lm_init(m->state, st.dev(lines), m->stride, st.dev(ini), copied_sessions, m->stream));
      DCUDA(m, cudaStreamSynchronize(m->stream));
    }
  }
  {
    std::vector<PromptView> rest;
    std::vector<const std::vector<int32_t>*> lists;
    std::vector<int32_t> lines, ini;
    for (int i = 0; i < n; ++i) {
      if (cached_slot[i] >= 0) continue;
      rest.push_back(prompts[i]);
      lists.push_back(&sessions[i]->pages);
      lines.push_back(sessions[i]->line);
      ini.insert(ini.end(), init + (size_t)i * OMNI_DUPLEX_STATE, init + (size_t)(i + 1) * OMNI_DUPLEX_STATE);
    }
    if (!rest.empty()) DTRY(prefill(m, (int)rest.size(), rest.data(), lists.data(), lines.data(), ini.data()));
  }
  DTRY(finish(m, 0));
  for (int i = 0; i < n; ++i) {
    sessions[i]->pos = row_counts[i];
    sessions[i]->frame = 0;
    for (int k = 0; k < OMNI_DUPLEX_DRAWN; ++k)
      sessions[i]->first_force[k] = first_force ? first_force[i * OMNI_DUPLEX_DRAWN + k] : -1;
  }
  return OMNI_OK;
}

}  // extern "C"

namespace {

// The tick's bucket (`bucket`, crates/omni-kern/src/lib.rs:31-36,97-101): the next power of two, capped at max_sessions.
int tick_bucket(const omni_duplex* m, int n) {
  int b = 1;
  while (b < n) b <<= 1;
  return std::min(b, m->cfg.max_sessions);
}

// One tick of n live sessions padded to bucket b (n = 0: the warm-up's tick, every row on the padding lease).
int tick_rows(omni_duplex* m, int n, int b, omni_duplex_session* const* sessions, const omni_duplex_step* steps,
              int32_t* emitted) {
  const omni_duplex_config& c = m->cfg;
  DCUDA(m, cudaSetDevice(m->device));
  Staging st{m};
  int32_t *pos = st.take(b), *slot = st.take(b), *lines = st.take(b), *indptr = st.take(b + 1);
  int32_t* pages = st.take((size_t)b * m->pages_per_session);
  int32_t *force = st.take((size_t)b * kDuplexDrawn), *force_caller = st.take((size_t)b * kDuplexBooks);
  int32_t *caller = st.take((size_t)b * kDuplexBooks), *seeds = st.take((size_t)b * 2);
  if (!seeds) return m->fail(OMNI_ERR_INVALID, "staging block too small");
  indptr[0] = 0;
  for (int i = 0; i < n; ++i) {
    const omni_duplex_session* s = sessions[i];
    const int ring = s->pos % c.context;
    pos[i] = s->pos;
    slot[i] = s->pages[ring >> 4] * 16 + (ring & 15);
    lines[i] = s->line;
    memcpy(pages + indptr[i], s->pages.data(), s->pages.size() * 4);
    indptr[i + 1] = indptr[i] + (int)s->pages.size();
    for (int k = 0; k < kDuplexDrawn; ++k) {  // the first tick takes what the prompt fixed (model.rs:392-396)
      const int f = steps[i].force[k];
      force[i * kDuplexDrawn + k] = s->frame == 0 && f < 0 ? s->first_force[k] : f;
    }
    memcpy(force_caller + i * kDuplexBooks, steps[i].force_caller, kDuplexBooks * 4);
    memcpy(caller + i * kDuplexBooks, steps[i].caller, kDuplexBooks * 4);
    seeds[2 * i] = (int32_t)(uint32_t)steps[i].seed;
    seeds[2 * i + 1] = (int32_t)(uint32_t)(steps[i].seed >> 32);
  }
  for (int i = n; i < b; ++i) {  // padding rows: position 0 of the padding lease, nothing forced, seed 0 (model.rs:403-415)
    pos[i] = 0;
    slot[i] = m->pad_page * 16;
    lines[i] = m->pad_line;
    pages[indptr[i]] = m->pad_page;
    indptr[i + 1] = indptr[i] + 1;
    for (int k = 0; k < kDuplexDrawn; ++k) force[i * kDuplexDrawn + k] = -1;
    for (int k = 0; k < kDuplexBooks; ++k) force_caller[i * kDuplexBooks + k] = -1, caller[i * kDuplexBooks + k] = 0;
    seeds[2 * i] = seeds[2 * i + 1] = 0;
  }
  m->launches = 0;
  DCUDA(m, cudaEventRecord(m->ev0, m->stream));
  DCUDA(m, cudaMemcpyAsync(m->in_dev, m->in_host, st.used, cudaMemcpyHostToDevice, m->stream));
  // The kernels of a tick and their arguments depend on b alone (positions, pages, forces and seeds are read from the
  // staged block, whose layout b fixes), so the sequence is captured once per bucket and replayed as a CUDA graph. The
  // first tick of a bucket runs eagerly (it creates the GEMM plans), the second is captured; omni_duplex_warmup does
  // both for every bucket before live traffic.
  auto body = [&]() -> int {
    // `Helium::step` (helium.rs:189-222)
    DLAUNCH(m, launch_lm_embed_state(m->state, st.dev(lines), m->stride, tables(m), m->x, m->rows_buf, b, c.dim, m->err,
                                     m->stream));
    DTRY(helium_forward(m, b, st.dev(pos), st.dev(slot), nullptr, st.dev(indptr), st.dev(pages)));
    DTRY(gemm(m, m->text_linear, c.text_vocab, c.dim, m->xn, b, m->text_logits, c.text_vocab));
    DLAUNCH(m, launch_lm_sample(m->text_logits, c.text_vocab, c.text_vocab, c.text_temperature, c.text_top_k,
                                st.dev(force), st.dev(seeds), 0, m->drawn, b, m->stream));
    DTRY(depformer_step(m, b, st.dev(force), st.dev(seeds)));
    DLAUNCH(m, launch_lm_advance(m->state, st.dev(lines), m->stride, m->drawn, st.dev(caller), st.dev(force_caller),
                                 m->emitted, b, m->stream));
    return OMNI_OK;
  };
  omni_duplex::TickGraph& tg = m->tick_graphs[b];
  if (!m->use_graphs || tg.seen == 0) {
    DTRY(body());
    tg.seen = 1;
  } else {
    if (!tg.exec) {
      DCUDA(m, cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
      const int rc = body();
      cudaGraph_t graph = nullptr;
      const cudaError_t end = cudaStreamEndCapture(m->stream, &graph);  // always ends the capture, also after a failure
      if (rc != OMNI_OK || end != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return rc != OMNI_OK ? rc : m->fail(OMNI_ERR_CUDA, "tick capture: %s", cudaGetErrorString(end));
      }
      const cudaError_t inst = cudaGraphInstantiate(&tg.exec, graph, 0);
      cudaGraphDestroy(graph);
      if (inst != cudaSuccess) {
        tg.exec = nullptr;
        return m->fail(OMNI_ERR_CUDA, "tick graph: %s", cudaGetErrorString(inst));
      }
      tg.nodes = m->launches;
    }
    DCUDA(m, cudaGraphLaunch(tg.exec, m->stream));
    m->launches = tg.nodes;
  }
  if (n > 0)
    DCUDA(m, cudaMemcpyAsync(m->out_host, m->emitted, (size_t)n * kDuplexDrawn * 4, cudaMemcpyDeviceToHost, m->stream));
  DTRY(finish(m, (size_t)n * kDuplexDrawn));
  if (n > 0) memcpy(emitted, m->out_host, (size_t)n * kDuplexDrawn * 4);
  return OMNI_OK;
}

}  // namespace

extern "C" {

int32_t omni_duplex_tick(omni_duplex* m, int32_t n, omni_duplex_session* const* sessions,
                         const omni_duplex_step* steps, int32_t* emitted) {
  if (!m || !sessions || !steps || !emitted) return OMNI_ERR_INVALID;
  const omni_duplex_config& c = m->cfg;
  if (n < 1 || n > c.max_sessions) return m->fail(OMNI_ERR_INVALID, "%d sessions in one tick", n);
  for (int i = 0; i < n; ++i) {
    if (!sessions[i] || !sessions[i]->live) return m->fail(OMNI_ERR_INVALID, "session %d is not open", i);
    if (sessions[i]->pos <= 0) return m->fail(OMNI_ERR_INVALID, "a session that was not started");
    for (int j = 0; j < i; ++j)
      if (sessions[j] == sessions[i]) return m->fail(OMNI_ERR_INVALID, "session %d appears twice", i);
  }
  DTRY(tick_rows(m, n, tick_bucket(m, n), sessions, steps, emitted));
  for (int i = 0; i < n; ++i) {
    sessions[i]->pos += 1;
    sessions[i]->frame += 1;
  }
  return OMNI_OK;
}

// `Model::warmup` (model.rs:202-240): every bucket's tick on the padding lease, twice (plans, then the captured graph),
// so that no live tick pays for a graph capture.
int32_t omni_duplex_warmup(omni_duplex* m) {
  if (!m) return OMNI_ERR_INVALID;
  std::vector<int> buckets;
  for (int b = 1; b < m->cfg.max_sessions; b <<= 1) buckets.push_back(b);
  buckets.push_back(m->cfg.max_sessions);
  for (int b : buckets)
    for (int pass = 0; pass < (m->use_graphs ? 2 : 1); ++pass) DTRY(tick_rows(m, 0, b, nullptr, nullptr, nullptr));
  return OMNI_OK;
}

int32_t omni_duplex_read(omni_duplex* m, int32_t buffer, int32_t s, void* dst, size_t bytes) {
  if (!m || !dst) return OMNI_ERR_INVALID;
  const omni_duplex_config& c = m->cfg;
  if (s < 0 || s >= c.max_sessions) return m->fail(OMNI_ERR_INVALID, "session index %d", s);
  DCUDA(m, cudaSetDevice(m->device));
  DCUDA(m, cudaStreamSynchronize(m->stream));
  switch (buffer) {
    case OMNI_DUPLEX_TEXT_LOGITS:
      if (bytes > (size_t)c.text_vocab * 2) return m->fail(OMNI_ERR_INVALID, "read past the buffer");
      DCUDA(m, cudaMemcpy(dst, m->text_logits + (size_t)s * c.text_vocab, bytes, cudaMemcpyDeviceToHost));
      return OMNI_OK;
    case OMNI_DUPLEX_AUDIO_LOGITS: {
      if (bytes > (size_t)kDepSteps * c.card * 2) return m->fail(OMNI_ERR_INVALID, "read past the buffer");
      size_t done = 0;
      for (int k = 0; k < kDepSteps && done < bytes; ++k) {
        const size_t part = std::min(bytes - done, (size_t)c.card * 2);
        DCUDA(m, cudaMemcpy(static_cast<char*>(dst) + done,
                            m->audio_logits + ((size_t)k * c.max_sessions + s) * c.card, part, cudaMemcpyDeviceToHost));
        done += part;
      }
      return OMNI_OK;
    }
    case OMNI_DUPLEX_ROWS:
      if (bytes > (size_t)kDuplexStreams * 4) return m->fail(OMNI_ERR_INVALID, "read past the buffer");
      DCUDA(m, cudaMemcpy(dst, m->rows_buf + (size_t)s * kDuplexStreams, bytes, cudaMemcpyDeviceToHost));
      return OMNI_OK;
    case OMNI_DUPLEX_DRAWN_BUF:
      if (bytes > (size_t)kDuplexDrawn * 4) return m->fail(OMNI_ERR_INVALID, "read past the buffer");
      DCUDA(m, cudaMemcpy(dst, m->drawn + (size_t)s * kDuplexDrawn, bytes, cudaMemcpyDeviceToHost));
      return OMNI_OK;
    default:
      return m->fail(OMNI_ERR_INVALID, "unknown buffer %d", buffer);
  }
}

int32_t omni_duplex_stats(const omni_duplex* m, float* last_call_gpu_ms, int32_t* last_call_launches) {
  if (!m) return OMNI_ERR_INVALID;
  if (last_call_gpu_ms) *last_call_gpu_ms = m->last_ms;
  if (last_call_launches) *last_call_launches = m->last_launches;
  return OMNI_OK;
}

}  // extern "C"
