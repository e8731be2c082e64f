// Host runtime of the talker token loop and its C ABI (include/omni_b200.h).
//
// Mirrors the reference's model shell (crates/omni-qwen3-tts/src/model.rs) and
// what kern-runtime provides underneath it: weights fused at load, a paged KV
// pool with leases, per-sequence state slots, batch buckets with a padding
// lease, host inputs staged in one block, one CUDA graph per (program, bucket),
// synchronous read-back of the frame.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "../../include/omni_b200.h"
#include "../../include/omni_b200_codec.h"
#include "gemm.h"
#include "kernels.h"
#include "predictor.h"
#include "tick.h"

namespace omni {

namespace {

const int kBuckets[] = {1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128};

int bucket_of(int n) {
  for (int b : kBuckets)
    if (b >= n) return b;
  return (n + 63) / 64 * 64;  // beyond the reference's largest bucket: multiples of 64
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, int64_t n) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2bfloat16(src[i]);
}

// dst = the fused [gate; up] rows of src regrouped as `granule` gate rows, the matching `granule` up rows, ...:
// one tensor-core tile of 2 * granule weight rows then holds a channel's gate and up columns for the SwiGLU epilogue.
__global__ void interleave_gate_up_kernel(const bf16* __restrict__ src, bf16* __restrict__ dst, int inter, int k,
                                          int granule) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 16-byte piece
  const int64_t per_row = k / 8, total = (int64_t)2 * inter * per_row;
  if (i >= total) return;
  const int64_t row = i / per_row, piece = i % per_row;
  const bool up = row >= inter;
  const int64_t c = up ? row - inter : row;
  const int64_t out_row = (c / granule) * 2 * granule + (up ? granule : 0) + c % granule;
  *reinterpret_cast<Pack8*>(dst + out_row * k + piece * 8) = *reinterpret_cast<const Pack8*>(src + row * k + piece * 8);
}

uint16_t host_f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

struct StackW {
  omni_stack_config cfg;
  struct Layer {
    bf16 *ln1, *qkv, *q_norm, *k_norm, *o, *ln2, *gate_up, *down;
  };
  std::vector<Layer> layers;
  bf16* norm = nullptr;
  int granule = 128;  // gate|up interleave (channels per group)
  int qkv_width() const { return (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim; }
  size_t kv_page_elems() const { return (size_t)cfg.kv_heads * 2 * OMNI_PAGE * cfg.head_dim; }
  AttnShape attn() const { return AttnShape{cfg.q_heads, cfg.kv_heads, cfg.head_dim, cfg.rms_eps, cfg.rope_theta}; }
};

struct Scratch {
  bf16 *x, *res, *qkv, *attn, *gate_up, *act;
};

// How the persistent kernel tiles one GEMM: weight rows per tile (the MMA N dimension) and K splits.
// A cost model in microseconds, fitted to the kernel's own per-phase timestamps on B200. What bounds a streaming CTA
// is its TMA unit (about 0.19 us per tiled copy whatever its size, two copies per ring stage) and the bytes the ring
// keeps under way, not the tensor pipe (a tcgen05.mma with M = 128 takes (128 + N) / 4 cycles of operand fetch,
// 48-64 cycles here): a 64-wide K block costs max(0.2 us, its bytes at 80 GB/s), a wave of work items pays ~1.5 us
// of pipeline fill, every K split costs ~0.3 us in the phase that sums the partial tiles, and a separate SiLU*up
// reduce phase costs ~5 us (one more grid barrier).
struct Tiling {
  int tile_n = 256, splits = 1;
  bool swiglu_direct = false;
  double cost = 1e30;
};

Tiling choose_tiling(int N, int K, int ctas, bool swiglu, int bn = 64) {
  Tiling best;
  const int nkb = K / 64;
  for (int direct = swiglu ? 1 : 0; direct >= 0; --direct) {
    for (int tn : {256, 128, 96, 64}) {
      // 96 rows (48 gate + 48 up channels) only for the fused SwiGLU epilogue: partial tiles are a power of two wide
      if (tn == 96 && (!direct || N % 96 != 0)) continue;
      const int tiles = (N + tn - 1) / tn;
      const int smax = direct ? 1 : std::min(8, nkb);
      for (int S = 1; S <= smax; ++S) {
        const int items = tiles * S, waves = (items + ctas - 1) / ctas, kb = (nkb + S - 1) / S;
        static const double tune[4] = {0.20, 80000.0, 1.5, 0.30};  // us floor per k-block, bytes per us, us per wave, us per split
        const double per_kb = std::max(tune[0], (tn * 128.0 + bn * 128.0) / tune[1]);  // weight + activation bytes
        double cost = waves * (kb * per_kb + tune[2]) + tune[3] * S;
        if (swiglu && !direct) cost += 5.0;
        if (cost < best.cost - 1e-9) best = Tiling{tn, S, direct != 0, cost};
      }
    }
  }
  return best;
}

}  // namespace
}  // namespace omni

using namespace omni;

struct omni_seq {
  std::vector<int32_t> pages;
  int32_t line = -1;
  int32_t prompt = 0, frames = 0, cap = 0;
  uint64_t seed = 0;
  bool live = false;
  omni_codec_stream* audio = nullptr;  // the sequence's slot in the attached codec decoder
};

constexpr int kTraceMaxPhases = 1024;

struct omni_talker {
  omni_talker_config cfg;
  int device = 0, sm_count = 148;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  std::string error;
  std::vector<void*> allocations;
  int64_t weight_bytes = 0, kv_bytes = 0;

  // weights
  StackW talker, pred;
  bf16 *text_emb = nullptr, *codec_emb = nullptr, *codec_head = nullptr;
  bf16 *fc1_w = nullptr, *fc1_b = nullptr, *fc2_w = nullptr, *fc2_b = nullptr, *mtp_w = nullptr, *mtp_b = nullptr;
  bf16 *p_emb = nullptr, *lm_heads = nullptr;
  bf16* p_emb_proj = nullptr;  // p_emb's rows sent through small_to_mtp_projection at load: [(groups - 1) * PV, p]
  bf16* p_qkv0 = nullptr;      // ... then through the predictor's first norm and q|k|v projection: [(groups - 1) * PV, qkv width]
  int text_vocab = 0;

  // pools
  int max_seqs = 0, max_rows = 0, pages_total = 0, page_table = 0;
  std::vector<bf16*> kv, pkv;  // per layer
  std::vector<int32_t> free_pages;
  std::vector<int32_t> free_lines;
  int pages_used = 0;
  char* seq_state = nullptr;
  int64_t seq_stride = 0;
  int seen_words = 0;
  omni_seq pad;
  std::vector<std::unique_ptr<omni_seq>> seqs;

  // staged inputs: one host (pinned) block mirrored on the device
  struct Inputs {
    size_t lines, pos, force, uniforms, indptr, d_pos, d_slot, pages;  // front block: every graph call
    size_t t_ids, t_codec, t_pos, t_slot, t_seq, last_row;             // prefill only
    size_t front_fixed_bytes, total_bytes;
  } in;
  char* in_host = nullptr;
  char* in_dev = nullptr;
  template <typename T>
  T* hin(size_t off) { return reinterpret_cast<T*>(in_host + off); }
  template <typename T>
  T* din(size_t off) { return reinterpret_cast<T*>(in_dev + off); }

  // activations and outputs
  Scratch T, P;
  bf16 *t_e = nullptr, *t_p = nullptr, *embeds = nullptr, *hidden = nullptr, *pad_embed = nullptr;
  bf16 *p_in = nullptr, *p_h = nullptr, *p_last = nullptr;
  bf16 *logits = nullptr, *p_logits = nullptr;
  int32_t* codes = nullptr;  // [max_seqs * 16] then the device error word
  uint32_t* err = nullptr;
  int32_t* out_host = nullptr;  // pinned mirror of `codes` + error word
  GemmScratch gemm_scratch;

  std::map<std::tuple<const void*, const void*, const void*, int, int>, TcGemmPlan> plans;
  std::map<std::pair<int, int>, cudaGraphExec_t> graphs;  // (program, bucket)
  std::map<std::pair<int, int>, int> graph_nodes;           // kernel nodes of each captured graph
  // the persistent tick kernel: one compiled phase list per (program, bucket)
  bool tick_ok = false;
  int tick_ctas = 0;
  uint32_t* tick_barrier = nullptr;
  uint32_t tick_barrier_base = 0;  // arrivals left in the counter by earlier launches
  // the code predictor's sub-steps as one launch of thread-block clusters (predictor.h): clusters that can be
  // resident at once (0: this device or shape cannot run it), one compiled entry list per bucket, exchange buffer
  int pred_clusters = 0;
  std::map<int, PredProgram> pred_programs;
  float* pred_vbuf = nullptr;
  unsigned long long* pred_trace = nullptr;
  const PredProgram* pred_trace_program = nullptr;
  std::map<std::pair<int, int>, TickProgram> tick_programs;
  int launches = 0, tick_phases = 0;
  std::string trace_path;  // omni_talker_trace: where the per-phase device timestamps of a tick are written
  unsigned long long* trace = nullptr;
  const TickProgram* trace_program = nullptr;
  omni_stats stats{};
  int last_n = 0;
  // omni_talker_step_begin / _end: up to two decode steps under way, each with its own pinned staging and read-back
  // blocks and events (the host prepares step t + 1 while the device runs step t)
  struct Flight {
    char* in_host = nullptr;
    int32_t* out_host = nullptr;
    cudaEvent_t start = nullptr, done = nullptr;
    int n = 0, launches = 0;
    std::vector<omni_seq*> seqs;  // with a codec decoder attached: whose frames these are
  } flight[2];
  int flight_first = 0, in_flight = 0;
  // the codec decoder that turns every frame into samples (omni_talker_attach_codec), or null: `wav` is zero-filled
  omni_codec* codec = nullptr;
  std::vector<float> wav_scratch;
  std::vector<omni_codec_stream*> audio_rows;

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

namespace {

#define CUDA_TRY(m, expr)                                                                      \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    if (e_ != cudaSuccess) return (m)->fail(OMNI_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

template <typename T>
int dev_alloc(omni_talker* m, T** out, size_t count, bool zero = false) {
  void* p = nullptr;
  const size_t bytes = std::max<size_t>(count * sizeof(T), 256);
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return m->fail(OMNI_ERR_CUDA, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
  if (zero) cudaMemset(p, 0, bytes);
  m->allocations.push_back(p);
  *out = static_cast<T*>(p);
  return OMNI_OK;
}

struct TensorIndex {
  std::unordered_map<std::string, const omni_tensor*> by_name;
  const omni_tensor* find(const std::string& n) const {
    auto it = by_name.find(n);
    return it == by_name.end() ? nullptr : it->second;
  }
};

// Copies one checkpoint tensor (rounded to bf16) to `dst`; shape must match.
int upload(omni_talker* m, const TensorIndex& idx, const std::string& name, std::initializer_list<int64_t> shape,
           bf16* dst) {
  const omni_tensor* t = idx.find(name);
  if (!t) return m->fail(OMNI_ERR_MISSING_TENSOR, "missing tensor %s", name.c_str());
  if (t->ndim != (int)shape.size()) return m->fail(OMNI_ERR_MISSING_TENSOR, "%s: rank %d", name.c_str(), t->ndim);
  int64_t count = 1;
  int d = 0;
  for (int64_t s : shape) {
    if (t->shape[d] != s)
      return m->fail(OMNI_ERR_MISSING_TENSOR, "%s: dim %d is %lld, expected %lld", name.c_str(), d,
                     (long long)t->shape[d], (long long)s);
    count *= s;
    ++d;
  }
  if (t->location == OMNI_DEVICE) {
    if (t->dtype == OMNI_BF16) {
      CUDA_TRY(m, cudaMemcpyAsync(dst, t->data, count * 2, cudaMemcpyDeviceToDevice, m->stream));
    } else {
      f32_to_bf16_kernel<<<(unsigned)((count + 255) / 256), 256, 0, m->stream>>>((const float*)t->data, dst, count);
      CUDA_TRY(m, cudaGetLastError());
    }
  } else if (t->dtype == OMNI_BF16) {
    CUDA_TRY(m, cudaMemcpy(dst, t->data, count * 2, cudaMemcpyHostToDevice));
  } else {
    std::vector<uint16_t> tmp(count);
    const float* src = (const float*)t->data;
    for (int64_t i = 0; i < count; ++i) tmp[i] = host_f2bf(src[i]);
    CUDA_TRY(m, cudaMemcpy(dst, tmp.data(), count * 2, cudaMemcpyHostToDevice));
  }
  m->weight_bytes += count * 2;
  return OMNI_OK;
}

#define TRY(expr)              \
  do {                         \
    int rc_ = (expr);          \
    if (rc_ != OMNI_OK) return rc_; \
  } while (0)

// `Stack::load` (crates/omni-qwen3/src/stack.rs:93-141): Q|K|V rows and
// gate|up rows fused into one weight each.
int load_stack(omni_talker* m, const TensorIndex& idx, const std::string& prefix, const omni_stack_config& c,
               StackW* out) {
  out->cfg = c;
  // gate and up channels are interleaved in groups of half the tile the persistent kernel will use for this GEMM
  out->granule = choose_tiling(2 * c.inter, c.hidden, std::max(1, m->tick_ctas > 0 ? m->tick_ctas : 148), true).tile_n / 2;
  if (c.inter % out->granule) out->granule = 64;
  const int64_t h = c.hidden, d = c.head_dim, q = (int64_t)c.q_heads * d, kv = (int64_t)c.kv_heads * d, I = c.inter;
  out->layers.resize(c.layers);
  for (int i = 0; i < c.layers; ++i) {
    const std::string p = prefix + ".layers." + std::to_string(i) + ".";
    StackW::Layer& L = out->layers[i];
    TRY(dev_alloc(m, &L.ln1, h));
    TRY(dev_alloc(m, &L.qkv, (q + 2 * kv) * h));
    TRY(dev_alloc(m, &L.q_norm, d));
    TRY(dev_alloc(m, &L.k_norm, d));
    TRY(dev_alloc(m, &L.o, h * q));
    TRY(dev_alloc(m, &L.ln2, h));
    TRY(dev_alloc(m, &L.gate_up, 2 * I * h));
    TRY(dev_alloc(m, &L.down, h * I));
    TRY(upload(m, idx, p + "input_layernorm.weight", {h}, L.ln1));
    TRY(upload(m, idx, p + "self_attn.q_proj.weight", {q, h}, L.qkv));
    TRY(upload(m, idx, p + "self_attn.k_proj.weight", {kv, h}, L.qkv + q * h));
    TRY(upload(m, idx, p + "self_attn.v_proj.weight", {kv, h}, L.qkv + (q + kv) * h));
    TRY(upload(m, idx, p + "self_attn.q_norm.weight", {d}, L.q_norm));
    TRY(upload(m, idx, p + "self_attn.k_norm.weight", {d}, L.k_norm));
    TRY(upload(m, idx, p + "self_attn.o_proj.weight", {h, q}, L.o));
    TRY(upload(m, idx, p + "post_attention_layernorm.weight", {h}, L.ln2));
    {
      bf16* fused = nullptr;  // [gate; up] as in the checkpoint, then regrouped (see interleave_gate_up_kernel)
      CUDA_TRY(m, cudaMalloc((void**)&fused, (size_t)2 * I * h * sizeof(bf16)));
      int rc = upload(m, idx, p + "mlp.gate_proj.weight", {I, h}, fused);
      if (rc == OMNI_OK) rc = upload(m, idx, p + "mlp.up_proj.weight", {I, h}, fused + I * h);
      if (rc == OMNI_OK) {
        const int64_t pieces = 2 * I * (h / 8);
        interleave_gate_up_kernel<<<(unsigned)((pieces + 255) / 256), 256, 0, m->stream>>>(fused, L.gate_up, (int)I, (int)h,
                                                                                     out->granule);
        if (cudaStreamSynchronize(m->stream) != cudaSuccess) rc = m->fail(OMNI_ERR_CUDA, "gate|up regroup failed");
      }
      cudaFree(fused);
      TRY(rc);
    }
    TRY(upload(m, idx, p + "mlp.down_proj.weight", {h, I}, L.down));
  }
  TRY(dev_alloc(m, &out->norm, h));
  TRY(upload(m, idx, prefix + ".norm.weight", {h}, out->norm));
  return OMNI_OK;
}

int alloc_scratch(omni_talker* m, const StackW& s, int rows, Scratch* out) {
  const omni_stack_config& c = s.cfg;
  TRY(dev_alloc(m, &out->x, (size_t)rows * c.hidden));
  TRY(dev_alloc(m, &out->res, (size_t)rows * c.hidden));
  TRY(dev_alloc(m, &out->qkv, (size_t)rows * s.qkv_width()));
  TRY(dev_alloc(m, &out->attn, (size_t)rows * c.q_heads * c.head_dim));
  TRY(dev_alloc(m, &out->gate_up, (size_t)rows * 2 * c.inter));
  TRY(dev_alloc(m, &out->act, (size_t)rows * c.inter));
  return OMNI_OK;
}

// ---- launching ---------------------------------------------------------------------

#define LAUNCH(m, expr)                                                                        \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    ++(m)->launches;                                                                           \
    if (e_ != cudaSuccess) return (m)->fail(OMNI_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

// y[rows, N] = x[rows, K] . w[N, K]^T on the path the row count calls for.
int gemm(omni_talker* m, const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy, Epilogue epi = {}) {
  const bool vector_path = m->cfg.gemm_path == 1 || rows <= 8 || !tc_supports(N, K, rows);
  if (vector_path) {
    LAUNCH(m, gemv_launch(w, N, K, x, rows, y, ldy, epi, m->sm_count, m->stream));
    return OMNI_OK;
  }
  const auto key = std::make_tuple((const void*)w, (const void*)x, (const void*)y, rows, epi.kind);
  auto it = m->plans.find(key);
  if (it == m->plans.end()) {
    TcGemmPlan plan;
    const int rc = tc_plan(&plan, w, N, K, x, rows, y, ldy, epi, m->sm_count);
    if (rc != 0) return m->fail(OMNI_ERR_CUDA, "tensor-map encode failed (%d) for N=%d K=%d rows=%d", rc, N, K, rows);
    if (plan.partial_floats() > m->gemm_scratch.partial_floats ||
        plan.tiles_n() * plan.row_tiles > m->gemm_scratch.counter_slots)
      return m->fail(OMNI_ERR_UNSUPPORTED, "split-K scratch too small for N=%d K=%d rows=%d", N, K, rows);
    it = m->plans.emplace(key, plan).first;
  }
  LAUNCH(m, tc_launch(it->second, m->gemm_scratch, m->err, m->stream));
  return OMNI_OK;
}

// One pass of a decoder stack: op order of `Stack::forward`
// (crates/omni-qwen3/src/stack.rs:152-203).
int stack_forward(omni_talker* m, const StackW& S, const Scratch& s, const bf16* input, int rows, const RowMap& map,
                  const std::vector<bf16*>& kv, int kv_pages, bf16* keep_out, int every, int which) {
  const omni_stack_config& c = S.cfg;
  const int h = c.hidden, I = c.inter, qd = c.q_heads * c.head_dim;
  const AttnShape a = S.attn();
  LAUNCH(m, launch_norm_copy(input, S.layers[0].ln1, s.x, s.res, rows, h, c.rms_eps, m->stream));
  for (int i = 0; i < c.layers; ++i) {
    const StackW::Layer& L = S.layers[i];
    TRY(gemm(m, L.qkv, S.qkv_width(), h, s.x, rows, s.qkv, S.qkv_width()));
    LAUNCH(m, launch_rope_kv(s.qkv, L.q_norm, L.k_norm, kv[i], map, rows, a, kv_pages, m->err, m->stream));
    LAUNCH(m, launch_attend(s.qkv, kv[i], s.attn, map, rows, a, m->err, m->stream));
    TRY(gemm(m, L.o, h, qd, s.attn, rows, s.x, h));
    LAUNCH(m, launch_add_norm(s.x, s.res, L.ln2, s.x, rows, h, c.rms_eps, 1, 0, m->stream));
    TRY(gemm(m, L.gate_up, 2 * I, h, s.x, rows, s.gate_up, 2 * I));
    LAUNCH(m, launch_silu_mul(s.gate_up, s.act, rows, I, S.granule, m->stream));
    TRY(gemm(m, L.down, h, I, s.act, rows, s.x, h));
    if (i + 1 < c.layers)
      LAUNCH(m, launch_add_norm(s.x, s.res, S.layers[i + 1].ln1, s.x, rows, h, c.rms_eps, 1, 0, m->stream));
    else
      LAUNCH(m, launch_add_norm(s.x, s.res, S.norm, keep_out, rows, h, c.rms_eps, every, which, m->stream));
  }
  return OMNI_OK;
}

SlotState slots(omni_talker* m) { return SlotState{m->seq_state, m->din<int32_t>(m->in.lines), m->seq_stride}; }

// `Talker::sample` (crates/omni-qwen3-tts/src/talker.rs:254-290).
int sample(omni_talker* m, int group, const bf16* logits, int rows) {
  const omni_talker_config& c = m->cfg;
  SampleParams p{};
  p.group = group;
  p.top_p = c.top_p;
  p.philox = c.sampler == OMNI_SAMPLER_PHILOX;
  p.seen_words = m->seen_words;
  if (group == 0) {
    p.vocab = c.talker.vocab;
    p.temperature = c.temperature;
    p.top_k = c.top_k;
    p.penalty = c.repetition_penalty;
    p.suppress_lo = c.talker.vocab - c.control_tokens;
    p.suppress_hi = c.talker.vocab;
    p.exempt = c.codec_eos_token_id;
    p.min_frames = c.min_frames;
    p.penalize = 1;
  } else {
    p.vocab = c.predictor.vocab;
    p.temperature = c.sub_temperature;
    p.top_k = c.sub_top_k;
    p.penalty = 1.f;
    p.suppress_lo = p.suppress_hi = 0;
    p.exempt = -1;
    p.min_frames = 0;
    p.penalize = 0;
  }
  LAUNCH(m, launch_sample(logits, p, m->din<int32_t>(m->in.pos), m->din<float>(m->in.uniforms),
                          m->din<int32_t>(m->in.force), slots(m), m->codes, rows, m->stream));
  return OMNI_OK;
}

// `Talker::advance` (talker.rs:224-251): the last frame's embedding through the talker.
int enqueue_advance(omni_talker* m, int b) {
  const omni_talker_config& c = m->cfg;
  const int h = c.talker.hidden;
  LAUNCH(m, launch_frame_embed(slots(m), m->pad_embed, m->codec_emb, c.talker.vocab, m->p_emb, c.predictor.vocab,
                               c.groups, m->t_e, b, h, m->err, m->stream));
  RowMap map;
  map.pos = m->din<int32_t>(m->in.d_pos);
  map.slot = m->din<int32_t>(m->in.d_slot);
  map.seq = nullptr;
  map.indptr = m->din<int32_t>(m->in.indptr);
  map.pages = m->din<int32_t>(m->in.pages);
  return stack_forward(m, m->talker, m->T, m->t_e, b, map, m->kv, m->pages_total, m->hidden, 1, 0);
}

// `Talker::tail` (talker.rs:293-356).
int enqueue_tail(omni_talker* m, int b) {
  const omni_talker_config& c = m->cfg;
  const int h = c.talker.hidden, p = c.predictor.hidden, V = c.talker.vocab, PV = c.predictor.vocab;
  TRY(gemm(m, m->codec_head, V, h, m->hidden, b, m->logits, V));
  TRY(sample(m, 0, m->logits, b));
  LAUNCH(m, launch_pred_input(m->hidden, m->codec_emb, V, m->codes, m->p_in, b, h, m->err, m->stream));
  Epilogue bias;
  bias.bias = m->mtp_b;
  bias.kind = kEpiBias;
  for (int g = 1; g < c.groups; ++g) {
    const int per = g == 1 ? 2 : 1, rows = b * per;
    if (g > 1)
      LAUNCH(m, launch_gather(m->codes + (g - 1), OMNI_GROUPS, m->p_emb + (size_t)(g - 2) * PV * h, PV, m->p_in, b, h,
                              m->err, m->stream));
    TRY(gemm(m, m->mtp_w, p, h, m->p_in, rows, m->p_h, p, bias));
    RowMap map;
    map.per = per;
    map.base = g == 1 ? 0 : g;
    TRY(stack_forward(m, m->pred, m->P, m->p_h, rows, map, m->pkv, m->max_seqs, m->p_last, per, per - 1));
    bf16* lg = m->p_logits + (size_t)(g - 1) * m->max_seqs * PV;
    TRY(gemm(m, m->lm_heads + (size_t)(g - 1) * PV * p, PV, p, m->p_last, b, lg, PV));
    TRY(sample(m, g, lg, b));
  }
  return OMNI_OK;
}

enum Program { kFirst = 0, kDecode = 1 };

int enqueue_program(omni_talker* m, int program, int b) {
  if (program == kDecode) TRY(enqueue_advance(m, b));
  return enqueue_tail(m, b);
}


// ---- the persistent tick kernel's phase list ------------------------------------------------------------------

int pick_bn(int rows) { return rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : rows <= 128 ? 128 : 256; }

struct TickBuilder {
  omni_talker* m;
  TickProgram* prog;
  int ctas;
  int offset = 0;  // CTA the next phase's first item lands on, so consecutive phases load different SMs first
  std::map<std::tuple<const void*, int, int, int, int>, int> map_cache;
  bool failed = false;

  int map_of(const bf16* base, int rows, int K, int box, int kbs) {
    const auto key = std::make_tuple((const void*)base, rows, K, box, kbs);
    auto it = map_cache.find(key);
    if (it != map_cache.end()) return it->second;
    const int idx = tick_add_map(prog, base, rows, K, box, kbs);
    if (idx < 0) failed = true;
    map_cache[key] = idx;
    return idx;
  }

  Phase blank(int type, int rows) {
    Phase ph;
    memset(&ph, 0, sizeof(ph));
    ph.type = type;
    ph.rows = rows;
    ph.cta_offset = offset;
    return ph;
  }

  // k-blocks per ring stage. A tiled TMA copy occupies the SM's TMA unit for about 0.19 us whatever its size and a
  // stage is two copies, so one k-block per stage (16-24 KB) caps a CTA near 45 GB/s; several k-blocks per copy lift
  // that. The most (up to 4) that divide a work item's k-blocks and still leave two stages in the ring measured best.
  int stage_kblocks(int nkb, int splits, int bn, int tile_n) const {
    const int cap = 4;
    if (nkb % splits) return 1;
    const int per = nkb / splits, ring = tick_ring_size();
    int best = 1;
    for (int kbs = 2; kbs <= std::min(cap, per); ++kbs)
      if (per % kbs == 0 && ring / (kbs * (bn + tile_n) * 128) >= 2) best = kbs;
    return best;
  }

  // y = x . w^T as f32 partial tiles (or, for gate|up, SwiGLU activations straight from the epilogue when the
  // cost model prefers no K split); returns the phase so the consumer knows tiles / splits / bn / tile_n.
  Phase gemm(const bf16* w, int N, int K, const bf16* x, int rows, bool swiglu = false, bf16* act = nullptr,
             int inter = 0, int granule = 0) {
    Phase ph = blank(kPhGemm, rows);
    // (the model's constants were fitted at 64 rows; taller activation tiles count their bytes, shorter ones measured
    // better with the 64-row figure)
    Tiling t = choose_tiling(N, K, ctas, swiglu, std::max(64, pick_bn(rows)));
    if (swiglu && t.tile_n != 2 * granule) {  // the weights were regrouped for another tile width: keep that one
      t.tile_n = 2 * granule;
      if (t.swiglu_direct) t.splits = 1;
    }
    if (swiglu && t.tile_n == 96) t.swiglu_direct = true, t.splits = 1;  // no partial tiles of that width
    ph.N = N;
    ph.K = K;
    ph.bn = pick_bn(rows);
    ph.tile_n = t.tile_n;
    ph.tiles = (N + t.tile_n - 1) / t.tile_n;
    ph.splits = t.splits;
    ph.mode = swiglu && t.swiglu_direct ? kGemmSwiglu : kGemmPartials;
    ph.i1 = stage_kblocks(K / 64, ph.splits, ph.bn, ph.tile_n);
    ph.wmap = map_of(w, N, K, t.tile_n, ph.i1);
    ph.xmap = map_of(x, rows, K, ph.bn, ph.i1);
    ph.dst0 = act;
    ph.i0 = inter;
    prog->phases.push_back(ph);
    prog->max_bn = std::max(prog->max_bn, ph.bn);
    if (ph.mode == kGemmPartials)
      prog->partial_floats = std::max(prog->partial_floats, (size_t)ph.splits * ph.tiles * ph.bn * ph.tile_n);
    offset = (offset + ph.tiles * ph.splits) % ctas;
    if (swiglu && ph.mode == kGemmPartials) {  // SiLU*up over the summed partial tiles
      Phase rs = blank(kPhReduceSilu, rows);
      rs.tiles = ph.tiles, rs.splits = ph.splits, rs.bn = ph.bn, rs.tile_n = ph.tile_n;
      rs.dst0 = act;
      rs.i0 = inter;
      prog->phases.push_back(rs);
    }
    return ph;
  }

  void row_phase(int type, const Phase& src, int rows, int dim, const bf16* bias, const bf16* gain, bf16* res, bf16* out,
                 float eps, int every = 1, int which = 0) {
    Phase ph = blank(type, rows);
    ph.N = dim;
    ph.tiles = src.tiles;
    ph.splits = src.splits;
    ph.bn = src.bn;
    ph.tile_n = src.tile_n;
    ph.src0 = bias;
    ph.src3 = gain;
    ph.dst0 = res;
    ph.dst1 = out;
    ph.f0 = eps;
    ph.i0 = every;
    ph.i1 = which;
    prog->phases.push_back(ph);
  }

  // One pass of a decoder stack over rows whose normalised input is already in s.x and residual in s.res:
  // `Stack::forward` (crates/omni-qwen3/src/stack.rs:152-203) with the reduce of every split-K GEMM folded into its
  // consumer and SiLU*up folded into the gate|up GEMM.
  // qkv0_table (optional): the first layer's q | k | v of every row, looked up by the code of group `code_group` (see
  // p_qkv0); that layer then has no q|k|v GEMM phase.
  void stack_pass(const StackW& S, const Scratch& s, int rows, bool paged, int per, int base,
                  const std::vector<bf16*>& kv, int kv_pages, bf16* keep_out, int every, int which,
                  const bf16* qkv0_table = nullptr, int code_group = 0) {
    const omni_stack_config& c = S.cfg;
    const int h = c.hidden, I = c.inter, qd = c.q_heads * c.head_dim;
    for (int i = 0; i < c.layers; ++i) {
      const StackW::Layer& L = S.layers[i];
      const bool looked_up = i == 0 && qkv0_table != nullptr;
      const Phase qkv = looked_up ? blank(kPhGemm, rows) : gemm(L.qkv, S.qkv_width(), h, s.x, rows);
      Phase at = blank(kPhRopeAttn, rows);
      at.tiles = qkv.tiles, at.splits = qkv.splits, at.bn = qkv.bn, at.tile_n = qkv.tile_n;
      if (looked_up) {
        at.tiles = 1, at.splits = 1, at.bn = 64, at.tile_n = 64;  // unused: nothing is read from the partial tiles
        at.src2 = qkv0_table, at.i7 = code_group, at.i8 = S.qkv_width();
      }
      at.i0 = c.q_heads, at.i1 = c.kv_heads, at.i2 = c.head_dim, at.i3 = per, at.i4 = base, at.i5 = paged, at.i6 = kv_pages;
      at.src0 = L.q_norm, at.src1 = L.k_norm;
      at.dst0 = kv[i], at.dst1 = s.attn;
      at.f0 = c.rms_eps, at.f1 = c.rope_theta;
      prog->phases.push_back(at);
      const Phase o = gemm(L.o, h, qd, s.attn, rows);
      row_phase(kPhAddNorm, o, rows, h, nullptr, L.ln2, s.res, s.x, c.rms_eps);
      gemm(L.gate_up, 2 * I, h, s.x, rows, true, s.act, I, S.granule);
      const Phase down = gemm(L.down, h, I, s.act, rows);
      if (i + 1 < c.layers)
        row_phase(kPhAddNorm, down, rows, h, nullptr, S.layers[i + 1].ln1, s.res, s.x, c.rms_eps);
      else
        row_phase(kPhAddNorm, down, rows, h, nullptr, S.norm, s.res, keep_out, c.rms_eps, every, which);
    }
  }

  void sample(const Phase& head, int group, int rows, bf16* logits_out, int ldl, int next, const bf16* table,
              const bf16* hidden, bf16* p_in, int dim, const bf16* gain = nullptr, float eps = 0.f, bf16* normed = nullptr) {
    const omni_talker_config& c = m->cfg;
    Phase ph = blank(kPhSample, rows);
    ph.tiles = head.tiles, ph.splits = head.splits, ph.bn = head.bn, ph.tile_n = head.tile_n;
    ph.dst0 = logits_out;
    ph.i0 = ldl;
    ph.f1 = c.top_p;
    ph.i7 = group;
    ph.i10 = c.sampler == OMNI_SAMPLER_PHILOX;
    if (group == 0) {
      ph.N = c.talker.vocab;
      ph.f0 = c.temperature, ph.f2 = c.repetition_penalty;
      ph.i1 = c.top_k, ph.i2 = c.talker.vocab - c.control_tokens, ph.i3 = c.talker.vocab;
      ph.i4 = c.codec_eos_token_id, ph.i5 = c.min_frames, ph.i6 = 1;
    } else {
      ph.N = c.predictor.vocab;
      ph.f0 = c.sub_temperature, ph.f2 = 1.f;
      ph.i1 = c.sub_top_k, ph.i2 = 0, ph.i3 = 0, ph.i4 = -1, ph.i5 = 0, ph.i6 = 0;
    }
    ph.i8 = next;
    ph.src0 = table;
    ph.src1 = hidden;
    ph.dst1 = p_in;
    ph.i9 = dim;
    ph.src3 = gain, ph.f3 = eps, ph.dst2 = normed;  // kNextProjected only
    prog->phases.push_back(ph);
    offset = (offset + rows) % ctas;
  }

  // `Talker::advance` + `Talker::tail` (talker.rs:224-251, 293-356) at bucket b. with_predictor = false: the list ends
  // with the first codebook's draw (which also writes the predictor's two input rows); the cluster kernel does the rest.
  void build(int program, int b, bool with_predictor = true) {
    const omni_talker_config& c = m->cfg;
    const int h = c.talker.hidden, p = c.predictor.hidden, V = c.talker.vocab, PV = c.predictor.vocab;
    if (program == kDecode) {
      Phase e = blank(kPhEmbedNorm, b);
      e.N = h;
      e.src0 = m->pad_embed, e.src1 = m->codec_emb, e.src2 = m->p_emb, e.src3 = m->talker.layers[0].ln1;
      e.dst0 = m->T.res, e.dst1 = m->T.x;
      e.i0 = V, e.i1 = PV, e.i2 = c.groups;
      e.f0 = c.talker.rms_eps;
      prog->phases.push_back(e);
      stack_pass(m->talker, m->T, b, true, 1, 0, m->kv, m->pages_total, m->hidden, 1, 0);
    }
    const Phase head = gemm(m->codec_head, V, h, m->hidden, b);
    sample(head, 0, b, m->logits, V, kNextHiddenAndCode, m->codec_emb, m->hidden, m->p_in, h);
    // From the second predictor pass on, a pass's one input row per session is the embedding of the code just drawn,
    // sent through the input projection (talker.rs:306-312). The projection of every table row was taken at load
    // (p_emb_proj), so the draw writes the pass's residual start and first normed row itself and the pass has no
    // projection GEMM and no ReduceNorm phase. The first pass (two rows per session, one of them the talker's
    // hidden state) keeps both.
    const bool folded = m->p_emb_proj != nullptr && (p == 128 || p == 256 || p == 512 || p == 1024 || p == 2048);
    for (int g = 1; g < c.groups && with_predictor; ++g) {
      const int per = g == 1 ? 2 : 1, rows = b * per;
      if (g == 1 || !folded) {
        const Phase mtp = gemm(m->mtp_w, p, h, m->p_in, rows);
        row_phase(kPhReduceNorm, mtp, rows, p, m->mtp_b, m->pred.layers[0].ln1, m->P.res, m->P.x, c.predictor.rms_eps);
      }
      const bool qkv_folded = folded && g >= 2 && m->p_qkv0 != nullptr;
      stack_pass(m->pred, m->P, rows, false, per, g == 1 ? 0 : g, m->pkv, m->max_seqs, m->p_last, per, per - 1,
                 qkv_folded ? m->p_qkv0 + (size_t)(g - 2) * PV * m->pred.qkv_width() : nullptr, g - 1);
      const Phase ph = gemm(m->lm_heads + (size_t)(g - 1) * PV * p, PV, p, m->p_last, b);
      const bool more = g + 1 < c.groups;
      bf16* lg = m->p_logits + (size_t)(g - 1) * m->max_seqs * PV;
      if (more && folded) {
        sample(ph, g, b, lg, PV, kNextProjected, m->p_emb_proj + (size_t)(g - 1) * PV * p, nullptr, m->P.res, p,
               m->pred.layers[0].ln1, c.predictor.rms_eps, m->P.x);
        if (m->p_qkv0) {  // the row the next pass's first attention phase will read
          Phase& sp = prog->phases.back();
          sp.src1 = m->p_qkv0 + (size_t)(g - 1) * PV * m->pred.qkv_width();
          sp.i11 = m->pred.qkv_width() * (int)sizeof(bf16);
        }
      }
      else {
        sample(ph, g, b, lg, PV, more ? kNextCode : kNextNone, more ? m->p_emb + (size_t)(g - 1) * PV * h : nullptr,
               nullptr, m->p_in, h);
      }
    }
  }
};

// ---- the cluster predictor kernel's entry list ----------------------------------------------------------------

// Sessions per cluster and clusters for bucket b (0 clusters: the bucket does not fit the resident clusters).
void pred_partition(const omni_talker* m, int b, int* per_cluster, int* clusters) {
  const int use = std::min(m->pred_clusters, b);
  *per_cluster = use > 0 ? (b + use - 1) / use : 0;
  *clusters = *per_cluster > 0 && *per_cluster <= kPredRows ? (b + *per_cluster - 1) / *per_cluster : 0;
}

bool pred_shape_ok(const omni_talker_config& c, int granule) {
  const omni_stack_config &t = c.talker, &p = c.predictor;
  const int C = p.q_heads;
  if (!(C == 2 || C == 4 || C == 8 || C == 16) || p.head_dim != 128 || 2 * p.kv_heads != C || p.hidden != 64 * C) return false;
  if ((2 * p.inter) % (C * 128) != 0 || !(granule == 32 || granule == 64)) return false;
  const int per = p.vocab / C;
  if (p.vocab % C || !(per == 64 || per % 128 == 0) || p.vocab % 16 || p.vocab > 4096) return false;
  if (t.hidden % 64 || p.hidden % 128 || p.inter % 64) return false;
  return c.groups >= 2;
}

bool pred_usable(const omni_talker* m, int b) {
  if (m->pred_clusters <= 0) return false;
  int per = 0, clusters = 0;
  pred_partition(m, b, &per, &clusters);
  return clusters > 0;
}

struct PredBuilder {
  omni_talker* m;
  PredProgram* prog;
  std::map<std::tuple<const void*, int64_t, int, int64_t, int, int>, int> map_cache;
  bool failed = false;
  int bars = 0;  // cluster barriers the kernel passes before the next entry

  int map_of(const bf16* base, int64_t rows, int K, int64_t row_stride, int box_rows, int kbs) {
    const auto key = std::make_tuple((const void*)base, rows, K, row_stride, box_rows, kbs);
    auto it = map_cache.find(key);
    if (it != map_cache.end()) return it->second;
    const int idx = pred_add_map(prog, base, rows, K, row_stride, box_rows, kbs);
    if (idx < 0) failed = true;
    map_cache[key] = idx;
    return idx;
  }
  static int stage_kblocks(int nkb, int cap) {
    for (int k = cap; k > 1; --k)
      if (nkb % k == 0) return k;
    return 1;
  }

  // One box of `rows` weight rows of w [n, K]; x: the activation rows read through TMA (nullptr: the resident tile).
  PredEntry& box(int epi, const bf16* w, int64_t n, int K, int rows, int wrow, int cta_stride, const bf16* x, int x_cols,
                 int64_t x_stride, int xz0) {
    PredEntry e;
    memset(&e, 0, sizeof(e));
    e.epi = epi;
    e.rows = rows;
    e.nkb = K / 64;
    e.kbs = stage_kblocks(e.nkb, rows == 64 ? 4 : 2);
    e.wmap = map_of(w, n, K, K, rows, e.kbs);
    e.w = w;
    e.wrow = wrow;
    e.cta_stride = cta_stride;
    e.xmap = x ? map_of(x, m->max_seqs, x_cols, x_stride, kPredRows, e.kbs) : -1;
    e.xz0 = xz0;
    e.need_bars = bars;
    prog->entries.push_back(e);
    return prog->entries.back();
  }

  // The sub-steps at positions 0 .. groups-1 of the frame (`Talker::tail`, talker.rs:300-356): position 0 is the
  // talker's hidden row (no head), position j >= 1 the embedding of code j-1 followed by head j-1 and the draw of
  // code j. The reference runs positions 0 and 1 as one two-row pass; row by row the arithmetic is the same.
  void build(int b) {
    const omni_talker_config& c = m->cfg;
    const omni_stack_config& pc = c.predictor;
    const int h = c.talker.hidden, p = pc.hidden, PV = pc.vocab, C = pc.q_heads, I = pc.inter, qd = pc.q_heads * pc.head_dim;
    const StackW& S = m->pred;
    PredConfig& cfg = prog->cfg;
    cfg.C = C, cfg.hidden = p, cfg.q_heads = pc.q_heads, cfg.kv_heads = pc.kv_heads, cfg.inter = I, cfg.granule = S.granule;
    cfg.vocab = PV, cfg.next_stride = 2 * h;
    cfg.temperature = c.sub_temperature, cfg.top_p = c.top_p, cfg.top_k = c.sub_top_k;
    cfg.philox = c.sampler == OMNI_SAMPLER_PHILOX;
    prog->rows = b;
    pred_partition(m, b, &prog->per_cluster, &prog->clusters);
    for (int j = 0; j < c.groups; ++j) {
      {  // the input row through small_to_mtp_projection (talker.rs:306-312): p_in holds [hidden | code embedding] per session
        PredEntry& e = box(kPeBiasNorm, m->mtp_w, p, h, 64, 0, 64, m->p_in, 2 * h, 2 * h, j == 0 ? 0 : h / 64);
        e.p0 = m->mtp_b, e.p1 = S.layers[0].ln1, e.eps = pc.rms_eps, e.pos = j;
        bars += 1;
      }
      for (int i = 0; i < pc.layers; ++i) {
        const StackW::Layer& L = S.layers[i];
        {
          PredEntry& e = box(kPeQ, L.qkv, S.qkv_width(), p, 128, 0, 128, nullptr, 0, 0, 0);
          e.p0 = L.q_norm, e.eps = pc.rms_eps, e.theta = pc.rope_theta, e.pos = j;
        }
        {
          PredEntry& e = box(kPeKv, L.qkv, S.qkv_width(), p, 128, pc.q_heads * 128, 128, nullptr, 0, 0, 0);
          e.wrow2 = (pc.q_heads + pc.kv_heads) * 128;
          e.p0 = L.k_norm, e.q0 = m->pkv[i], e.q1 = m->P.attn, e.eps = pc.rms_eps, e.theta = pc.rope_theta, e.pos = j;
          bars += 2;
        }
        {
          PredEntry& e = box(kPeAddNorm, L.o, p, qd, 64, 0, 64, m->P.attn, qd, qd, 0);
          e.p1 = L.ln2, e.eps = pc.rms_eps, e.pos = j;
          bars += 1;
        }
        const int gu_rows = 2 * I / C, gu_boxes = gu_rows / 128;
        for (int bb = 0; bb < gu_boxes; ++bb) {
          PredEntry& e = box(kPeSwiglu, L.gate_up, 2 * I, p, 128, bb * 128, gu_rows, nullptr, 0, 0, 0);
          e.q0 = m->P.act, e.last = bb + 1 == gu_boxes, e.pos = j;
          if (e.last) bars += 1;
        }
        {
          PredEntry& e = box(kPeAddNorm, L.down, p, I, 64, 0, 64, m->P.act, I, I, 0);
          e.p1 = i + 1 < pc.layers ? S.layers[i + 1].ln1 : S.norm, e.eps = pc.rms_eps, e.pos = j;
          bars += 1;
        }
      }
      if (j == 0) continue;
      const int per = PV / C, hb = per == 64 ? 64 : 128, head_boxes = per / hb;
      for (int bb = 0; bb < head_boxes; ++bb) {
        PredEntry& e = box(kPeHead, m->lm_heads, (int64_t)(c.groups - 1) * PV, p, hb, (j - 1) * PV + bb * hb, per, nullptr, 0, 0, 0);
        e.col0 = bb * hb, e.group = j, e.pos = j, e.last = bb + 1 == head_boxes;
        e.q0 = m->p_logits + (size_t)(j - 1) * m->max_seqs * PV;
        if (e.last) {
          const bool more = j + 1 < c.groups;
          e.next_dim = more ? h : 0;
          e.p0 = more ? m->p_emb + (size_t)(j - 1) * PV * h : nullptr;
          e.q1 = m->p_in + h;  // the code-embedding half of a session's input row
          bars += 2;
        }
      }
    }
  }
};

bool tick_usable(const omni_talker* m, int b) {
  if (!m->tick_ok) return false;
  const omni_stack_config &t = m->cfg.talker, &p = m->cfg.predictor;
  auto ok = [&](const omni_stack_config& s) {
    return tick_supports(s.hidden, s.head_dim, s.q_heads, s.kv_heads, 2 * b) && s.inter % 64 == 0 && s.hidden % 64 == 0 &&
           (s.q_heads * s.head_dim) % 64 == 0;
  };
  // the draw phase reads the head's partial sums four columns at a time
  return ok(t) && ok(p) && t.vocab % 4 == 0 && p.vocab % 4 == 0;
}

int run_tick_program(omni_talker* m, int program, int b) {
  const bool clusters = pred_usable(m, b);  // the predictor's sub-steps run as a second launch of thread-block clusters
  auto key = std::make_pair(program, b);
  auto it = m->tick_programs.find(key);
  if (it == m->tick_programs.end()) {
    TickProgram prog;
    TickBuilder builder{m, &prog, m->tick_ctas};
    builder.build(program, b, !clusters);
    if (builder.failed) return m->fail(OMNI_ERR_CUDA, "tensor-map encode failed while compiling the tick program");
    if (prog.partial_floats > m->gemm_scratch.partial_floats)
      return m->fail(OMNI_ERR_UNSUPPORTED, "split-K scratch too small for the tick program");
    if (tick_upload(&prog) != 0) return m->fail(OMNI_ERR_CUDA, "uploading the tick program failed");
    it = m->tick_programs.emplace(key, prog).first;
  }
  TickIo io;
  io.lines = m->din<int32_t>(m->in.lines);
  io.frames = m->din<int32_t>(m->in.pos);
  io.uniforms = m->din<float>(m->in.uniforms);
  io.force = m->din<int32_t>(m->in.force);
  io.d_pos = m->din<int32_t>(m->in.d_pos);
  io.d_slot = m->din<int32_t>(m->in.d_slot);
  io.indptr = m->din<int32_t>(m->in.indptr);
  io.pages = m->din<int32_t>(m->in.pages);
  io.state = m->seq_state;
  io.stride = m->seq_stride;
  io.codes = m->codes;
  io.seen_words = m->seen_words;
  m->tick_phases = (int)it->second.phases.size();
  // (omni_talker_trace named a file: the per-phase device timestamps of the last tick of a call are written there)
  if (!m->trace_path.empty() && !m->trace) TRY(dev_alloc(m, &m->trace, (size_t)4 * kTraceMaxPhases * m->tick_ctas, true));
  if (m->trace && m->tick_phases <= kTraceMaxPhases) {
    m->trace_program = &it->second;
    CUDA_TRY(m, cudaMemsetAsync(m->trace, 0, (size_t)4 * kTraceMaxPhases * m->tick_ctas * 8, m->stream));
  }
  LAUNCH(m, tick_launch(it->second, io, m->gemm_scratch.partials, m->tick_barrier, &m->tick_barrier_base, m->err,
                        m->tick_ctas, m->stream,
                        m->trace && m->tick_phases <= kTraceMaxPhases ? m->trace : nullptr));
  if (clusters) {
    auto pit = m->pred_programs.find(b);
    if (pit == m->pred_programs.end()) {
      PredProgram prog;
      PredBuilder builder{m, &prog};
      builder.build(b);
      if (builder.failed) return m->fail(OMNI_ERR_CUDA, "tensor-map encode failed while compiling the predictor program");
      if (pred_upload(&prog) != 0) return m->fail(OMNI_ERR_CUDA, "uploading the predictor program failed");
      pit = m->pred_programs.emplace(b, prog).first;
    }
    if (!m->trace_path.empty() && !m->pred_trace) TRY(dev_alloc(m, &m->pred_trace, (size_t)3 * 4096, true));
    m->pred_trace_program = m->pred_trace ? &pit->second : nullptr;
    LAUNCH(m, pred_launch(pit->second, io, m->pred_vbuf, m->err, m->stream,
                          m->pred_trace && pit->second.entries.size() <= 4096 ? m->pred_trace : nullptr));
  }
  return OMNI_OK;
}

// Runs a graph program at bucket b: the persistent tick kernel when the shapes allow it, else the per-op kernels
// as a replay of their captured graph (or eager launches).
int run_program(omni_talker* m, int program, int b) {
  m->launches = 0;
  if (m->cfg.tick_kernel && tick_usable(m, b)) return run_tick_program(m, program, b);
  if (!m->cfg.use_graphs) return enqueue_program(m, program, b);
  auto key = std::make_pair(program, b);
  auto it = m->graphs.find(key);
  if (it == m->graphs.end()) {
    CUDA_TRY(m, cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    const int rc = enqueue_program(m, program, b);
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(m->stream, &graph);
    if (rc != OMNI_OK) {
      if (graph) cudaGraphDestroy(graph);
      return rc;
    }
    if (e != cudaSuccess) return m->fail(OMNI_ERR_CUDA, "graph capture: %s", cudaGetErrorString(e));
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return m->fail(OMNI_ERR_CUDA, "graph instantiate: %s", cudaGetErrorString(e));
    it = m->graphs.emplace(key, exec).first;
    m->stats.bucket = b;
    m->graph_nodes[key] = m->launches;
  }
  m->launches = m->graph_nodes[key];
  CUDA_TRY(m, cudaGraphLaunch(it->second, m->stream));
  return OMNI_OK;
}

}  // namespace

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Offsets of the staged inputs (names of crates/omni-qwen3-tts/src/model.rs:266-303,348-359).
void layout_inputs(omni_talker* m) {
  auto& in = m->in;
  const size_t B = m->max_seqs, T = m->max_rows;
  size_t at = 0;
  auto take = [&](size_t bytes) {
    const size_t here = at;
    at = align_up(at + bytes, 16);
    return here;
  };
  in.lines = take(B * 4);
  in.pos = take(B * 4);
  in.force = take(B * OMNI_GROUPS * 4);
  in.uniforms = take(B * OMNI_GROUPS * 4);
  in.indptr = take((B + 1) * 4);
  in.d_pos = take(B * 4);
  in.d_slot = take(B * 4);
  in.front_fixed_bytes = at;
  in.pages = take((size_t)m->page_table * 4);
  in.t_ids = take(T * 4);
  in.t_codec = take(T * 4);
  in.t_pos = take(T * 4);
  in.t_slot = take(T * 4);
  in.t_seq = take(T * 4);
  in.last_row = take(B * 4);
  in.total_bytes = at;
}

int32_t slot_of_seq(const omni_seq& s, int pos) { return s.pages[pos / OMNI_PAGE] * OMNI_PAGE + pos % OMNI_PAGE; }

struct FrameRow {
  const omni_seq* seq;
  int position;  // talker position the last frame goes in
  int frame;     // index of the frame this call draws
  const omni_draw* draw;
};

// `Model::graph_inputs` (model.rs:197-218): per-sequence inputs of a graph call
// padded to its bucket with the pad lease; returns the bytes of the front
// block (fixed part + the page lists) to copy.
size_t stage_graph_inputs(omni_talker* m, char* host, const std::vector<FrameRow>& rows, int b, bool talker) {
  auto& in = m->in;
  int32_t* lines = reinterpret_cast<int32_t*>(host + in.lines);
  int32_t* pos = reinterpret_cast<int32_t*>(host + in.pos);
  int32_t* force = reinterpret_cast<int32_t*>(host + in.force);
  float* uniforms = reinterpret_cast<float*>(host + in.uniforms);
  int32_t* indptr = reinterpret_cast<int32_t*>(host + in.indptr);
  int32_t* d_pos = reinterpret_cast<int32_t*>(host + in.d_pos);
  int32_t* d_slot = reinterpret_cast<int32_t*>(host + in.d_slot);
  int32_t* pages = reinterpret_cast<int32_t*>(host + in.pages);
  int np = 0;
  indptr[0] = 0;
  for (int s = 0; s < b; ++s) {
    const bool real = s < (int)rows.size();
    const omni_seq& q = real ? *rows[s].seq : m->pad;
    lines[s] = q.line;
    pos[s] = real ? rows[s].frame : 0;
    for (int g = 0; g < OMNI_GROUPS; ++g) {
      uniforms[s * OMNI_GROUPS + g] = real ? rows[s].draw->uniforms[g] : 0.5f;
      force[s * OMNI_GROUPS + g] = real ? rows[s].draw->force[g] : -1;
    }
    const int position = real ? rows[s].position : 0;
    d_pos[s] = position;
    d_slot[s] = slot_of_seq(q, position);
    if (talker) {
      // only the pages up to the row's position are read
      const int used = position / OMNI_PAGE + 1;
      for (int i = 0; i < used; ++i) pages[np++] = q.pages[i];
    }
    indptr[s + 1] = np;
  }
  return in.pages + (size_t)np * 4;
}


// Writes one line per phase of the last traced tick: its shape, then (ns, relative to the median time at which the
// CTAs saw the previous barrier complete) the median and the latest over CTAs of: first activation tile in shared
// memory, first accumulator complete, own share done, barrier seen complete.
void dump_trace(omni_talker* m) {
  if (m->pred_trace && m->pred_trace_program && !m->trace_path.empty()) {
    // the cluster kernel's entries: "entry epilogue rows k-blocks position start loop end" (ns after the first entry's start)
    const PredProgram& prog = *m->pred_trace_program;
    std::vector<unsigned long long> t(3 * prog.entries.size());
    if (cudaMemcpy(t.data(), m->pred_trace, t.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess) {
      if (FILE* f = fopen((m->trace_path + ".pred").c_str(), "w")) {
        for (size_t i = 0; i < prog.entries.size(); ++i) {
          const PredEntry& e = prog.entries[i];
          fprintf(f, "%zu %d %d %d %d %lld %lld %lld\n", i, e.epi, e.rows, e.nkb, e.pos, (long long)(t[3 * i] - t[0]),
                  (long long)(t[3 * i + 1] - t[0]), (long long)(t[3 * i + 2] - t[0]));
        }
        fclose(f);
      }
    }
  }
  if (!m->trace || !m->trace_program || m->trace_path.empty()) return;
  const TickProgram& prog = *m->trace_program;
  const size_t G = (size_t)m->tick_ctas, P = prog.phases.size();
  std::vector<unsigned long long> t(4 * G * P);
  if (cudaMemcpy(t.data(), m->trace, t.size() * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return;
  FILE* f = fopen(m->trace_path.c_str(), "w");
  if (!f) return;
  fprintf(f, "phase type N K tiles splits bn rows tile_n dur x_med x_max acc_med acc_max work_med work_max bar_med bar_max\n");
  auto stat = [&](size_t p, int k, long long origin, long long* med, long long* mx) {
    std::vector<long long> v;
    for (size_t c = 0; c < G; ++c) {
      const unsigned long long x = t[(p * G + c) * 4 + k];
      if (x) v.push_back((long long)x - origin);
    }
    if (v.empty()) {
      *med = *mx = 0;
      return;
    }
    std::sort(v.begin(), v.end());
    *med = v[v.size() / 2];
    *mx = v.back();
  };
  long long origin = 0, unused;
  stat(0, 3, 0, &origin, &unused);
  for (size_t i = 1; i < P; ++i) {
    const Phase& ph = prog.phases[i];
    long long s[8];
    for (int k = 0; k < 4; ++k) stat(i, k, origin, &s[2 * k], &s[2 * k + 1]);
    fprintf(f, "%zu %d %d %d %d %d %d %d %d %lld", i, ph.type, ph.N, ph.K, ph.tiles, ph.splits, ph.bn, ph.rows, ph.tile_n, s[6]);
    for (int k = 0; k < 8; ++k) fprintf(f, " %lld", s[k]);
    fprintf(f, "\n");
    origin += s[6];
  }
  fclose(f);
}

// The frames' audio: with a codec decoder attached every frame of every sequence goes through it (its streams advance
// whether or not the caller takes the samples); without one `wav` is zero-filled.
int decode_audio(omni_talker* m, int n, omni_seq* const* seqs, const int32_t* codes, float* wav) {
  if (!m->codec) {
    if (wav) memset(wav, 0, (size_t)n * 1920 * sizeof(float));
    return OMNI_OK;
  }
  if (!wav) {
    m->wav_scratch.resize((size_t)n * 1920);
    wav = m->wav_scratch.data();
  }
  m->audio_rows.resize(n);
  for (int i = 0; i < n; ++i) m->audio_rows[i] = seqs[i]->audio;
  const int rc = omni_codec_decode(m->codec, n, m->audio_rows.data(), codes, wav);
  if (rc != OMNI_OK) return m->fail(rc, "codec decoder: %s", omni_codec_last_error(m->codec));
  return OMNI_OK;
}

int finish_call(omni_talker* m, int n, omni_seq* const* seqs, int32_t* codes, float* wav) {
  CUDA_TRY(m, cudaMemcpyAsync(m->out_host, m->codes, ((size_t)m->max_seqs * OMNI_GROUPS + 1) * 4,
                              cudaMemcpyDeviceToHost, m->stream));
  CUDA_TRY(m, cudaEventRecord(m->ev1, m->stream));
  CUDA_TRY(m, cudaStreamSynchronize(m->stream));
  cudaEventElapsedTime(&m->stats.last_call_gpu_ms, m->ev0, m->ev1);
  m->stats.last_call_launches = m->launches;
  const uint32_t err = (uint32_t)m->out_host[(size_t)m->max_seqs * OMNI_GROUPS];
  if (err != 0) {
    m->tick_barrier_base = ~0u;  // CTAs of the failed launch may not all have arrived: restart the counter
    cudaMemsetAsync(m->err, 0, 4, m->stream);
    cudaStreamSynchronize(m->stream);
    return m->fail(OMNI_ERR_DEVICE, "device error word 0x%x (1: barrier wait ran out, 2: index out of range)", err);
  }
  memcpy(codes, m->out_host, (size_t)n * OMNI_GROUPS * 4);
  m->last_n = n;
  return decode_audio(m, n, seqs, codes, wav);
}

}  // namespace

extern "C" {

const char* omni_version(void) { return "omni_b200 0.1 (sm_100a)"; }

int32_t omni_bucket(int32_t n) { return bucket_of(n); }

int32_t omni_talker_trace(omni_talker* m, const char* path) {
  if (!m) return OMNI_ERR_INVALID;
  m->trace_path = path ? path : "";
  return OMNI_OK;
}

const char* omni_talker_last_error(const omni_talker* m) { return m ? m->error.c_str() : "null model"; }

void omni_talker_destroy(omni_talker* m) {
  if (!m) return;
  cudaSetDevice(m->device);
  if (m->stream) cudaStreamSynchronize(m->stream);
  for (auto& g : m->graphs) cudaGraphExecDestroy(g.second);
  for (auto& t : m->tick_programs) tick_free(&t.second);
  for (auto& t : m->pred_programs) pred_free(&t.second);
  for (void* p : m->allocations) cudaFree(p);
  if (m->in_host) cudaFreeHost(m->in_host);
  if (m->out_host) cudaFreeHost(m->out_host);
  for (auto& f : m->flight) {
    if (f.in_host) cudaFreeHost(f.in_host);
    if (f.out_host) cudaFreeHost(f.out_host);
    if (f.start) cudaEventDestroy(f.start);
    if (f.done) cudaEventDestroy(f.done);
  }
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

static int create_impl(omni_talker* m, const omni_tensor* tensors, int32_t n_tensors) {
  const omni_talker_config& c = m->cfg;
  const omni_stack_config &t = c.talker, &pc = c.predictor;
  if (c.groups < 2 || c.groups > OMNI_GROUPS) return m->fail(OMNI_ERR_UNSUPPORTED, "groups %d", c.groups);
  if (t.vocab > 4096 || pc.vocab > 4096) return m->fail(OMNI_ERR_UNSUPPORTED, "the sampler takes vocabularies up to 4096");
  for (const omni_stack_config* s : {&t, &pc}) {
    if (s->head_dim != 64 && s->head_dim != 128) return m->fail(OMNI_ERR_UNSUPPORTED, "head_dim %d", s->head_dim);
    if (s->hidden % 8 || s->hidden > 8192 || s->inter % 64) return m->fail(OMNI_ERR_UNSUPPORTED, "hidden %d / intermediate %d", s->hidden, s->inter);
    const int g = s->kv_heads > 0 ? s->q_heads / s->kv_heads : 0;
    if (g * s->kv_heads != s->q_heads || !(g == 1 || g == 2 || g == 4 || g == 5 || g == 8))
      return m->fail(OMNI_ERR_UNSUPPORTED, "%d query heads over %d key heads", s->q_heads, s->kv_heads);
  }
  if (c.max_batch < 1 || c.max_tokens < 1) return m->fail(OMNI_ERR_INVALID, "limits");
  if (c.top_p < 1.f && (c.top_k <= 0 || c.top_k > 512 || c.sub_top_k <= 0 || c.sub_top_k > 512))
    return m->fail(OMNI_ERR_UNSUPPORTED, "top_p < 1 needs 0 < top_k <= 512");

  CUDA_TRY(m, cudaSetDevice(m->device));
  cudaDeviceProp prop;
  CUDA_TRY(m, cudaGetDeviceProperties(&prop, m->device));
  if (prop.major != 10) return m->fail(OMNI_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is sm_100a only", m->device, prop.major, prop.minor);
  m->sm_count = prop.multiProcessorCount;
  CUDA_TRY(m, cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
  CUDA_TRY(m, cudaEventCreate(&m->ev0));
  CUDA_TRY(m, cudaEventCreate(&m->ev1));
  if (tc_init() != 0) return m->fail(OMNI_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  tc_configure();

  if (c.tick_kernel) {
    m->tick_ctas = tick_configure(m->device);
    m->tick_ok = m->tick_ctas > 0;
    TRY(dev_alloc(m, &m->tick_barrier, 64, true));
  }

  TensorIndex idx;
  for (int i = 0; i < n_tensors; ++i) idx.by_name[tensors[i].name] = &tensors[i];
  const int64_t h = t.hidden, p = pc.hidden, V = t.vocab, PV = pc.vocab, G = c.groups;
  const omni_tensor* te = idx.find("talker.model.text_embedding.weight");
  if (!te || te->ndim != 2) return m->fail(OMNI_ERR_MISSING_TENSOR, "missing tensor talker.model.text_embedding.weight");
  m->text_vocab = (int)te->shape[0];
  if (c.tts_pad_token_id < 0 || c.tts_pad_token_id >= m->text_vocab) return m->fail(OMNI_ERR_INVALID, "tts_pad_token_id");

  TRY(dev_alloc(m, &m->text_emb, (size_t)m->text_vocab * h));
  TRY(upload(m, idx, "talker.model.text_embedding.weight", {m->text_vocab, h}, m->text_emb));
  TRY(dev_alloc(m, &m->codec_emb, V * h));
  TRY(upload(m, idx, "talker.model.codec_embedding.weight", {V, h}, m->codec_emb));
  TRY(dev_alloc(m, &m->codec_head, V * h));
  TRY(upload(m, idx, "talker.codec_head.weight", {V, h}, m->codec_head));
  TRY(dev_alloc(m, &m->fc1_w, h * h));
  TRY(dev_alloc(m, &m->fc1_b, h));
  TRY(dev_alloc(m, &m->fc2_w, h * h));
  TRY(dev_alloc(m, &m->fc2_b, h));
  TRY(upload(m, idx, "talker.text_projection.linear_fc1.weight", {h, h}, m->fc1_w));
  TRY(upload(m, idx, "talker.text_projection.linear_fc1.bias", {h}, m->fc1_b));
  TRY(upload(m, idx, "talker.text_projection.linear_fc2.weight", {h, h}, m->fc2_w));
  TRY(upload(m, idx, "talker.text_projection.linear_fc2.bias", {h}, m->fc2_b));
  TRY(dev_alloc(m, &m->mtp_w, p * h));
  TRY(dev_alloc(m, &m->mtp_b, p));
  TRY(upload(m, idx, "talker.code_predictor.small_to_mtp_projection.weight", {p, h}, m->mtp_w));
  TRY(upload(m, idx, "talker.code_predictor.small_to_mtp_projection.bias", {p}, m->mtp_b));
  // the predictor's G-1 embedding tables and heads stacked (talker.rs:85-93,119-130)
  TRY(dev_alloc(m, &m->p_emb, (G - 1) * PV * h));
  TRY(dev_alloc(m, &m->lm_heads, (G - 1) * PV * p));
  for (int g = 0; g < G - 1; ++g) {
    TRY(upload(m, idx, "talker.code_predictor.model.codec_embedding." + std::to_string(g) + ".weight", {PV, h},
               m->p_emb + (size_t)g * PV * h));
    TRY(upload(m, idx, "talker.code_predictor.lm_head." + std::to_string(g) + ".weight", {PV, p},
               m->lm_heads + (size_t)g * PV * p));
  }
  TRY(load_stack(m, idx, "talker.model", t, &m->talker));
  TRY(load_stack(m, idx, "talker.code_predictor.model", pc, &m->pred));
  if (c.tick_kernel == 3 && m->tick_ok && pred_shape_ok(c, m->pred.granule)) m->pred_clusters = pred_configure(pc.q_heads);

  // pools (model.rs:111-131,306-309)
  m->max_seqs = bucket_of(c.max_batch);
  m->max_rows = std::max(c.max_tokens, 2 * m->max_seqs);
  const size_t kv_token_bytes = (size_t)t.layers * 2 * t.kv_heads * t.head_dim * 2;
  const size_t kv_tokens = (size_t)(c.kv_gib * (double)(1ull << 30)) / kv_token_bytes;
  m->pages_total = (int)((kv_tokens + OMNI_PAGE - 1) / OMNI_PAGE) + 1;
  m->page_table = m->pages_total + m->max_seqs;
  m->kv.resize(t.layers);
  for (int i = 0; i < t.layers; ++i) TRY(dev_alloc(m, &m->kv[i], (size_t)m->pages_total * m->talker.kv_page_elems(), true));
  m->kv_bytes = (int64_t)t.layers * m->pages_total * m->talker.kv_page_elems() * 2;
  m->pkv.resize(pc.layers);
  for (int i = 0; i < pc.layers; ++i) TRY(dev_alloc(m, &m->pkv[i], (size_t)m->max_seqs * m->pred.kv_page_elems(), true));
  for (int i = m->pages_total - 1; i >= 0; --i) m->free_pages.push_back(i);
  // per-sequence slot: last frame, repetition bitmap, Philox seed
  m->seen_words = (int)((V + 31) / 32);
  m->seq_stride = (int64_t)align_up(4 * (OMNI_GROUPS + m->seen_words + (m->seen_words & 1)) + 8, 256);
  const int lines = c.max_batch + 1;
  TRY(dev_alloc(m, &m->seq_state, (size_t)lines * m->seq_stride, true));
  for (int i = lines - 1; i >= 0; --i) m->free_lines.push_back(i);

  layout_inputs(m);
  CUDA_TRY(m, cudaHostAlloc((void**)&m->in_host, m->in.total_bytes, cudaHostAllocDefault));
  memset(m->in_host, 0, m->in.total_bytes);
  TRY(dev_alloc(m, &m->in_dev, m->in.total_bytes, true));
  CUDA_TRY(m, cudaHostAlloc((void**)&m->out_host, ((size_t)m->max_seqs * OMNI_GROUPS + 1) * 4, cudaHostAllocDefault));

  TRY(alloc_scratch(m, m->talker, m->max_rows, &m->T));
  TRY(alloc_scratch(m, m->pred, 2 * m->max_seqs, &m->P));
  TRY(dev_alloc(m, &m->t_e, (size_t)m->max_rows * h));
  TRY(dev_alloc(m, &m->t_p, (size_t)m->max_rows * h));
  TRY(dev_alloc(m, &m->embeds, (size_t)m->max_rows * h));
  TRY(dev_alloc(m, &m->hidden, (size_t)m->max_seqs * h, true));
  TRY(dev_alloc(m, &m->pad_embed, h));
  TRY(dev_alloc(m, &m->p_in, (size_t)2 * m->max_seqs * h));
  TRY(dev_alloc(m, &m->p_h, (size_t)2 * m->max_seqs * p));
  TRY(dev_alloc(m, &m->p_last, (size_t)m->max_seqs * p));
  if (m->pred_clusters > 0) TRY(dev_alloc(m, &m->pred_vbuf, (size_t)m->max_seqs * p, true));
  TRY(dev_alloc(m, &m->logits, (size_t)m->max_seqs * V, true));
  TRY(dev_alloc(m, &m->p_logits, (size_t)(G - 1) * m->max_seqs * PV, true));
  TRY(dev_alloc(m, &m->codes, (size_t)m->max_seqs * OMNI_GROUPS + 1, true));
  m->err = reinterpret_cast<uint32_t*>(m->codes + (size_t)m->max_seqs * OMNI_GROUPS);
  // split-K scratch: the widest N the loop multiplies times the tallest row tile, with headroom for splits
  {
    const size_t widest = std::max<size_t>({(size_t)m->talker.qkv_width(), (size_t)2 * t.inter, (size_t)h, (size_t)V,
                                            (size_t)2 * pc.inter, (size_t)m->pred.qkv_width(), (size_t)PV});
    m->gemm_scratch.partial_floats = (size_t)(widest + 128) * 256 * 16;
    m->gemm_scratch.counter_slots = 4096;
    TRY(dev_alloc(m, &m->gemm_scratch.partials, m->gemm_scratch.partial_floats));
    TRY(dev_alloc(m, &m->gemm_scratch.counters, (size_t)m->gemm_scratch.counter_slots, true));
  }

  // the pad lease: one page, one slot (model.rs:130)
  m->pad.pages = {m->free_pages.back()};
  m->free_pages.pop_back();
  m->pad.line = m->free_lines.back();
  m->free_lines.pop_back();
  m->pad.live = true;
  m->pad.cap = OMNI_PAGE;
  m->pages_used = 1;

  // `Talker::init` (talker.rs:169-183): the <tts_pad> embedding through the text projection
  {
    int32_t* ids = m->hin<int32_t>(m->in.t_ids);
    ids[0] = c.tts_pad_token_id;
    CUDA_TRY(m, cudaMemcpyAsync(m->din<int32_t>(m->in.t_ids), ids, 4, cudaMemcpyHostToDevice, m->stream));
    LAUNCH(m, launch_gather(m->din<int32_t>(m->in.t_ids), 1, m->text_emb, m->text_vocab, m->t_e, 1, (int)h, m->err,
                            m->stream));
    Epilogue e1, e2;
    e1.bias = m->fc1_b, e1.kind = kEpiBiasSilu;
    e2.bias = m->fc2_b, e2.kind = kEpiBias;
    TRY(gemm(m, m->fc1_w, (int)h, (int)h, m->t_e, 1, m->t_p, (int)h, e1));
    TRY(gemm(m, m->fc2_w, (int)h, (int)h, m->t_p, 1, m->pad_embed, (int)h, e2));
    CUDA_TRY(m, cudaStreamSynchronize(m->stream));
  }
  // The residual codebooks' embedding tables through small_to_mtp_projection, once: from its second pass on the
  // predictor's input row is projection(embedding of the code just drawn) (talker.rs:306-312), a linear map of a
  // table row, so the persistent kernel looks the projected row up instead of running the projection every pass.
  // Same arithmetic as the per-pass GEMM: bf16(bf16(W . e) + bias).
  if (c.tick_kernel != 0 && m->tick_ok && G > 2) {
    const int64_t total = (G - 1) * PV;
    TRY(dev_alloc(m, &m->p_emb_proj, (size_t)total * p));
    Epilogue bias;
    bias.bias = m->mtp_b, bias.kind = kEpiBias;
    const int64_t chunk = 256;
    for (int64_t r0 = 0; r0 < total; r0 += chunk)
      TRY(gemm(m, m->mtp_w, (int)p, (int)h, m->p_emb + r0 * h, (int)std::min(chunk, total - r0), m->p_emb_proj + r0 * p,
               (int)p, bias));
    // ... and on through the first layer's input norm and q|k|v projection: that layer's q | k | v of a pass's row
    // depend on the code alone too (attention is where the pass first meets its earlier rows)
    const int64_t qw = m->pred.qkv_width();
    bf16 *xn = nullptr, *res = nullptr;
    TRY(dev_alloc(m, &m->p_qkv0, (size_t)total * qw));
    TRY(dev_alloc(m, &xn, (size_t)chunk * p));
    TRY(dev_alloc(m, &res, (size_t)chunk * p));
    for (int64_t r0 = 0; r0 < total; r0 += chunk) {
      const int rows = (int)std::min(chunk, total - r0);
      LAUNCH(m, launch_norm_copy(m->p_emb_proj + r0 * p, m->pred.layers[0].ln1, xn, res, rows, (int)p, pc.rms_eps, m->stream));
      TRY(gemm(m, m->pred.layers[0].qkv, (int)qw, (int)p, xn, rows, m->p_qkv0 + r0 * qw, (int)qw));
    }
    CUDA_TRY(m, cudaStreamSynchronize(m->stream));
    m->plans.clear();  // the plans of these one-off products are not needed again
  }
  return OMNI_OK;
}

int32_t omni_talker_create(const omni_talker_config* cfg, const omni_tensor* tensors, int32_t n_tensors,
                           int32_t device, omni_talker** out) {
  if (!cfg || !tensors || !out) return OMNI_ERR_INVALID;
  omni_talker* m = new omni_talker();
  m->cfg = *cfg;
  m->device = device;
  const int rc = create_impl(m, tensors, n_tensors);
  *out = m;  // returned even on failure so the caller can read the error; destroy() frees it
  return rc;
}

int32_t omni_talker_open(omni_talker* m, int32_t prompt_tokens, int32_t max_frames, omni_seq** out) {
  if (!m || !out || prompt_tokens < 1 || max_frames < 1) return OMNI_ERR_INVALID;
  *out = nullptr;
  const int need = (prompt_tokens + max_frames + OMNI_PAGE - 1) / OMNI_PAGE;
  // model.rs:141-144: a request that could never fit beside the pad lease is refused for good
  if (need + (int)m->pad.pages.size() > m->pages_total) return OMNI_DENIED_EXCEEDS_POOL;
  if (need > (int)m->free_pages.size() || m->free_lines.empty()) return OMNI_DENIED_BUSY;
  auto s = std::make_unique<omni_seq>();
  for (int i = 0; i < need; ++i) {
    s->pages.push_back(m->free_pages.back());
    m->free_pages.pop_back();
  }
  s->line = m->free_lines.back();
  m->free_lines.pop_back();
  s->prompt = prompt_tokens;
  s->cap = prompt_tokens + max_frames;
  s->live = true;
  m->pages_used += need;
  // a fresh slot starts zeroed: empty repetition bitmap, frame of zeros, seed 0
  cudaSetDevice(m->device);
  const cudaError_t e = cudaMemsetAsync(m->seq_state + (size_t)s->line * m->seq_stride, 0, m->seq_stride, m->stream);
  if (e != cudaSuccess) {  // hand the lease back: nothing of this call may stay taken
    for (int32_t p : s->pages) m->free_pages.push_back(p);
    m->free_lines.push_back(s->line);
    m->pages_used -= need;
    return m->fail(OMNI_ERR_CUDA, "clearing the sequence slot: %s", cudaGetErrorString(e));
  }
  if (m->codec) {  // the decoder's state slot travels with the lease
    const int rc = omni_codec_open(m->codec, &s->audio);
    if (rc != OMNI_OK) {
      for (int32_t p : s->pages) m->free_pages.push_back(p);
      m->free_lines.push_back(s->line);
      m->pages_used -= need;
      return rc == OMNI_DENIED_BUSY ? rc : m->fail(rc, "codec decoder: %s", omni_codec_last_error(m->codec));
    }
  }
  *out = s.get();
  m->seqs.push_back(std::move(s));
  return OMNI_OK;
}

int32_t omni_talker_attach_codec(omni_talker* m, omni_codec* codec) {
  if (!m) return OMNI_ERR_INVALID;
  if (!m->seqs.empty() || m->in_flight > 0) return m->fail(OMNI_ERR_INVALID, "attach or detach the codec decoder while no sequence is open");
  if (codec && omni_codec_samples_per_frame(codec) != 1920)
    return m->fail(OMNI_ERR_UNSUPPORTED, "the codec decoder gives %d samples per frame, `wav` rows hold 1920", omni_codec_samples_per_frame(codec));
  m->codec = codec;
  return OMNI_OK;
}

int32_t omni_talker_close(omni_talker* m, omni_seq* seq) {
  if (!m || !seq) return OMNI_ERR_INVALID;
  if (m->in_flight > 0) return m->fail(OMNI_ERR_INVALID, "a step is under way: end it before closing a sequence");
  // the handle is looked up before it is touched: a handle closed before (or never opened here) points at freed memory
  for (size_t i = 0; i < m->seqs.size(); ++i) {
    if (m->seqs[i].get() != seq) continue;
    if (!seq->live) return OMNI_ERR_INVALID;
    if (seq->audio && m->codec) omni_codec_close(m->codec, seq->audio);
    for (int32_t p : seq->pages) m->free_pages.push_back(p);
    m->free_lines.push_back(seq->line);
    m->pages_used -= (int)seq->pages.size();
    m->seqs.erase(m->seqs.begin() + i);
    return OMNI_OK;
  }
  return OMNI_ERR_INVALID;
}

int32_t omni_talker_seq_seed(omni_talker* m, omni_seq* seq, uint64_t seed) {
  if (!m || !seq || !seq->live) return OMNI_ERR_INVALID;
  seq->seed = seed;
  const size_t off = (size_t)seq->line * m->seq_stride + 4 * (OMNI_GROUPS + m->seen_words + (m->seen_words & 1));
  CUDA_TRY(m, cudaMemcpyAsync(m->seq_state + off, &seq->seed, 8, cudaMemcpyHostToDevice, m->stream));
  CUDA_TRY(m, cudaStreamSynchronize(m->stream));
  return OMNI_OK;
}

int32_t omni_talker_seq_frames(const omni_seq* seq) { return seq ? seq->frames : -1; }

int32_t omni_talker_is_end(const omni_talker* m, const int32_t* frame) {
  return m && frame && frame[0] == m->cfg.codec_eos_token_id;
}

int32_t omni_talker_start(omni_talker* m, int32_t n, omni_seq* const* seqs, const int32_t* text_ids,
                          const int32_t* codec_ids, const int32_t* prompt_lens, const omni_draw* draws,
                          int32_t* codes, float* wav) {
  if (!m || !seqs || !text_ids || !codec_ids || !prompt_lens || !draws || !codes) return OMNI_ERR_INVALID;
  if (m->in_flight > 0) return m->fail(OMNI_ERR_INVALID, "a step is under way: end it before a start");
  const omni_talker_config& c = m->cfg;
  if (n < 1 || n > c.max_batch) return m->fail(OMNI_ERR_INVALID, "%d sequences in one call", n);
  int64_t tokens = 0;
  for (int s = 0; s < n; ++s) {
    if (!seqs[s] || !seqs[s]->live || seqs[s]->frames != 0 || prompt_lens[s] != seqs[s]->prompt)
      return m->fail(OMNI_ERR_INVALID, "sequence %d is not fresh", s);
    for (int r = 0; r < s; ++r)
      if (seqs[r] == seqs[s]) return m->fail(OMNI_ERR_INVALID, "sequence %d listed twice", s);
    tokens += prompt_lens[s];
  }
  if (tokens > c.max_tokens) return m->fail(OMNI_ERR_INVALID, "%lld prompt tokens exceed %d", (long long)tokens, c.max_tokens);
  for (int64_t r = 0; r < tokens; ++r) {
    if (text_ids[r] < 0 || text_ids[r] >= m->text_vocab) return m->fail(OMNI_ERR_INVALID, "text id %d at row %lld", text_ids[r], (long long)r);
    if (codec_ids[r] < -1 || codec_ids[r] >= c.talker.vocab) return m->fail(OMNI_ERR_INVALID, "codec id %d at row %lld", codec_ids[r], (long long)r);
  }
  for (int s = 0; s < n; ++s)
    for (int g = 0; g < OMNI_GROUPS; ++g)
      if (draws[s].force[g] >= (g == 0 ? c.talker.vocab : c.predictor.vocab))
        return m->fail(OMNI_ERR_INVALID, "forced code %d of group %d", draws[s].force[g], g);
  CUDA_TRY(m, cudaSetDevice(m->device));

  // `Rows::push_seq` (model.rs:278-289): one row per prompt token
  auto& in = m->in;
  int32_t *t_ids = m->hin<int32_t>(in.t_ids), *t_codec = m->hin<int32_t>(in.t_codec), *t_pos = m->hin<int32_t>(in.t_pos),
          *t_slot = m->hin<int32_t>(in.t_slot), *t_seq = m->hin<int32_t>(in.t_seq), *last_row = m->hin<int32_t>(in.last_row),
          *indptr = m->hin<int32_t>(in.indptr), *pages = m->hin<int32_t>(in.pages);
  int row = 0, np = 0;
  indptr[0] = 0;
  for (int s = 0; s < n; ++s) {
    const omni_seq& q = *seqs[s];
    for (int t = 0; t < q.prompt; ++t, ++row) {
      t_ids[row] = text_ids[row];
      t_codec[row] = codec_ids[row];
      t_pos[row] = t;
      t_slot[row] = slot_of_seq(q, t);
      t_seq[row] = s;
    }
    last_row[s] = row - 1;
    for (int32_t p : q.pages) pages[np++] = p;
    indptr[s + 1] = np;
  }
  const int T = (int)tokens, h = c.talker.hidden;
  CUDA_TRY(m, cudaEventRecord(m->ev0, m->stream));
  CUDA_TRY(m, cudaMemcpyAsync(m->in_dev, m->in_host, in.total_bytes, cudaMemcpyHostToDevice, m->stream));
  m->launches = 0;
  // `Talker::prefill` (talker.rs:186-221)
  LAUNCH(m, launch_gather(m->din<int32_t>(in.t_ids), 1, m->text_emb, m->text_vocab, m->t_e, T, h, m->err, m->stream));
  Epilogue e1;
  e1.bias = m->fc1_b, e1.kind = kEpiBiasSilu;
  TRY(gemm(m, m->fc1_w, h, h, m->t_e, T, m->t_p, h, e1));
  TRY(gemm(m, m->fc2_w, h, h, m->t_p, T, m->embeds, h));
  LAUNCH(m, launch_prompt_codec(m->embeds, m->fc2_b, m->codec_emb, c.talker.vocab, m->din<int32_t>(in.t_codec), T, h,
                                m->err, m->stream));
  RowMap map;
  map.pos = m->din<int32_t>(in.t_pos);
  map.slot = m->din<int32_t>(in.t_slot);
  map.seq = m->din<int32_t>(in.t_seq);
  map.indptr = m->din<int32_t>(in.indptr);
  map.pages = m->din<int32_t>(in.pages);
  TRY(stack_forward(m, m->talker, m->T, m->embeds, T, map, m->kv, m->pages_total, m->T.x, 1, 0));
  LAUNCH(m, launch_gather(m->din<int32_t>(in.last_row), 1, m->T.x, T, m->hidden, n, h, m->err, m->stream));
  const int prefill_launches = m->launches;
  // the staging block is reused below: let the copy above and the prefill finish first
  CUDA_TRY(m, cudaStreamSynchronize(m->stream));

  // the `first` program on the prompt's last hidden state (model.rs:171-175)
  std::vector<FrameRow> rows(n);
  for (int s = 0; s < n; ++s) rows[s] = FrameRow{seqs[s], 0, 0, &draws[s]};
  const int b = bucket_of(n);
  const size_t bytes = stage_graph_inputs(m, m->in_host, rows, b, false);
  CUDA_TRY(m, cudaMemcpyAsync(m->in_dev, m->in_host, bytes, cudaMemcpyHostToDevice, m->stream));
  TRY(run_program(m, kFirst, b));
  m->launches += prefill_launches;
  m->stats.bucket = b;
  TRY(finish_call(m, n, seqs, codes, wav));
  for (int s = 0; s < n; ++s) seqs[s]->frames = 1;
  return OMNI_OK;
}

static int check_step(omni_talker* m, int n, omni_seq* const* seqs, const omni_draw* draws, int ticks) {
  if (m->in_flight > 0 && ticks != 0)
    return m->fail(OMNI_ERR_INVALID, "%d step(s) begun with omni_talker_step_begin are still to be ended", m->in_flight);
  if (ticks == 0) ticks = 1;
  const omni_talker_config& c = m->cfg;
  if (n < 1 || n > c.max_batch) return m->fail(OMNI_ERR_INVALID, "%d sequences in one call", n);
  for (int s = 0; s < n; ++s) {
    if (!seqs[s] || !seqs[s]->live || seqs[s]->frames < 1) return m->fail(OMNI_ERR_INVALID, "sequence %d has not started", s);
    for (int r = 0; r < s; ++r)
      if (seqs[r] == seqs[s]) return m->fail(OMNI_ERR_INVALID, "sequence %d listed twice", s);
    if (seqs[s]->prompt + seqs[s]->frames - 1 + ticks > seqs[s]->cap)
      return m->fail(OMNI_ERR_INVALID, "sequence %d is at its frame cap", s);
  }
  for (int64_t i = 0; i < (int64_t)n * ticks; ++i)
    for (int g = 0; g < OMNI_GROUPS; ++g)
      if (draws[i].force[g] >= (g == 0 ? c.talker.vocab : c.predictor.vocab))
        return m->fail(OMNI_ERR_INVALID, "forced code %d of group %d", draws[i].force[g], g);
  return OMNI_OK;
}

int32_t omni_talker_step(omni_talker* m, int32_t n, omni_seq* const* seqs, const omni_draw* draws, int32_t* codes,
                         float* wav) {
  if (!m || !seqs || !draws || !codes) return OMNI_ERR_INVALID;
  TRY(check_step(m, n, seqs, draws, 1));
  CUDA_TRY(m, cudaSetDevice(m->device));
  std::vector<FrameRow> rows(n);
  for (int s = 0; s < n; ++s) rows[s] = FrameRow{seqs[s], seqs[s]->prompt + seqs[s]->frames - 1, seqs[s]->frames, &draws[s]};
  const int b = bucket_of(n);
  const size_t bytes = stage_graph_inputs(m, m->in_host, rows, b, true);
  CUDA_TRY(m, cudaEventRecord(m->ev0, m->stream));
  CUDA_TRY(m, cudaMemcpyAsync(m->in_dev, m->in_host, bytes, cudaMemcpyHostToDevice, m->stream));
  TRY(run_program(m, kDecode, b));
  m->stats.bucket = b;
  TRY(finish_call(m, n, seqs, codes, wav));
  for (int s = 0; s < n; ++s) seqs[s]->frames += 1;
  return OMNI_OK;
}

int32_t omni_talker_step_begin(omni_talker* m, int32_t n, omni_seq* const* seqs, const omni_draw* draws) {
  if (!m || !seqs || !draws) return OMNI_ERR_INVALID;
  if (m->in_flight >= 2) return m->fail(OMNI_ERR_INVALID, "two steps are under way: end the older one first");
  TRY(check_step(m, n, seqs, draws, 0));
  CUDA_TRY(m, cudaSetDevice(m->device));
  omni_talker::Flight& f = m->flight[(m->flight_first + m->in_flight) % 2];
  if (!f.in_host) {  // first use of this slot (before any stream capture: these are allocations)
    CUDA_TRY(m, cudaHostAlloc((void**)&f.in_host, m->in.total_bytes, cudaHostAllocDefault));
    CUDA_TRY(m, cudaHostAlloc((void**)&f.out_host, ((size_t)m->max_seqs * OMNI_GROUPS + 1) * 4, cudaHostAllocDefault));
    CUDA_TRY(m, cudaEventCreate(&f.start));
    CUDA_TRY(m, cudaEventCreate(&f.done));
  }
  std::vector<FrameRow> rows(n);
  for (int s = 0; s < n; ++s) rows[s] = FrameRow{seqs[s], seqs[s]->prompt + seqs[s]->frames - 1, seqs[s]->frames, &draws[s]};
  const int b = bucket_of(n);
  const size_t bytes = stage_graph_inputs(m, f.in_host, rows, b, true);
  CUDA_TRY(m, cudaEventRecord(f.start, m->stream));
  CUDA_TRY(m, cudaMemcpyAsync(m->in_dev, f.in_host, bytes, cudaMemcpyHostToDevice, m->stream));
  TRY(run_program(m, kDecode, b));
  m->stats.bucket = b;
  CUDA_TRY(m, cudaMemcpyAsync(f.out_host, m->codes, ((size_t)m->max_seqs * OMNI_GROUPS + 1) * 4, cudaMemcpyDeviceToHost,
                              m->stream));
  CUDA_TRY(m, cudaEventRecord(f.done, m->stream));
  f.n = n;
  f.launches = m->launches;
  if (m->codec) f.seqs.assign(seqs, seqs + n);
  m->in_flight += 1;
  for (int s = 0; s < n; ++s) seqs[s]->frames += 1;  // the next step_begin computes its positions from these
  return OMNI_OK;
}

int32_t omni_talker_step_end(omni_talker* m, int32_t* codes, float* wav) {
  if (!m || !codes) return OMNI_ERR_INVALID;
  if (m->in_flight < 1) return m->fail(OMNI_ERR_INVALID, "no step under way");
  CUDA_TRY(m, cudaSetDevice(m->device));
  omni_talker::Flight& f = m->flight[m->flight_first];
  CUDA_TRY(m, cudaEventSynchronize(f.done));
  m->flight_first ^= 1;
  m->in_flight -= 1;
  cudaEventElapsedTime(&m->stats.last_call_gpu_ms, f.start, f.done);
  m->stats.last_call_launches = f.launches;
  const uint32_t err = (uint32_t)f.out_host[(size_t)m->max_seqs * OMNI_GROUPS];
  if (err != 0) {
    // a step begun after this one ran on the same error word: wait for it, drop it, then clear the word
    CUDA_TRY(m, cudaStreamSynchronize(m->stream));
    m->in_flight = 0;
    m->tick_barrier_base = ~0u;
    cudaMemsetAsync(m->err, 0, 4, m->stream);
    cudaStreamSynchronize(m->stream);
    return m->fail(OMNI_ERR_DEVICE, "device error word 0x%x (1: barrier wait ran out, 2: index out of range)", err);
  }
  memcpy(codes, f.out_host, (size_t)f.n * OMNI_GROUPS * 4);
  m->last_n = f.n;
  return decode_audio(m, f.n, f.seqs.data(), codes, wav);
}

int32_t omni_talker_run_ticks(omni_talker* m, int32_t n, omni_seq* const* seqs, int32_t ticks, const omni_draw* draws,
                              int32_t* codes, float* tick_ms) {
  if (!m || !seqs || !draws || ticks < 1) return OMNI_ERR_INVALID;
  TRY(check_step(m, n, seqs, draws, ticks));
  CUDA_TRY(m, cudaSetDevice(m->device));
  const int b = bucket_of(n);
  // every tick's front block, built on the host, staged on the device before the first tick
  size_t block = 0;
  std::vector<char> host;
  std::vector<FrameRow> rows(n);
  std::vector<size_t> used(ticks);
  {
    // the last tick reads the most pages; size every block for it
    for (int s = 0; s < n; ++s) rows[s] = FrameRow{seqs[s], seqs[s]->prompt + seqs[s]->frames - 2 + ticks, 0, &draws[s]};
    std::vector<char> probe(m->in.total_bytes);
    block = align_up(stage_graph_inputs(m, probe.data(), rows, b, true), 256);
  }
  host.resize(block * ticks);
  for (int t = 0; t < ticks; ++t) {
    for (int s = 0; s < n; ++s)
      rows[s] = FrameRow{seqs[s], seqs[s]->prompt + seqs[s]->frames - 1 + t, seqs[s]->frames + t, &draws[(size_t)t * n + s]};
    std::vector<char> tmp(m->in.total_bytes);
    used[t] = stage_graph_inputs(m, tmp.data(), rows, b, true);
    memcpy(host.data() + block * t, tmp.data(), used[t]);
  }
  char* staged = nullptr;
  int32_t* codes_dev = nullptr;
  cudaError_t e = cudaMalloc((void**)&staged, block * ticks);
  if (e != cudaSuccess) return m->fail(OMNI_ERR_CUDA, "cudaMalloc staged inputs: %s", cudaGetErrorString(e));
  const size_t frame_bytes = (size_t)n * OMNI_GROUPS * 4;
  e = cudaMalloc((void**)&codes_dev, frame_bytes * ticks);
  if (e != cudaSuccess) {
    cudaFree(staged);
    return m->fail(OMNI_ERR_CUDA, "cudaMalloc codes: %s", cudaGetErrorString(e));
  }
  std::vector<cudaEvent_t> ev(ticks + 1);
  for (auto& x : ev) cudaEventCreate(&x);
  int rc = OMNI_OK;
  auto body = [&]() -> int {
    CUDA_TRY(m, cudaMemcpyAsync(staged, host.data(), block * ticks, cudaMemcpyHostToDevice, m->stream));
    CUDA_TRY(m, cudaStreamSynchronize(m->stream));
    CUDA_TRY(m, cudaEventRecord(ev[0], m->stream));
    for (int t = 0; t < ticks; ++t) {
      CUDA_TRY(m, cudaMemcpyAsync(m->in_dev, staged + block * t, used[t], cudaMemcpyDeviceToDevice, m->stream));
      TRY(run_program(m, kDecode, b));
      CUDA_TRY(m, cudaMemcpyAsync(codes_dev + (size_t)t * n * OMNI_GROUPS, m->codes, frame_bytes,
                                  cudaMemcpyDeviceToDevice, m->stream));
      CUDA_TRY(m, cudaEventRecord(ev[t + 1], m->stream));
    }
    CUDA_TRY(m, cudaStreamSynchronize(m->stream));
    uint32_t err = 0;
    CUDA_TRY(m, cudaMemcpy(&err, m->err, 4, cudaMemcpyDeviceToHost));
    if (err != 0) {
      m->tick_barrier_base = ~0u;
      cudaMemset(m->err, 0, 4);
      return m->fail(OMNI_ERR_DEVICE, "device error word 0x%x", err);
    }
    if (codes) CUDA_TRY(m, cudaMemcpy(codes, codes_dev, frame_bytes * ticks, cudaMemcpyDeviceToHost));
    float total = 0.f;
    for (int t = 0; t < ticks; ++t) {
      float ms = 0.f;
      cudaEventElapsedTime(&ms, ev[t], ev[t + 1]);
      if (tick_ms) tick_ms[t] = ms;
      total += ms;
    }
    m->stats.last_call_gpu_ms = total;
    m->stats.last_call_launches = m->launches * ticks;
    m->stats.bucket = b;
    dump_trace(m);
    return OMNI_OK;
  };
  rc = body();
  for (auto& x : ev) cudaEventDestroy(x);
  cudaFree(staged);
  cudaFree(codes_dev);
  if (rc == OMNI_OK) {
    for (int s = 0; s < n; ++s) seqs[s]->frames += ticks;
    m->last_n = n;
  }
  return rc;
}

int32_t omni_talker_read(omni_talker* m, int32_t buffer, int32_t s, void* dst, size_t bytes) {
  if (!m || !dst) return OMNI_ERR_INVALID;
  const omni_talker_config& c = m->cfg;
  CUDA_TRY(m, cudaSetDevice(m->device));
  CUDA_TRY(m, cudaStreamSynchronize(m->stream));
  const size_t V = c.talker.vocab, PV = c.predictor.vocab, h = c.talker.hidden;
  switch (buffer) {
    case OMNI_BUF_LOGITS:
      if (s < 0 || s >= m->max_seqs || bytes != V * 2) return m->fail(OMNI_ERR_INVALID, "logits read");
      CUDA_TRY(m, cudaMemcpy(dst, m->logits + (size_t)s * V, bytes, cudaMemcpyDeviceToHost));
      return OMNI_OK;
    case OMNI_BUF_P_LOGITS:
      if (s < 0 || s >= m->max_seqs || bytes != (size_t)(c.groups - 1) * PV * 2) return m->fail(OMNI_ERR_INVALID, "p_logits read");
      for (int g = 0; g < c.groups - 1; ++g)  // row (g, s) sits at g * max_seqs + s (talker.rs:347)
        CUDA_TRY(m, cudaMemcpy((char*)dst + (size_t)g * PV * 2, m->p_logits + ((size_t)g * m->max_seqs + s) * PV, PV * 2,
                               cudaMemcpyDeviceToHost));
      return OMNI_OK;
    case OMNI_BUF_EMBEDS:
      if (bytes > (size_t)m->max_rows * h * 2) return m->fail(OMNI_ERR_INVALID, "embeds read");
      CUDA_TRY(m, cudaMemcpy(dst, m->embeds, bytes, cudaMemcpyDeviceToHost));
      return OMNI_OK;
    case OMNI_BUF_HIDDEN:
      if (s < 0 || s >= m->max_seqs || bytes != h * 2) return m->fail(OMNI_ERR_INVALID, "hidden read");
      CUDA_TRY(m, cudaMemcpy(dst, m->hidden + (size_t)s * h, bytes, cudaMemcpyDeviceToHost));
      return OMNI_OK;
    case OMNI_BUF_PAD_EMBED:
      if (bytes != h * 2) return m->fail(OMNI_ERR_INVALID, "pad_embed read");
      CUDA_TRY(m, cudaMemcpy(dst, m->pad_embed, bytes, cudaMemcpyDeviceToHost));
      return OMNI_OK;
  }
  return m->fail(OMNI_ERR_INVALID, "unknown buffer %d", buffer);
}

int32_t omni_talker_stats(omni_talker* m, omni_stats* out) {
  if (!m || !out) return OMNI_ERR_INVALID;
  m->stats.pages_total = m->pages_total;
  m->stats.pages_used = m->pages_used;
  m->stats.weight_bytes = m->weight_bytes;
  m->stats.kv_bytes = m->kv_bytes;
  *out = m->stats;
  return OMNI_OK;
}

}  // extern "C"
