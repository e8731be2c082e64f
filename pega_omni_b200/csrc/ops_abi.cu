// Operator-level C ABI (include/omni_b200_ops.h): each kernel as a plain call
// over caller-owned device buffers.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/omni_b200.h"
#include "../../include/omni_b200_ops.h"
#include "codec.h"
#include "gemm.h"
#include "duplex.h"
#include "kernels.h"

using namespace omni;

struct omni_ops {
  int device = 0, sm_count = 148;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev[2] = {nullptr, nullptr};
  GemmScratch scratch;
  uint32_t* err = nullptr;
  std::string error;
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

#define OPS_CUDA(ctx, expr)                                                                       \
  do {                                                                                            \
    cudaError_t e_ = (expr);                                                                      \
    if (e_ != cudaSuccess) return (ctx)->fail(OMNI_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

extern "C" {

int32_t omni_ops_create(int32_t device, omni_ops** out) {
  if (!out) return OMNI_ERR_INVALID;
  omni_ops* c = new omni_ops();
  *out = c;
  c->device = device;
  OPS_CUDA(c, cudaSetDevice(device));
  cudaDeviceProp prop;
  OPS_CUDA(c, cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return c->fail(OMNI_ERR_UNSUPPORTED, "device is sm_%d%d; this library is sm_100a only", prop.major, prop.minor);
  c->sm_count = prop.multiProcessorCount;
  OPS_CUDA(c, cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
  OPS_CUDA(c, cudaEventCreate(&c->ev[0]));
  OPS_CUDA(c, cudaEventCreate(&c->ev[1]));
  if (tc_init() != 0) return c->fail(OMNI_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  tc_configure();
  c->scratch.partial_floats = (size_t)64 << 20;  // 256 MB of f32 partials: any test shape
  c->scratch.counter_slots = 1 << 16;
  OPS_CUDA(c, cudaMalloc((void**)&c->scratch.partials, c->scratch.partial_floats * 4));
  OPS_CUDA(c, cudaMalloc((void**)&c->scratch.counters, (size_t)c->scratch.counter_slots * 4));
  OPS_CUDA(c, cudaMemset(c->scratch.counters, 0, (size_t)c->scratch.counter_slots * 4));
  OPS_CUDA(c, cudaMalloc((void**)&c->err, 256));
  OPS_CUDA(c, cudaMemset(c->err, 0, 256));
  return OMNI_OK;
}

void omni_ops_destroy(omni_ops* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  cudaFree(c->scratch.partials);
  cudaFree(c->scratch.counters);
  cudaFree(c->err);
  if (c->ev[0]) cudaEventDestroy(c->ev[0]);
  if (c->ev[1]) cudaEventDestroy(c->ev[1]);
  if (c->stream) cudaStreamDestroy(c->stream);
  delete c;
}

const char* omni_ops_last_error(const omni_ops* c) { return c ? c->error.c_str() : "null context"; }

int32_t omni_ops_sync(omni_ops* c, uint32_t* word) {
  if (!c) return OMNI_ERR_INVALID;
  OPS_CUDA(c, cudaStreamSynchronize(c->stream));
  uint32_t w = 0;
  OPS_CUDA(c, cudaMemcpy(&w, c->err, 4, cudaMemcpyDeviceToHost));
  if (word) *word = w;
  if (w != 0) {
    cudaMemset(c->err, 0, 4);
    return c->fail(OMNI_ERR_DEVICE, "device error word 0x%x", w);
  }
  return OMNI_OK;
}

int32_t omni_ops_mark(omni_ops* c, int32_t which) {
  if (!c || which < 0 || which > 1) return OMNI_ERR_INVALID;
  OPS_CUDA(c, cudaEventRecord(c->ev[which], c->stream));
  return OMNI_OK;
}

int32_t omni_ops_elapsed_ms(omni_ops* c, float* ms) {
  if (!c || !ms) return OMNI_ERR_INVALID;
  OPS_CUDA(c, cudaEventSynchronize(c->ev[1]));
  OPS_CUDA(c, cudaEventElapsedTime(ms, c->ev[0], c->ev[1]));
  return OMNI_OK;
}

int32_t omni_op_gemm(omni_ops* c, const void* w, int32_t N, int32_t K, const void* x, int32_t rows, void* y,
                     int32_t ldy, int32_t path, int32_t splits, const void* bias, int32_t epilogue) {
  if (!c || !w || !x || !y || N < 1 || K < 8 || rows < 1) return OMNI_ERR_INVALID;
  if (epilogue != OMNI_EPI_NONE && !bias) return c->fail(OMNI_ERR_INVALID, "epilogue %d needs a bias", epilogue);
  Epilogue epi;
  epi.bias = static_cast<const bf16*>(bias);
  epi.kind = epilogue;
  if (path == OMNI_GEMM_TENSOR_ROWS) {
    if (!rm_supports(N, K, rows)) return c->fail(OMNI_ERR_UNSUPPORTED, "rows-on-M path needs rows <= 128, K %% 64 == 0, K <= 4096");
    RmGemmPlan plan;
    const int rc = rm_plan(&plan, (const bf16*)w, N, K, (const bf16*)x, rows, (bf16*)y, ldy, epi, c->sm_count);
    if (rc != 0) return c->fail(OMNI_ERR_CUDA, "tensor-map encode failed (%d)", rc);
    OPS_CUDA(c, rm_launch(plan, c->err, c->stream));
    return OMNI_OK;
  }
  const bool tensor = path == OMNI_GEMM_TENSOR || (path == OMNI_GEMM_AUTO && rows > 8 && tc_supports(N, K, rows));
  if (!tensor) {
    OPS_CUDA(c, gemv_launch((const bf16*)w, N, K, (const bf16*)x, rows, (bf16*)y, ldy, epi, c->sm_count, c->stream));
    return OMNI_OK;
  }
  if (!tc_supports(N, K, rows)) return c->fail(OMNI_ERR_UNSUPPORTED, "tensor path needs K %% 64 == 0");
  TcGemmPlan plan;
  const int rc = tc_plan(&plan, (const bf16*)w, N, K, (const bf16*)x, rows, (bf16*)y, ldy, epi, c->sm_count, splits);
  if (rc != 0) return c->fail(OMNI_ERR_CUDA, "tensor-map encode failed (%d)", rc);
  OPS_CUDA(c, tc_launch(plan, c->scratch, c->err, c->stream));
  return OMNI_OK;
}

int32_t omni_op_norm_copy(omni_ops* c, const void* x, const void* w, void* out, void* res, int32_t rows, int32_t dim,
                          float eps) {
  if (!c) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_norm_copy((const bf16*)x, (const bf16*)w, (bf16*)out, (bf16*)res, rows, dim, eps, c->stream));
  return OMNI_OK;
}

int32_t omni_op_add_norm(omni_ops* c, const void* x, void* res, const void* w, void* out, int32_t rows, int32_t dim,
                         float eps, int32_t every, int32_t which) {
  if (!c || every < 1 || which < 0 || which >= every) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_add_norm((const bf16*)x, (bf16*)res, (const bf16*)w, (bf16*)out, rows, dim, eps, every, which,
                              c->stream));
  return OMNI_OK;
}

int32_t omni_op_silu_mul(omni_ops* c, const void* gate_up, void* act, int32_t rows, int32_t inter) {
  if (!c || inter % 8) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_silu_mul((const bf16*)gate_up, (bf16*)act, rows, inter, 0, c->stream));
  return OMNI_OK;
}

int32_t omni_op_rope_attend(omni_ops* c, void* qkv, const void* q_norm, const void* k_norm, void* kv,
                            int32_t kv_pages, const int32_t* pos, const int32_t* slot, const int32_t* seq,
                            const int32_t* indptr, const int32_t* pages, int32_t rows, int32_t q_heads,
                            int32_t kv_heads, int32_t head_dim, float eps, float theta, void* out) {
  if (!c || !pos || !slot || !indptr || !pages) return OMNI_ERR_INVALID;
  RowMap map;
  map.pos = pos;
  map.slot = slot;
  map.seq = seq;
  map.indptr = indptr;
  map.pages = pages;
  const AttnShape a{q_heads, kv_heads, head_dim, eps, theta};
  OPS_CUDA(c, launch_rope_kv((bf16*)qkv, (const bf16*)q_norm, (const bf16*)k_norm, (bf16*)kv, map, rows, a, kv_pages,
                             c->err, c->stream));
  OPS_CUDA(c, launch_attend((const bf16*)qkv, (const bf16*)kv, (bf16*)out, map, rows, a, c->err, c->stream));
  return OMNI_OK;
}

int32_t omni_op_sample(omni_ops* c, const void* logits, int32_t vocab, float temperature, int32_t top_k, float top_p,
                       float penalty, int32_t suppress_lo, int32_t suppress_hi, int32_t exempt, int32_t min_frames,
                       const int32_t* frames, const float* uniforms, const int32_t* force, void* state,
                       const int32_t* lines, int64_t stride, int32_t penalize, int32_t philox, int32_t* codes,
                       int32_t group, int32_t rows) {
  if (!c || group < 0 || group >= OMNI_GROUPS) return OMNI_ERR_INVALID;
  SampleParams p{};
  p.vocab = vocab;
  p.temperature = temperature;
  p.top_k = top_k;
  p.top_p = top_p;
  p.penalty = penalty;
  p.suppress_lo = suppress_lo;
  p.suppress_hi = suppress_hi;
  p.exempt = exempt;
  p.min_frames = min_frames;
  p.penalize = penalize;
  p.group = group;
  p.philox = philox;
  p.seen_words = (vocab + 31) / 32;
  if (top_p < 1.f && (top_k <= 0 || top_k > 1024))
    return c->fail(OMNI_ERR_UNSUPPORTED, "top_p < 1 needs 0 < top_k <= 1024 (the nucleus filter ranks the survivors of the top-k cut)");
  OPS_CUDA(c, launch_sample((const bf16*)logits, p, frames, uniforms, force, SlotState{state, lines, stride}, codes,
                            rows, c->stream));
  return OMNI_OK;
}

int32_t omni_op_lm_norm(omni_ops* c, const void* y, void* x, const void* alpha, void* out, int32_t rows, int32_t dim,
                        float eps) {
  if (!c || !x) return OMNI_ERR_INVALID;
  if (y)
    OPS_CUDA(c, launch_lm_add_norm((const bf16*)y, (bf16*)x, (const bf16*)alpha, (bf16*)out, rows, dim, eps, c->stream));
  else
    OPS_CUDA(c, launch_lm_norm((const bf16*)x, (const bf16*)alpha, (bf16*)out, rows, dim, eps, c->stream));
  return OMNI_OK;
}

int32_t omni_op_lm_tp_add_norm(omni_ops* c, const void* mine, const void* peer, void* x, const void* alpha, void* out,
                               int32_t rows, int32_t dim, float eps, void* words) {
  if (!c || !mine || !peer || !x || !words) return OMNI_ERR_INVALID;
  TpLink link;
  uint32_t* w = static_cast<uint32_t*>(words);
  link.my_flag = w, link.peer_flag = w + 16, link.counter = w + 32, link.finished = w + 48;
  OPS_CUDA(c, launch_lm_tp_add_norm((const bf16*)mine, (const bf16*)peer, (bf16*)x, (const bf16*)alpha, (bf16*)out, rows,
                                    dim, eps, link, c->err, c->stream));
  return OMNI_OK;
}

int32_t omni_op_lm_embed(omni_ops* c, const int32_t* ids, const void* text_emb, int32_t text_rows,
                         const void* audio_emb, int32_t card_rows, void* out, int32_t rows, int32_t dim) {
  if (!c || !ids || !out) return OMNI_ERR_INVALID;
  const DuplexTables t{(const bf16*)text_emb, (const bf16*)audio_emb, text_rows, card_rows};
  OPS_CUDA(c, launch_lm_embed_ids(ids, nullptr, nullptr, 0, t, (bf16*)out, rows, dim, c->err, c->stream));
  return OMNI_OK;
}

int32_t omni_op_lm_rope_attend(omni_ops* c, void* qkv, void* kv, int32_t kv_pages, const int32_t* pos,
                               const int32_t* slot, const int32_t* seq, const int32_t* indptr, const int32_t* pages,
                               int32_t rows, int32_t heads, float coef, float scale, int32_t context, void* out) {
  if (!c || !qkv || !kv || !pos || !slot || !indptr || !pages || !out) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_lm_rope_kv((bf16*)qkv, pos, slot, kv, rows, heads, coef, kv_pages, c->err, c->stream));
  OPS_CUDA(c, launch_lm_attend((const bf16*)qkv, kv, pos, seq, indptr, pages, (bf16*)out, rows, heads, scale, context,
                               kv_pages, c->err, c->stream));
  return OMNI_OK;
}

int32_t omni_op_lm_dep_embed_norm(omni_ops* c, const void* projected, int32_t k, const void* table, int32_t table_rows,
                                  const int32_t* drawn, const void* alpha, void* x, void* xn, int32_t rows, int32_t dim,
                                  float eps) {
  if (!c || k < 0 || k >= kDepSteps) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_lm_dep_embed_norm((const bf16*)projected, k, (const bf16*)table, table_rows, drawn,
                                       (const bf16*)alpha, (bf16*)x, (bf16*)xn, rows, dim, eps, c->err, c->stream));
  return OMNI_OK;
}

int32_t omni_op_lm_dep_kv_attend(omni_ops* c, const void* qkv, void* ws, int32_t step, void* out, int32_t rows,
                                 int32_t heads, float scale) {
  if (!c) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_lm_dep_kv_attend((const bf16*)qkv, (bf16*)ws, step, (bf16*)out, rows, heads, scale, c->stream));
  return OMNI_OK;
}

int32_t omni_op_lm_sample(omni_ops* c, const void* logits, int32_t vocab, int64_t ld, float temperature, int32_t top_k,
                          const int32_t* force, const int32_t* seeds, int32_t col, int32_t* drawn, int32_t rows) {
  if (!c || !logits || !force || !seeds || !drawn) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_lm_sample((const bf16*)logits, vocab, ld, temperature, top_k, force, seeds, col, drawn, rows,
                               c->stream));
  return OMNI_OK;
}

int32_t omni_op_lm_advance(omni_ops* c, void* state, const int32_t* lines, int64_t stride, const int32_t* init,
                           const int32_t* drawn, const int32_t* caller, const int32_t* force_caller, int32_t* emitted,
                           int32_t rows) {
  if (!c || !state || !lines) return OMNI_ERR_INVALID;
  if (init) OPS_CUDA(c, launch_lm_init(state, lines, stride, init, rows, c->stream));
  if (drawn) {
    if (!caller || !force_caller || !emitted) return OMNI_ERR_INVALID;
    OPS_CUDA(c, launch_lm_advance(state, lines, stride, drawn, caller, force_caller, emitted, rows, c->stream));
  }
  return OMNI_OK;
}

int32_t omni_op_higgs_frame_embed(omni_ops* c, void* state, const int32_t* lines, int64_t stride, const void* table,
                                  void* out, int32_t rows, int32_t dim, int32_t vocab) {
  if (!c || !state || !lines || !table || !out) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_higgs_frame_embed(SlotState{state, lines, stride}, (const bf16*)table, (bf16*)out, rows, dim, vocab,
                                       c->err, c->stream));
  return OMNI_OK;
}

int32_t omni_op_higgs_sample(omni_ops* c, const void* logits, int32_t vocab, float temperature, int32_t top_k,
                             const float* uniforms, const int32_t* force, void* state, const int32_t* lines,
                             int64_t stride, int32_t* codes, int32_t rows) {
  if (!c || !logits || !uniforms || !force || !state || !lines || !codes) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_higgs_sample((const bf16*)logits, vocab, temperature, top_k, uniforms, force,
                                  SlotState{state, lines, stride}, codes, rows, c->stream));
  return OMNI_OK;
}

int32_t omni_higgs_delay_forced_from(const omni_higgs_delay* d) {
  return d ? std::min(d->steps + 1, OMNI_HIGGS_BOOKS) : OMNI_ERR_INVALID;
}

int32_t omni_higgs_delay_advance(omni_higgs_delay* d, int32_t first) {
  if (!d) return OMNI_ERR_INVALID;
  if (d->done) return 1;
  if (d->steps < OMNI_HIGGS_BOOKS) {  // the ramp: an end drawn here is not one
    d->steps += 1;
  } else if (d->countdown > 0) {
    d->countdown -= 1;
    d->done = d->countdown <= 1;
    if (d->done) d->countdown = 0;
  } else if (first == OMNI_HIGGS_EOC) {
    d->countdown = OMNI_HIGGS_BOOKS - 2 + 1;  // books - 2 more steps; stored + 1 so that 0 means "not running"
  }
  return d->done;
}

int32_t omni_higgs_undelay(const int32_t* rows, int32_t n_rows, int32_t* frames) {
  if (n_rows < 0 || (n_rows > 0 && (!rows || !frames))) return OMNI_ERR_INVALID;
  const int n = std::max(n_rows - (OMNI_HIGGS_BOOKS - 1), 0);
  for (int t = 0; t < n; ++t)
    for (int b = 0; b < OMNI_HIGGS_BOOKS; ++b) frames[t * OMNI_HIGGS_BOOKS + b] = rows[(t + b) * OMNI_HIGGS_BOOKS + b];
  return n;
}

// ---- streaming codec decoder ---------------------------------------------------------------------------------------

int32_t omni_op_codec_rvq(omni_ops* c, const int32_t* codes, const void* books, void* out, int32_t n, int32_t half,
                          int32_t book_rows) {
  if (!c || !codes || !books || !out || half % 8) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_rvq(codes, (const bf16*)books, (bf16*)out, n, half, book_rows, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_add_norm(omni_ops* c, const void* add, int64_t add_stride, void* res, const void* w, void* out,
                               int32_t rows, int32_t dim, float eps) {
  if (!c || !add || !res || !w || !out || dim % 256 || dim > 1024) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_add_norm((const bf16*)add, add_stride, (bf16*)res, (const bf16*)w, (bf16*)out, rows, dim, eps,
                                    c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_window_attend(omni_ops* c, const void* qkv, void* state, const int32_t* lines, const int32_t* pos,
                                    int64_t stride, int64_t ring_offset, void* out, int32_t n, int32_t heads, float theta) {
  if (!c || !qkv || !state || !lines || !pos || !out) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_window_attend((const bf16*)qkv, CodecStateRef{(char*)state, lines, pos, stride}, ring_offset,
                                         (bf16*)out, n, heads, theta, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_bias_gelu(omni_ops* c, void* x, const void* bias, int64_t rows, int32_t cols) {
  if (!c || !x || !bias || cols % 8) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_bias_gelu((bf16*)x, (const bf16*)bias, rows, cols, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_bias_snake(omni_ops* c, const void* x, const void* bias, const float* alpha, const float* inv_b,
                                 void* out, int64_t rows, int32_t cols) {
  if (!c || !x || !bias || !alpha || !inv_b || !out || cols % 8) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_bias_snake((const bf16*)x, (const bf16*)bias, alpha, inv_b, (bf16*)out, rows, cols, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_stage(omni_ops* c, const void* x, const void* bias, const float* alpha, const float* inv_b,
                            void* state, const int32_t* lines, const int32_t* pos, int64_t stride, int64_t hist_offset,
                            void* padded, int32_t n, int32_t T, int32_t C, int32_t H) {
  if (!c || !x || !bias || !state || !lines || !pos || !padded || C % 8 || (alpha != nullptr) != (inv_b != nullptr))
    return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_stage((const bf16*)x, (const bf16*)bias, alpha, inv_b, CodecStateRef{(char*)state, lines, pos, stride},
                                 hist_offset, (bf16*)padded, n, T, C, H, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_gather_taps(omni_ops* c, const void* padded, void* col, int32_t n, int32_t T, int32_t C,
                                  int32_t taps, int32_t dil) {
  if (!c || !padded || !col || C % 8) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_gather_taps((const bf16*)padded, (bf16*)col, n, T, C, taps, dil, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_conv(omni_ops* c, const void* w, int32_t N, int32_t C, int32_t taps, int32_t dil, const void* padded,
                           int32_t T, int32_t n_streams, void* y, int32_t epilogue, const void* bias, const float* alpha,
                           const float* inv_b) {
  if (!c || !w || !padded || !y || epilogue < 0 || epilogue > 2) return OMNI_ERR_INVALID;
  if (epilogue == kConvBiasSnake && (!bias || !alpha || !inv_b)) return OMNI_ERR_INVALID;
  conv_configure();
  ConvGemmPlan plan;
  const int rc = conv_plan(&plan, (const bf16*)w, N, C, taps, dil, (const bf16*)padded, T, n_streams, (bf16*)y, epilogue,
                           (const bf16*)bias, alpha, inv_b, c->sm_count);
  if (rc != 0) return c->fail(OMNI_ERR_UNSUPPORTED, "conv plan refused (%d): N=%d C=%d taps=%d T=%d", rc, N, C, taps, T);
  OPS_CUDA(c, conv_launch(plan, c->err, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_overlap_add(omni_ops* c, const void* z, const void* bias, void* state, const int32_t* lines,
                                  const int32_t* pos, int64_t stride, int64_t prev_offset, void* out, int32_t n, int32_t L,
                                  int32_t r, int32_t C) {
  if (!c || !z || !bias || !state || !lines || !out || C % 8) return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_overlap_add((const bf16*)z, (const bf16*)bias, CodecStateRef{(char*)state, lines, pos, stride},
                                       prev_offset, (bf16*)out, n, L, r, C, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_dwconv_ln(omni_ops* c, const void* z, const void* zb, const void* w, const void* b, const void* ln_w,
                                const void* ln_b, void* state, const int32_t* lines, const int32_t* pos, int64_t stride,
                                int64_t hist_offset, void* xin, void* out, int32_t n, int32_t T, int32_t r, int32_t C,
                                float eps) {
  if (!c || !z || !zb || !w || !b || !ln_w || !ln_b || !state || !lines || !pos || !xin || !out || C % 8 || C > 8192)
    return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_dwconv_ln((const bf16*)z, (const bf16*)zb, (const bf16*)w, (const bf16*)b, (const bf16*)ln_w,
                                     (const bf16*)ln_b, CodecStateRef{(char*)state, lines, pos, stride}, hist_offset,
                                     (bf16*)xin, (bf16*)out, n, T, r, C, eps, c->stream));
  return OMNI_OK;
}

int32_t omni_op_codec_out_conv(omni_ops* c, const void* x, const void* bias, const float* alpha, const float* inv_b,
                               const void* w, const void* wb, void* state, const int32_t* lines, const int32_t* pos,
                               int64_t stride, int64_t hist_offset, float* wav, int32_t n, int32_t T, int32_t C) {
  if (!c || !x || !bias || !alpha || !inv_b || !w || !wb || !state || !lines || !pos || !wav || T % 64 || C % 32 || C > 128)
    return OMNI_ERR_INVALID;
  OPS_CUDA(c, launch_codec_out_conv((const bf16*)x, (const bf16*)bias, alpha, inv_b, (const bf16*)w, (const bf16*)wb,
                                    CodecStateRef{(char*)state, lines, pos, stride}, hist_offset, wav, n, T, C, c->stream));
  return OMNI_OK;
}

}  // extern "C"
