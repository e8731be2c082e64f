/* omni_b200_ops.h — operator-level C ABI: each kernel of the token loop on its
 * own, over caller-owned DEVICE buffers. The reference exposes its kernels as
 * named ops of a manifest (`Gen::launch` / `Gen::gemm_rows`,
 * crates/omni-kern/src/lib.rs:103-224); these entry points are the same ops as
 * plain calls, used by the parity tests and micro-benchmarks. All tensors are
 * bf16 row-major unless stated; every call is asynchronous on the context's
 * stream, `omni_ops_sync` waits and returns the device error word.
 */
#ifndef OMNI_B200_OPS_H
#define OMNI_B200_OPS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct omni_ops omni_ops;

enum omni_gemm_path {
  OMNI_GEMM_AUTO = 0,
  OMNI_GEMM_VECTOR = 1,
  OMNI_GEMM_TENSOR = 2,      /* weights on the MMA M dimension, split-K */
  OMNI_GEMM_TENSOR_ROWS = 3  /* input rows on the MMA M dimension (rows <= 128, K <= 4096), no split */
};
enum omni_epilogue { OMNI_EPI_NONE = 0, OMNI_EPI_BIAS = 1, OMNI_EPI_BIAS_SILU = 2 };

int32_t omni_ops_create(int32_t device, omni_ops** out);
void omni_ops_destroy(omni_ops* ctx);
/* Waits for the context's stream; returns 0, OMNI_ERR_CUDA (-2) or, when a
 * kernel raised the device error word, OMNI_ERR_DEVICE (-3) with the word in *word. */
int32_t omni_ops_sync(omni_ops* ctx, uint32_t* word);
/* Device time in ms between the two most recent omni_ops_mark calls (CUDA events on the context's stream). */
int32_t omni_ops_mark(omni_ops* ctx, int32_t which /* 0 = begin, 1 = end */);
int32_t omni_ops_elapsed_ms(omni_ops* ctx, float* ms);
const char* omni_ops_last_error(const omni_ops* ctx);

/* y[rows, N] = x[rows, K] . w[N, K]^T, the `extern:cublaslt_bf16_tn` op of
 * crates/omni-kern/src/lib.rs:159-173, with an optional fused bias epilogue
 * (`talker_bias` / `talker_bias_silu`, talker.cu:45-51). splits = 0 lets the
 * library choose the K split of the tensor-core path. */
int32_t omni_op_gemm(omni_ops* ctx, const void* w, int32_t N, int32_t K, const void* x, int32_t rows, void* y,
                     int32_t ldy, int32_t path, int32_t splits, const void* bias, int32_t epilogue);

/* `qwen3_norm_copy` (crates/omni-qwen3/kernels/qwen3.cu:18-31). */
int32_t omni_op_norm_copy(omni_ops* ctx, const void* x, const void* w, void* out, void* res, int32_t rows,
                          int32_t dim, float eps);
/* `qwen3_add_norm` (qwen3.cu:37-57). */
int32_t omni_op_add_norm(omni_ops* ctx, const void* x, void* res, const void* w, void* out, int32_t rows, int32_t dim,
                         float eps, int32_t every, int32_t which);
/* `qwen3_silu_mul` (qwen3.cu:59-61). */
int32_t omni_op_silu_mul(omni_ops* ctx, const void* gate_up, void* act, int32_t rows, int32_t inter);

/* `qwen3_rope` + `qwen3_attend` (qwen3.cu:109-240) over a paged KV in this
 * library's layout kv[page][kv_head][K|V][16][head_dim]. Row n sits at pos[n],
 * writes slot[n] = page*16 + pos%16, belongs to sequence seq[n] (NULL: row n is
 * sequence n) whose pages are pages[indptr[s]..]. qkv: [rows, (hq+2hk)*d], q is
 * normed and rotated in place; out: [rows, hq*d]. */
int32_t omni_op_rope_attend(omni_ops* ctx, void* qkv, const void* q_norm, const void* k_norm, void* kv,
                            int32_t kv_pages, const int32_t* pos, const int32_t* slot, const int32_t* seq,
                            const int32_t* indptr, const int32_t* pages, int32_t rows, int32_t q_heads,
                            int32_t kv_heads, int32_t head_dim, float eps, float theta, void* out);

/* `talker_sample` (crates/omni-qwen3-tts/kernels/talker.cu:259-293). state:
 * per-sequence slots of `stride` bytes, each i32 last_frame[16], u32
 * seen[ceil(vocab/32)], then (8-byte aligned) the u64 Philox seed. */
int32_t omni_op_sample(omni_ops* ctx, const void* logits, int32_t vocab, float temperature, int32_t top_k,
                       float top_p, float penalty, int32_t suppress_lo, int32_t suppress_hi, int32_t exempt,
                       int32_t min_frames, const int32_t* frames, const float* uniforms, const int32_t* force,
                       void* state, const int32_t* lines, int64_t stride, int32_t penalize, int32_t philox,
                       int32_t* codes, int32_t group, int32_t rows);

/* ---- duplex (PersonaPlex) kernels, one call each: crates/omni-personaplex/kernels/lm.cu --------------------------
 * Helium KV layout of this library (one buffer per layer, FP8 E4M3 + one f32 scale per (token, head)):
 *   kv[page][head][ K: 16 tokens x 128 B | V: 16 tokens x 128 B | K scales: 16 x f32 | V scales: 16 x f32 ]
 * a token's slot is page * 16 + ring position % 16. */

/* `lm_norm` (lm.cu:86-92) when y is NULL: out = x * (alpha * rsqrt(eps + mean(x^2))).
 * `lm_add_norm` (lm.cu:95-106) otherwise: x = bf16(x + y), out = norm(x); out NULL: `lm_add` (lm.cu:109-120). */
int32_t omni_op_lm_norm(omni_ops* ctx, const void* y, void* x, const void* alpha, void* out, int32_t rows,
                        int32_t dim, float eps);

/* One rank's side of the tensor-parallel pair's exchange (include/omni_b200_duplex.h; no counterpart in the
 * reference): waits (at most 2 s) until the flag word words[0] has reached this exchange's number words[32] + 1, which
 * it also stores to words[16] (in the model: the peer's flag), then y = bf16(mine + peer), x = bf16(x + y),
 * out = norm(x), and the last CTA advances words[32]. words: 64 zero-initialised u32 in device memory
 * (0: this rank's flag, 16: where the peer's flag is written, 32: exchange counter, 48: CTA counter). With a flag that
 * nothing raises the wait runs out: the device error word is set (status OMNI_ERR_DEVICE at the next
 * omni_ops_sync) and peer counts as zero. This entry exists so that the kernel's arithmetic and its bounded wait can
 * be tested on one GPU. */
int32_t omni_op_lm_tp_add_norm(omni_ops* ctx, const void* mine, const void* peer, void* x, const void* alpha, void* out,
                               int32_t rows, int32_t dim, float eps, void* words);

/* `lm_embed_prompt` (lm.cu:47-59) without voices: out[r] = sum of the embeddings of ids[r][0..17), every add rounded
 * to bf16, audio streams first, -1 = no token. text_emb [text_rows, dim], audio_emb [16 * card_rows, dim]. */
int32_t omni_op_lm_embed(omni_ops* ctx, const int32_t* ids, const void* text_emb, int32_t text_rows,
                         const void* audio_emb, int32_t card_rows, void* out, int32_t rows, int32_t dim);

/* `lm_rope` + `lm_attend` (lm.cu:129-290): rows of [q | k | v] (heads of 128): interleaved rotary embedding, K and V
 * quantised to E4M3 into slot[n], attention of row n (session seq[n], or n when seq is NULL) over the first
 * min(pos[n] + 1, context) ring positions of its pages. q is rotated in place. */
int32_t omni_op_lm_rope_attend(omni_ops* ctx, void* qkv, void* kv, int32_t kv_pages, const int32_t* pos,
                               const int32_t* slot, const int32_t* seq, const int32_t* indptr, const int32_t* pages,
                               int32_t rows, int32_t heads, float coef, float scale, int32_t context, void* out);

/* `lm_dep_embed_norm` (lm.cu:301-313) then `lm_dep_kv_attend` is a separate call below.
 * x = bf16(projected[s][k] + table[drawn[s][k]]), xn = norm(x). */
int32_t omni_op_lm_dep_embed_norm(omni_ops* ctx, const void* projected, int32_t k, const void* table,
                                  int32_t table_rows, const int32_t* drawn, const void* alpha, void* x, void* xn,
                                  int32_t rows, int32_t dim, float eps);

/* `lm_dep_kv_attend` (lm.cu:319-366): step's K and V into ws ([rows][8][K | V][heads * 64]), causal attention over
 * steps 0..step. */
int32_t omni_op_lm_dep_kv_attend(omni_ops* ctx, const void* qkv, void* ws, int32_t step, void* out, int32_t rows,
                                 int32_t heads, float scale);

/* `lm_sample` (lm.cu:423-537): Gumbel-max over the top-k into drawn[s][col]; force[s][col] >= 0 is taken. */
int32_t omni_op_lm_sample(omni_ops* ctx, const void* logits, int32_t vocab, int64_t ld, float temperature,
                          int32_t top_k, const int32_t* force, const int32_t* seeds, int32_t col, int32_t* drawn,
                          int32_t rows);

/* `lm_init` (lm.cu:576-581) when init is not NULL, then `lm_advance` (lm.cu:546-573) when drawn is not NULL. */
int32_t omni_op_lm_advance(omni_ops* ctx, void* state, const int32_t* lines, int64_t stride, const int32_t* init,
                           const int32_t* drawn, const int32_t* caller, const int32_t* force_caller,
                           int32_t* emitted, int32_t rows);

/* ---- Higgs-style speech model glue: crates/omni-higgs-audio/kernels/higgs.cu, src/delay.rs ---------------------- */

/* `higgs_frame_embed` (higgs.cu:24-37): out[s] = bf16(f32 sum over the 8 codebooks of table[b * vocab + code_b]),
 * codes = the first 8 words of the sequence's state slot (state + lines[s] * stride). */
int32_t omni_op_higgs_frame_embed(omni_ops* ctx, void* state, const int32_t* lines, int64_t stride, const void* table,
                                  void* out, int32_t rows, int32_t dim, int32_t vocab);

/* `higgs_sample` (higgs.cu:186-208): eight independent draws per row over logits [rows, 8, vocab] against
 * uniforms [rows, 8]; force [rows, 8] >= 0 is taken (the delay pattern arrives here); codes [rows, 8] and the slot. */
int32_t omni_op_higgs_sample(omni_ops* ctx, const void* logits, int32_t vocab, float temperature, int32_t top_k,
                             const float* uniforms, const int32_t* force, void* state, const int32_t* lines,
                             int64_t stride, int32_t* codes, int32_t rows);

/* `Delay` (crates/omni-higgs-audio/src/delay.rs:19-46), host only: which codebooks the next step does not draw (they
 * read OMNI_HIGGS_BOC) and when generation ends. Zero-initialise for a new run. */
#define OMNI_HIGGS_BOOKS 8
#define OMNI_HIGGS_BOC 1024
#define OMNI_HIGGS_EOC 1025
typedef struct omni_higgs_delay {
  int32_t steps;
  int32_t countdown; /* 0: none running; otherwise steps left + 1 */
  int32_t done;
} omni_higgs_delay;
/* `Delay::forced_from` (delay.rs:27-29): the first codebook the next step does not draw. */
int32_t omni_higgs_delay_forced_from(const omni_higgs_delay* d);
/* `Delay::advance` (delay.rs:33-46): takes the step's codebook 0 draw; 1 when generation has ended. */
int32_t omni_higgs_delay_advance(omni_higgs_delay* d, int32_t first);
/* `undelay` (delay.rs:50-54): frames [max(n_rows - 7, 0), 8] from delayed rows [n_rows, 8]; returns the frame count. */
int32_t omni_higgs_undelay(const int32_t* rows, int32_t n_rows, int32_t* frames);

/* The tensor-core GEMM of omni_op_gemm for callers that cannot allocate device memory. It has no counterpart in the
 * reference. Two kinds of caller are meant: a serving process that handed every free byte of HBM to its KV pool at
 * start-up, where a later cudaMalloc simply fails; and an engine thread in the middle of a live tick, where
 * cudaMalloc / cudaFree would synchronise the whole device and stall every other session's stream. This entry
 * point needs no context object and calls no cudaMalloc, cudaFree or allocating library routine: the split-K
 * scratch (f32 partial tiles, tile counters, the error word) is a fixed array inside the library image, present on
 * every GPU that loads the library for as long as the process lives.
 *
 *  - Inputs and outputs are the caller's device buffers, as for omni_op_gemm (tensor-core path only: K a
 *    multiple of 64, operands 16-byte aligned). `stream` is a cudaStream_t (NULL = the default stream).
 *  - Limits: splits * row_tiles * ceil(N/128) * 128 * BN <= 4 Mi floats (BN = rows rounded up to 16/32/64/128/256)
 *    and row_tiles * ceil(N/128) <= 2048. Larger problems are refused with OMNI_ERR_UNSUPPORTED and a message
 *    naming the sizes; nothing is launched.
 *  - The first call on each device looks up the arrays' device addresses (with that device current) and raises the
 *    kernels' shared-memory limits. Make that first call before starting any stream capture on that device.
 *  - All calls share the one array and it keeps the previous call's contents; the counters and the error word are
 *    cleared on the stream before each launch. Two calls whose kernels overlapped on the GPU would race on it, so
 *    the entry point holds a process-wide lock from its set-up until its kernel has finished: calls from several
 *    host threads run one after the other. `stream` must belong to the current device (checked).
 *  - The call waits for its kernel and returns 0, or a negative omni_status with a human-readable reason in
 *    `message` (caller-owned, may be NULL). */
int32_t omni_op_gemm_noalloc(const void* w, int32_t N, int32_t K, const void* x, int32_t rows, void* y, int32_t ldy,
                             int32_t splits, const void* bias, int32_t epilogue, void* stream, char* message,
                             size_t message_len);

/* ---- streaming codec decoder: crates/omni-qwen3-tts/kernels/codec.cu, src/codec.rs -------------------------------
 * A per-stream state is `state + lines[s] * stride` bytes plus the entry's own byte offset; `pos[s]` is the number of
 * frames stream s has decoded before the call (histories are two halves, frame p reads half p & 1 and writes the
 * other). Channel counts are multiples of 8. */

/* `codec_rvq` (codec.cu:66-82): out[s] = [book 0 row codes[s][0] | bf16(f32 sum of books 1..15 rows)], books
 * [16 * book_rows, half]; a codebook-0 code >= book_rows reads as 0. */
int32_t omni_op_codec_rvq(omni_ops* ctx, const int32_t* codes, const void* books, void* out, int32_t n, int32_t half,
                          int32_t book_rows);
/* `codec_add_rms_norm` / `codec_bias_rms_norm` (codec.cu:117-170): v = res + add (add_stride 0: one row for all);
 * res = bf16(v); out = bf16(v * (rsqrt(mean v^2 + eps) * w)); out may be add. dim a multiple of 256 up to 1024. */
int32_t omni_op_codec_add_norm(omni_ops* ctx, const void* add, int64_t add_stride, void* res, const void* w, void* out,
                               int32_t rows, int32_t dim, float eps);
/* `codec_attention` (codec.cu:177-283): rotary embedding of q and k, k and v into the stream's ring
 * (K[72][heads * 64] then V, frame p at p % 72), q against the last min(p + 1, 72) frames. qkv [n, 3 * heads * 64]. */
int32_t omni_op_codec_window_attend(omni_ops* ctx, const void* qkv, void* state, const int32_t* lines, const int32_t* pos,
                                    int64_t stride, int64_t ring_offset, void* out, int32_t n, int32_t heads, float theta);
/* `codec_bias_gelu` (codec.cu:84-98), in place; `codec_bias_snake` (codec.cu:100-109). */
int32_t omni_op_codec_bias_gelu(omni_ops* ctx, void* x, const void* bias, int64_t rows, int32_t cols);
int32_t omni_op_codec_bias_snake(omni_ops* ctx, const void* x, const void* bias, const float* alpha, const float* inv_b,
                                 void* out, int64_t rows, int32_t cols);
/* The input side of `codec_im2col` / `codec_im2col_snake` (codec.cu:291-337) without the im2col matrix:
 * padded[s][r] = r < H ? history row r : bf16(act(x[s * T + r - H] + bias)), act SnakeBeta when alpha is given; the last
 * H rows become the next frame's history. `gather_taps` then writes the reference's matrix from it:
 * col[s * T + t][j * C + c] = padded[s][t + j * dil][c]. */
int32_t omni_op_codec_stage(omni_ops* ctx, const void* x, const void* bias, const float* alpha, const float* inv_b,
                            void* state, const int32_t* lines, const int32_t* pos, int64_t stride, int64_t hist_offset,
                            void* padded, int32_t n, int32_t T, int32_t C, int32_t H);
int32_t omni_op_codec_gather_taps(omni_ops* ctx, const void* padded, void* col, int32_t n, int32_t T, int32_t C,
                                  int32_t taps, int32_t dil);
/* The conv itself as an implicit GEMM on tcgen05 (what `codec_im2col` + the runtime's GEMM compute, codec.rs:60-93):
 * y[s * T + t][n] (+)= sum over taps j, channels c of padded[s][t + j * dil][c] * w[n][j * C + c]; epilogue 0: store,
 * 1: y = bf16(y + a), 2: y = bf16(snake(bf16(a) + bias[n])). taps = 1: padded is the dense [n_streams * T, C] input. */
int32_t omni_op_codec_conv(omni_ops* ctx, const void* w, int32_t N, int32_t C, int32_t taps, int32_t dil,
                           const void* padded, int32_t T, int32_t n_streams, void* y, int32_t epilogue, const void* bias,
                           const float* alpha, const float* inv_b);
/* `codec_col2im` (codec.cu:339-372): transposed conv with kernel 2r, stride r, over z [n, L, 2r * C]. */
int32_t omni_op_codec_overlap_add(omni_ops* ctx, const void* z, const void* bias, void* state, const int32_t* lines,
                                  const int32_t* pos, int64_t stride, int64_t prev_offset, void* out, int32_t n, int32_t L,
                                  int32_t r, int32_t C);
/* `codec_dwconv_ln` (codec.cu:381-446): xin = bf16(z + zb[row % r]); depthwise 7-tap causal conv; LayerNorm -> out. */
int32_t omni_op_codec_dwconv_ln(omni_ops* ctx, const void* z, const void* zb, const void* w, const void* b,
                                const void* ln_w, const void* ln_b, void* state, const int32_t* lines, const int32_t* pos,
                                int64_t stride, int64_t hist_offset, void* xin, void* out, int32_t n, int32_t T, int32_t r,
                                int32_t C, float eps);
/* `codec_conv_out` (codec.cu:455-513): last SnakeBeta, the C -> 1 conv of 7 taps, the clamp; wav f32 [n][T] (the
 * reference stores the same values as bf16). T a multiple of 64, C a multiple of 32 up to 128. */
int32_t omni_op_codec_out_conv(omni_ops* ctx, const void* x, const void* bias, const float* alpha, const float* inv_b,
                               const void* w, const void* wb, void* state, const int32_t* lines, const int32_t* pos,
                               int64_t stride, int64_t hist_offset, float* wav, int32_t n, int32_t T, int32_t C);

#ifdef __cplusplus
}
#endif
#endif /* OMNI_B200_OPS_H */
