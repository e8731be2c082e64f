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

enum omni_gemm_path { OMNI_GEMM_AUTO = 0, OMNI_GEMM_VECTOR = 1, OMNI_GEMM_TENSOR = 2 };
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
 *    cleared on the stream before each launch. Two calls whose kernels overlap on the GPU (different streams or
 *    threads) race on it: serialise them.
 *  - The call waits for its kernel and returns 0, or a negative omni_status with a human-readable reason in
 *    `message` (caller-owned, may be NULL). */
int32_t omni_op_gemm_noalloc(const void* w, int32_t N, int32_t K, const void* x, int32_t rows, void* y, int32_t ldy,
                             int32_t splits, const void* bias, int32_t epilogue, void* stream, char* message,
                             size_t message_len);

#ifdef __cplusplus
}
#endif
#endif /* OMNI_B200_OPS_H */
