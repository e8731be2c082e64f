// Launchers of the non-GEMM kernels of the duplex (PersonaPlex) token loop: the Helium temporal transformer with an
// FP8 ring KV, the depformer's per-codebook passes, the Gumbel-max draw and the token bookkeeping.
// Value semantics follow crates/omni-personaplex/kernels/lm.cu; the memory layout is this library's own.
//
// Helium KV (one buffer per layer), FP8 E4M3 with one f32 scale per (token, head):
//   kv[page][head][ K: 16 tokens x 128 B | V: 16 tokens x 128 B | K scales: 16 x f32 | V scales: 16 x f32 ]
// so one (page, head) is one contiguous block of kDuplexPageHeadBytes; a token's slot is page * 16 + ring_pos % 16.
// Bytes per token and layer are the reference's (2 * heads * 128 + 2 * heads * 4, helium.rs:84).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "util.cuh"

namespace omni {

constexpr int kDuplexStreams = 17;  // text, the agent's 8 codebooks, the caller's 8 (config.rs:26)
constexpr int kDuplexBooks = 8;
constexpr int kDuplexDrawn = 1 + kDuplexBooks;
constexpr int kDuplexStateWords = kDuplexStreams + kDuplexBooks - 1;  // input row + pending caller codes
constexpr int kHeliumHeadDim = 128;
constexpr int kDepHeadDim = 64;
constexpr int kDepSteps = 8;
constexpr int kDuplexPageHeadBytes = 2 * 16 * kHeliumHeadDim + 2 * 16 * 4;

struct DuplexTables {
  const bf16* text_emb;   // [text_vocab + 1, dim]
  const bf16* audio_emb;  // [16 * (card + 1), dim]
  int text_rows, card_rows;  // rows per table (text_vocab + 1, card + 1)
};

// out[r] = embedding of row r's 17 ids (`ids`: [rows, 17]); a voice row (voice && voice[r] >= 0) copies voices[voice[r]].
cudaError_t launch_lm_embed_ids(const int32_t* ids, const int32_t* voice, const bf16* voices, int voice_rows,
                                DuplexTables t, bf16* out, int rows, int dim, uint32_t* err, cudaStream_t s);
// out[s] = embedding of session s's input row (first 17 words of its state); the row is also copied to rows_out.
cudaError_t launch_lm_embed_state(const void* state, const int32_t* lines, int64_t stride, DuplexTables t, bf16* out,
                                  int32_t* rows_out, int rows, int dim, uint32_t* err, cudaStream_t s);
// out = x * (alpha * rsqrt(eps + mean(x^2)))
cudaError_t launch_lm_norm(const bf16* x, const bf16* alpha, bf16* out, int rows, int dim, float eps, cudaStream_t s);
// x = bf16(x + y); out = norm(x) (out == nullptr: the add alone)
cudaError_t launch_lm_add_norm(const bf16* y, bf16* x, const bf16* alpha, bf16* out, int rows, int dim, float eps,
                               cudaStream_t s);
// The words of a tensor-parallel pair's exchange: `my_flag` lives in this rank's memory and is written by the peer,
// `peer_flag` is the peer's, mapped here; `counter` numbers the exchanges, `finished` counts a launch's CTAs.
struct TpLink {
  uint32_t *my_flag = nullptr, *peer_flag = nullptr, *counter = nullptr, *finished = nullptr;
};
// y = bf16(mine + peer) over both ranks' partial rows, then x = bf16(x + y); out = norm(x) (out == nullptr: the add alone)
cudaError_t launch_lm_tp_add_norm(const bf16* mine, const bf16* peer, bf16* x, const bf16* alpha, bf16* out, int rows,
                                  int dim, float eps, const TpLink& link, uint32_t* err, cudaStream_t s);
// Rows [q | k | v] of `heads` heads of 128: interleaved rotary embedding of q in place; k rotated, then k and v
// quantised per head to E4M3 with scale max(amax / 448, 1e-12) into the row's slot.
cudaError_t launch_lm_rope_kv(bf16* qkv, const int32_t* pos, const int32_t* slots, void* kv, int rows, int heads,
                              float coef, int kv_pages, uint32_t* err, cudaStream_t s);
// Row n of session (seq ? seq[n] : n) attends to the first min(pos[n] + 1, context) ring positions of its session.
cudaError_t launch_lm_attend(const bf16* qkv, const void* kv, const int32_t* pos, const int32_t* seq,
                             const int32_t* indptr, const int32_t* pages, bf16* out, int rows, int heads, float scale,
                             int context, int kv_pages, uint32_t* err, cudaStream_t s);
// Depformer step k: x = bf16(projected[s][k] + table[drawn[s][k]]); xn = norm(x).
cudaError_t launch_lm_dep_embed_norm(const bf16* projected, int k, const bf16* table, int table_rows,
                                     const int32_t* drawn, const bf16* alpha, bf16* x, bf16* xn, int rows, int dim,
                                     float eps, uint32_t* err, cudaStream_t s);
// Depformer step `step`: K and V of the step into the session's workspace ([8][K | V][heads * 64] per session),
// causal attention over steps 0..step. One warp per (session, head).
cudaError_t launch_lm_dep_kv_attend(const bf16* qkv, bf16* ws, int step, bf16* out, int rows, int heads, float scale,
                                    cudaStream_t s);
// Gumbel-max draw over the top-k of bf16 logits (row stride ld) into drawn[s][col]; force[s][col] >= 0 is taken as is.
cudaError_t launch_lm_sample(const bf16* logits, int vocab, int64_t ld, float temperature, int top_k,
                             const int32_t* force, const int32_t* seeds, int col, int32_t* drawn, int rows,
                             cudaStream_t s);
// After the draws: the emitted frame, the session's next input row and pending caller codes.
cudaError_t launch_lm_advance(void* state, const int32_t* lines, int64_t stride, const int32_t* drawn,
                              const int32_t* caller, const int32_t* force_caller, int32_t* emitted, int rows,
                              cudaStream_t s);
// state[line s][0 .. 24) = init[s]
cudaError_t launch_lm_init(void* state, const int32_t* lines, int64_t stride, const int32_t* init, int rows,
                           cudaStream_t s);

// Copies `tokens` KV slots of one layer from src_slot[r] to dst_slot[r] (keys, values and both scales of every head):
// a cached prefix into a new session's ring (`lm_copy_kv`, lm.cu:584-593).
cudaError_t launch_lm_copy_kv(void* kv, const int32_t* src_slot, const int32_t* dst_slot, int tokens, int heads,
                              int kv_pages, uint32_t* err, cudaStream_t s);

}  // namespace omni
