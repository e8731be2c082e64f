// Host-side launchers of every non-GEMM kernel of the token loop.
//
// KV layout (one buffer per decoder layer):
//   kv[page][kv_head][K | V][16 tokens][head_dim]   bf16
// so one (page, head) holds its 16 keys and its 16 values in one contiguous
// 2 * 16 * head_dim * 2-byte block. A token's slot is page_id * 16 + pos % 16,
// the same number the reference's `t_slot` input carries. The code predictor's
// per-frame KV uses the same layout with page id = the sequence's row, so one
// set of kernels serves both the paged talker and the dense predictor.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "util.cuh"

namespace omni {

// How rows of a pass map to sequences, positions and KV pages.
struct RowMap {
  // paged (pages != nullptr): row n sits at pos[n], writes slot[n], belongs to
  // sequence seq[n] (or n when seq == nullptr), whose pages are
  // pages[indptr[s] .. indptr[s+1]).
  const int32_t* pos = nullptr;
  const int32_t* slot = nullptr;
  const int32_t* seq = nullptr;
  const int32_t* indptr = nullptr;
  const int32_t* pages = nullptr;
  // dense (pages == nullptr): `per` consecutive rows per sequence at positions
  // base, base+1, ...; sequence s uses page s.
  int per = 1, base = 0;
};

struct AttnShape {
  int q_heads, kv_heads, head_dim;
  float rms_eps, rope_theta;
};

// res = x; out = bf16(x * rsqrt(mean(x^2) + eps) * w). One block per row.
cudaError_t launch_norm_copy(const bf16* x, const bf16* w, bf16* out, bf16* res, int rows, int dim, float eps,
                             cudaStream_t s);
// res = bf16(x + res); out[n / every] = bf16((x + res) * rsqrt(..) * w) for rows n % every == which.
cudaError_t launch_add_norm(const bf16* x, bf16* res, const bf16* w, bf16* out, int rows, int dim, float eps,
                            int every, int which, cudaStream_t s);
// act = bf16(bf16(silu(gate)) * up) over fused [gate | up] rows (interleaved = g > 0: g gate channels, g up, g gate, ...).
cudaError_t launch_silu_mul(const bf16* gate_up, bf16* act, int rows, int inter, int interleaved, cudaStream_t s);
// Per-head RMSNorm of q and k, rotary embedding, K and V into the row's slot; q in place.
cudaError_t launch_rope_kv(bf16* qkv, const bf16* q_norm, const bf16* k_norm, bf16* kv, const RowMap& map, int rows,
                           const AttnShape& a, int kv_pages, uint32_t* err, cudaStream_t s);
// Decode/prefill attention of every row over positions 0..pos of its sequence.
cudaError_t launch_attend(const bf16* qkv, const bf16* kv, bf16* out, const RowMap& map, int rows, const AttnShape& a,
                          uint32_t* err, cudaStream_t s);

// out[r] = table[ids[r * stride]]
cudaError_t launch_gather(const int32_t* ids, int stride, const bf16* table, int table_rows, bf16* out, int rows,
                          int dim, uint32_t* err, cudaStream_t s);
// x[r] = bf16(x[r] + bias (+ table[ids[r]] when ids[r] >= 0))
cudaError_t launch_prompt_codec(bf16* x, const bf16* bias, const bf16* table, int table_rows, const int32_t* ids,
                                int rows, int dim, uint32_t* err, cudaStream_t s);

struct SlotState {
  void* state;           // base of the per-sequence state pool
  const int32_t* lines;  // slot index of each row of the call
  int64_t stride;        // bytes per slot
};

// out[s] = bf16(pad + codec_emb[c0] + sum_g p_emb[(g-1) * p_vocab + c_g]) from the slot's last frame.
cudaError_t launch_frame_embed(SlotState st, const bf16* pad, const bf16* codec_emb, int vocab, const bf16* p_emb,
                               int p_vocab, int groups, bf16* out, int rows, int dim, uint32_t* err, cudaStream_t s);
// out[2s] = hidden[s]; out[2s+1] = codec_emb[codes[s*16]].
cudaError_t launch_pred_input(const bf16* hidden, const bf16* codec_emb, int vocab, const int32_t* codes, bf16* out,
                              int rows, int dim, uint32_t* err, cudaStream_t s);

struct SampleParams {
  int vocab;
  float temperature;
  int top_k;
  float top_p;
  float penalty;
  int suppress_lo, suppress_hi, exempt, min_frames;
  int penalize;  // group 0: repetition penalty over the slot's bitmap
  int group;
  int philox;    // uniforms from Philox keyed by the slot's seed instead of `uniforms`
  int seen_words;  // 32-bit words of the slot's bitmap (offset of the seed behind it)
};

// One block per row: logits processors + draw; writes codes[s*16+group], the slot's last frame and bitmap.
cudaError_t launch_sample(const bf16* logits, const SampleParams& p, const int32_t* frames, const float* uniforms,
                          const int32_t* force, SlotState st, int32_t* codes, int rows, cudaStream_t s);

// out[s] = bf16(sum over the 8 codebooks of table[b * vocab + code_b]) from the slot's last frame (i32 codes[8]).
cudaError_t launch_higgs_frame_embed(SlotState st, const bf16* table, bf16* out, int rows, int dim, int vocab,
                                     uint32_t* err, cudaStream_t s);
// A block per (row, codebook) over logits [rows, 8, vocab]: temperature, top-k with ties, draw against
// uniforms[row][b]; force[row][b] >= 0 is taken; writes codes[row][b] and word b of the row's slot.
cudaError_t launch_higgs_sample(const bf16* logits, int vocab, float temperature, int top_k, const float* uniforms,
                                const int32_t* force, SlotState st, int32_t* codes, int rows, cudaStream_t s);

}  // namespace omni
