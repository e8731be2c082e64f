// Talker / code-predictor glue: embedding gathers, the frame embedding, the
// predictor's first input and the fused sampler. Value semantics follow
// crates/omni-qwen3-tts/kernels/talker.cu; ids outside their tables raise the
// device error word instead of reading out of bounds.
#include "kernels.h"
#include "sampler.cuh"

namespace omni {

constexpr int kGroups = 16;

__global__ void gather_kernel(const int32_t* __restrict__ ids, int stride, const bf16* __restrict__ table,
                              int table_rows, bf16* __restrict__ out, int dim, uint32_t* err) {
  const int c = threadIdx.x * 8;
  int64_t id = ids[(int64_t)blockIdx.x * stride];
  if (id < 0 || id >= table_rows) {
    if (threadIdx.x == 0) raise(err, kErrBadIndex);
    id = 0;
  }
  *reinterpret_cast<uint4*>(out + (int64_t)blockIdx.x * dim + c) =
      *reinterpret_cast<const uint4*>(table + id * dim + c);
}

// `talker_prompt_codec` (talker.cu:55-71): x + bias (+ codec embedding), one rounding.
__global__ void prompt_codec_kernel(bf16* __restrict__ x, const bf16* __restrict__ bias,
                                    const bf16* __restrict__ table, int table_rows, const int32_t* __restrict__ ids,
                                    int dim, uint32_t* err) {
  const int c = threadIdx.x * 8;
  bf16* row = x + (int64_t)blockIdx.x * dim + c;
  int id = ids[blockIdx.x];
  if (id >= table_rows) {
    if (threadIdx.x == 0) raise(err, kErrBadIndex);
    id = -1;
  }
  float v[8], b[8], e[8];
  ld8(row, v);
  ld8(bias + c, b);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] += b[k];
  if (id >= 0) {
    ld8(table + (int64_t)id * dim + c, e);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] += e[k];
  }
  st8(row, v);
}

__device__ __forceinline__ int32_t* slot_of(const SlotState& st, int s) {
  return reinterpret_cast<int32_t*>(static_cast<char*>(st.state) + (int64_t)st.lines[s] * st.stride);
}

// `talker_frame_embed` (talker.cu:76-96): f32 sum in the order pad, codebook 0,
// codebooks 1.., one rounding.
__global__ void frame_embed_kernel(SlotState st, const bf16* __restrict__ pad, const bf16* __restrict__ codec_emb,
                                   int vocab, const bf16* __restrict__ p_emb, int p_vocab, int groups,
                                   bf16* __restrict__ out, int dim, uint32_t* err) {
  const int s = blockIdx.x, c = threadIdx.x * 8;
  const int32_t* codes = slot_of(st, s);
  float acc[8], e[8];
  ld8(pad + c, acc);
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f + acc[k];
  int c0 = codes[0];
  if (c0 < 0 || c0 >= vocab) {
    if (threadIdx.x == 0) raise(err, kErrBadIndex);
    c0 = 0;
  }
  ld8(codec_emb + (int64_t)c0 * dim + c, e);
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] += e[k];
  for (int g = 1; g < groups; ++g) {
    int cg = codes[g];
    if (cg < 0 || cg >= p_vocab) {
      if (threadIdx.x == 0) raise(err, kErrBadIndex);
      cg = 0;
    }
    ld8(p_emb + ((int64_t)(g - 1) * p_vocab + cg) * dim + c, e);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += e[k];
  }
  st8(out + (int64_t)s * dim + c, acc);
}

// `talker_pred_input` (talker.cu:100-106).
__global__ void pred_input_kernel(const bf16* __restrict__ hidden, const bf16* __restrict__ codec_emb, int vocab,
                                  const int32_t* __restrict__ codes, bf16* __restrict__ out, int dim, uint32_t* err) {
  const int s = blockIdx.x, c = threadIdx.x * 8;
  const bf16* src;
  if (blockIdx.y == 0) {
    src = hidden + (int64_t)s * dim;
  } else {
    int id = codes[s * kGroups];
    if (id < 0 || id >= vocab) {
      if (threadIdx.x == 0) raise(err, kErrBadIndex);
      id = 0;
    }
    src = codec_emb + (int64_t)id * dim;
  }
  *reinterpret_cast<uint4*>(out + ((int64_t)2 * s + blockIdx.y) * dim + c) = *reinterpret_cast<const uint4*>(src + c);
}

cudaError_t launch_gather(const int32_t* ids, int stride, const bf16* table, int table_rows, bf16* out, int rows,
                          int dim, uint32_t* err, cudaStream_t s) {
  gather_kernel<<<rows, dim / 8, 0, s>>>(ids, stride, table, table_rows, out, dim, err);
  return cudaGetLastError();
}

cudaError_t launch_prompt_codec(bf16* x, const bf16* bias, const bf16* table, int table_rows, const int32_t* ids,
                                int rows, int dim, uint32_t* err, cudaStream_t s) {
  prompt_codec_kernel<<<rows, dim / 8, 0, s>>>(x, bias, table, table_rows, ids, dim, err);
  return cudaGetLastError();
}

cudaError_t launch_frame_embed(SlotState st, const bf16* pad, const bf16* codec_emb, int vocab, const bf16* p_emb,
                               int p_vocab, int groups, bf16* out, int rows, int dim, uint32_t* err, cudaStream_t s) {
  frame_embed_kernel<<<rows, dim / 8, 0, s>>>(st, pad, codec_emb, vocab, p_emb, p_vocab, groups, out, dim, err);
  return cudaGetLastError();
}

cudaError_t launch_pred_input(const bf16* hidden, const bf16* codec_emb, int vocab, const int32_t* codes, bf16* out,
                              int rows, int dim, uint32_t* err, cudaStream_t s) {
  pred_input_kernel<<<dim3(rows, 2), dim / 8, 0, s>>>(hidden, codec_emb, vocab, codes, out, dim, err);
  return cudaGetLastError();
}

// ---- token selection ----------------------------------------------------------
// One 1024-thread block per row; the algorithm lives in sampler.cuh.

__global__ void __launch_bounds__(1024) sample_kernel(const bf16* __restrict__ logits, sampler::Params prm,
                                                      const int32_t* __restrict__ frames,
                                                      const float* __restrict__ uniforms,
                                                      const int32_t* __restrict__ force, SlotState st,
                                                      int32_t* __restrict__ codes) {
  using Team = sampler::Team<1024, sampler::CtaSync>;
  __shared__ sampler::Shared sh;
  const int s = blockIdx.x;
  const bf16* l = logits + (int64_t)s * prm.vocab;
  int32_t* slot = slot_of(st, s);
  Team::sample_row([&](int i, int) { return __bfloat162float(l[i]); }, prm, frames[s], uniforms[s * kGroups + prm.group],
                   force[s * kGroups + prm.group], slot, Team::seen_word(slot, prm, threadIdx.x),
                   codes + s * kGroups + prm.group, threadIdx.x, sh);
}

cudaError_t launch_sample(const bf16* logits, const SampleParams& p, const int32_t* frames, const float* uniforms,
                          const int32_t* force, SlotState st, int32_t* codes, int rows, cudaStream_t s) {
  if (p.vocab > sampler::kVocabMax || p.vocab < 1) return cudaErrorInvalidValue;
  // the nucleus filter ranks at most kMaxNucleus survivors of the top-k cut: without a cut that small it would
  // silently drop candidates in arrival order
  if (p.top_p < 1.f && (p.top_k <= 0 || p.top_k > sampler::kMaxNucleus)) return cudaErrorInvalidValue;
  sampler::Params prm{p.vocab,  p.temperature, p.top_k,    p.top_p, p.penalty, p.suppress_lo, p.suppress_hi,
                      p.exempt, p.min_frames,  p.penalize, p.group, p.philox,  p.seen_words};
  sample_kernel<<<rows, 1024, 0, s>>>(logits, prm, frames, uniforms, force, st, codes);
  return cudaGetLastError();
}

}  // namespace omni
