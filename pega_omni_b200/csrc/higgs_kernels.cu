// The glue around the Qwen3 body of the Higgs-style speech model: the fused eight-codebook frame embedding and the
// eight independent code draws of a step. Value semantics follow crates/omni-higgs-audio/kernels/higgs.cu; codes
// outside the table raise the device error word instead of reading out of bounds. The draw is the talker's
// (sampler.cuh) without penalty and suppression: the reference's two samplers share their algorithm and the
// association order of their block scan (higgs.cu:66-183, talker.cu:108-257).
#include "kernels.h"
#include "sampler.cuh"

namespace omni {

constexpr int kHiggsBooks = 8;

// `higgs_frame_embed` (higgs.cu:24-37): the f32 sum of the last frame's codebook embeddings (codebook b at row
// b * vocab + code of the fused table), rounded once.
__global__ void higgs_frame_embed_kernel(SlotState st, const bf16* __restrict__ table, bf16* __restrict__ out, int dim,
                                         int vocab, uint32_t* err) {
  const int s = blockIdx.x, c = threadIdx.x * 8;
  const int32_t* codes =
      reinterpret_cast<const int32_t*>(static_cast<const char*>(st.state) + (int64_t)st.lines[s] * st.stride);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, e[8];
  for (int b = 0; b < kHiggsBooks; ++b) {
    int code = codes[b];
    if (code < 0 || code >= vocab) {
      if (threadIdx.x == 0) raise(err, kErrBadIndex);
      code = 0;
    }
    ld8(table + ((int64_t)b * vocab + code) * dim + c, e);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] += e[k];
  }
  st8(out + (int64_t)s * dim + c, acc);
}

// `higgs_sample` (higgs.cu:186-208): a block per (sequence, codebook) over logits[s][b][vocab]; the code goes to
// codes[s][b] and to word b of the sequence's slot.
__global__ void __launch_bounds__(1024)
    higgs_sample_kernel(const bf16* __restrict__ logits, int vocab, float temperature, int top_k,
                        const float* __restrict__ uniforms, const int32_t* __restrict__ force, SlotState st,
                        int32_t* __restrict__ codes) {
  using Team = sampler::Team<1024, sampler::CtaSync>;
  __shared__ sampler::Shared sh;
  const int s = blockIdx.x, b = blockIdx.y;
  int32_t* own = reinterpret_cast<int32_t*>(static_cast<char*>(st.state) + (int64_t)st.lines[s] * st.stride);
  const bf16* l = logits + ((int64_t)s * kHiggsBooks + b) * vocab;
  sampler::Params prm{};
  prm.vocab = vocab;
  prm.temperature = temperature;
  prm.top_k = top_k;
  prm.top_p = 1.f;
  prm.penalty = 1.f;
  prm.exempt = -1;
  prm.group = b;
  Team::sample_row([&](int i, int) { return __bfloat162float(l[i]); }, prm, 0, uniforms[s * kHiggsBooks + b],
                   force[s * kHiggsBooks + b], own, 0u, codes + s * kHiggsBooks + b, threadIdx.x, sh);
}

cudaError_t launch_higgs_frame_embed(SlotState st, const bf16* table, bf16* out, int rows, int dim, int vocab,
                                     uint32_t* err, cudaStream_t s) {
  if (dim % 8 || dim / 8 > 1024) return cudaErrorInvalidValue;
  higgs_frame_embed_kernel<<<rows, dim / 8, 0, s>>>(st, table, out, dim, vocab, err);
  return cudaGetLastError();
}

cudaError_t launch_higgs_sample(const bf16* logits, int vocab, float temperature, int top_k, const float* uniforms,
                                const int32_t* force, SlotState st, int32_t* codes, int rows, cudaStream_t s) {
  if (vocab < 1 || vocab > sampler::kVocabMax) return cudaErrorInvalidValue;
  higgs_sample_kernel<<<dim3(rows, kHiggsBooks), 1024, 0, s>>>(logits, vocab, temperature, top_k, uniforms, force, st,
                                                               codes);
  return cudaGetLastError();
}

}  // namespace omni
