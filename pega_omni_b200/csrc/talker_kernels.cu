// Talker / code-predictor glue: embedding gathers, the frame embedding, the
// predictor's first input and the fused sampler. Value semantics follow
// crates/omni-qwen3-tts/kernels/talker.cu; ids outside their tables raise the
// device error word instead of reading out of bounds.
#include "kernels.h"

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
  *reinterpret_cast<Pack8*>(out + (int64_t)blockIdx.x * dim + c) =
      *reinterpret_cast<const Pack8*>(table + id * dim + c);
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
  *reinterpret_cast<Pack8*>(out + ((int64_t)2 * s + blockIdx.y) * dim + c) = *reinterpret_cast<const Pack8*>(src + c);
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

// ---- token selection ------------------------------------------------------------
//
// One 1024-thread block per row, four consecutive logits per thread, vocabulary
// at most 4096. The chain is the one of talker.cu:108-293: repetition penalty
// and suppression on the raw logits, temperature, top-k with ties kept (the
// k-th largest found by a radix select over order-preserving integer keys),
// softmax numerators with __expf, and an inverse-CDF walk in vocabulary order
// against one uniform. To land on the same token as the reference for the same
// logits and uniform, the probability prefix sums are associated exactly as its
// block scan does: per-thread sum of four, shuffle-up inclusive scan inside a
// warp, the same scan over the 32 warp totals, exclusive prefix formed as
// (warp_before + inclusive) - own.
// Not in the reference: top_p < 1 (nucleus filter after top-k) and uniforms
// from Philox4x32-10 keyed by the sequence's seed.

constexpr int kSampleThreads = 1024;
constexpr int kPer = 4;
constexpr int kMaxNucleus = 1024;

__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float philox_uniform(uint64_t seed, uint32_t frame, uint32_t group) {
  uint32_t c0 = frame, c1 = group, c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
    const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = h1 ^ c1 ^ k0, n2 = h0 ^ c3 ^ k1;
    c0 = n0, c1 = l1, c2 = n2, c3 = l0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return (float)(c0 >> 8) * (1.0f / 16777216.0f);
}

struct SampleShared {
  uint32_t hist[256];
  float red[32];
  float scan[32];
  uint32_t sel_prefix, sel_left;
  int token, last;
  unsigned long long best;
  int n_cand;
  int cand_idx[kMaxNucleus];
  float cand_p[kMaxNucleus];
  int sorted_idx[kMaxNucleus];
  float sorted_p[kMaxNucleus];
  uint32_t drop[128];
};

// The k-th largest key among the row's keys (ties share it): four 8-bit digits
// from the top, each pass histogramming the keys that match the digits fixed so far.
__device__ uint32_t kth_largest_key(const uint32_t* key, int vocab, uint32_t k, SampleShared& sh) {
  const int tid = threadIdx.x;
  uint32_t prefix = 0, left = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) sh.hist[tid] = 0;
    __syncthreads();
    const uint32_t fixed = shift == 24 ? 0u : 0xffffffffu << (shift + 8);
#pragma unroll
    for (int j = 0; j < kPer; ++j)
      if (tid * kPer + j < vocab && ((key[j] ^ prefix) & fixed) == 0) atomicAdd(&sh.hist[(key[j] >> shift) & 255], 1u);
    __syncthreads();
    if (tid < 32) {
      // lane t holds digits 8t..8t+7; count of keys in strictly higher lanes via a suffix scan
      uint32_t c[8], mine = 0;
#pragma unroll
      for (int b = 0; b < 8; ++b) mine += c[b] = sh.hist[tid * 8 + b];
      uint32_t suffix = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t other = __shfl_down_sync(0xffffffffu, suffix, o);
        if (tid + o < 32) suffix += other;
      }
      uint32_t above = suffix - mine;
#pragma unroll
      for (int b = 7; b >= 0; --b) {
        if (above < left && above + c[b] >= left) {
          sh.sel_prefix = prefix | (uint32_t)(tid * 8 + b) << shift;
          sh.sel_left = left - above;
        }
        above += c[b];
      }
    }
    __syncthreads();
    prefix = sh.sel_prefix;
    left = sh.sel_left;
  }
  return prefix;
}

// Exclusive prefix of `own` across the block in thread order, and the block total.
__device__ float exclusive_scan(float own, float* total, SampleShared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) sh.scan[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    float wsum = sh.scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, wsum, o);
      if (lane >= o) wsum += up;
    }
    sh.scan[lane] = wsum;
  }
  __syncthreads();
  const float before = warp > 0 ? sh.scan[warp - 1] : 0.f;
  *total = sh.scan[31];
  __syncthreads();
  return before + incl - own;
}

__device__ int draw_token(const float* v, int vocab, float temperature, int top_k, float top_p, float u,
                          SampleShared& sh) {
  const int tid = threadIdx.x;
  if (temperature <= 0.f) {  // argmax, lowest index on ties
    if (tid == 0) sh.best = 0ull;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = tid * kPer + j;
      if (i < vocab) atomicMax(&sh.best, (unsigned long long)order_key(v[j]) << 32 | (uint32_t)(4095 - i));
    }
    __syncthreads();
    return 4095 - (int)(sh.best & 0xffffffffull);
  }
  float x[kPer];
  uint32_t key[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    x[j] = v[j] / temperature;
    key[j] = order_key(x[j]);
  }
  const int keep = top_k > 0 && top_k < vocab ? top_k : vocab;
  const uint32_t threshold = keep < vocab ? kth_largest_key(key, vocab, (uint32_t)keep, sh) : 0u;
  const float m = block_fmax(fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3])), sh.red);
  float p[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) p[j] = tid * kPer + j < vocab && key[j] >= threshold ? __expf(x[j] - m) : 0.f;

  if (top_p < 1.f) {
    // compact the survivors, rank them by (probability desc, index asc), walk the
    // ranking once and drop every token whose preceding mass already reaches top_p
    if (tid == 0) sh.n_cand = 0;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kPer; ++j)
      if (p[j] > 0.f) {
        const int at = atomicAdd(&sh.n_cand, 1);
        if (at < kMaxNucleus) {
          sh.cand_idx[at] = tid * kPer + j;
          sh.cand_p[at] = p[j];
        }
      }
    __syncthreads();
    const int nc = min(sh.n_cand, kMaxNucleus);
    for (int a = tid; a < nc; a += blockDim.x) {
      const float pa = sh.cand_p[a];
      const int ia = sh.cand_idx[a];
      int rank = 0;
      for (int b = 0; b < nc; ++b) {
        const float pb = sh.cand_p[b];
        rank += (pb > pa) || (pb == pa && sh.cand_idx[b] < ia);
      }
      sh.sorted_idx[rank] = ia;
      sh.sorted_p[rank] = pa;
    }
    __syncthreads();
    if (tid < 128) sh.drop[tid] = 0u;
    __syncthreads();
    if (tid == 0) {
      float tot = 0.f;
      for (int r = 0; r < nc; ++r) tot += sh.sorted_p[r];
      float before = 0.f;
      for (int r = 0; r < nc; ++r) {
        const float mine = sh.sorted_p[r];
        if (r > 0 && before >= top_p * tot) {
          const int idx = sh.sorted_idx[r];
          sh.drop[idx >> 5] |= 1u << (idx & 31);
        }
        before += mine;
      }
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = tid * kPer + j;
      if (sh.drop[i >> 5] >> (i & 31) & 1u) p[j] = 0.f;
    }
  }

  float own = 0.f;
#pragma unroll
  for (int j = 0; j < kPer; ++j) own += p[j];
  if (tid == 0) {
    sh.token = -1;
    sh.last = 0;
  }
  float total;
  float run = exclusive_scan(own, &total, sh);
  const float target = u * total;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    if (p[j] > 0.f) {
      atomicMax(&sh.last, tid * kPer + j);
      if (run <= target && target < run + p[j]) atomicMax(&sh.token, tid * kPer + j);
    }
    run += p[j];
  }
  __syncthreads();
  return sh.token >= 0 ? sh.token : sh.last;
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const bf16* __restrict__ logits, SampleParams prm,
                                                                const int32_t* __restrict__ frames,
                                                                const float* __restrict__ uniforms,
                                                                const int32_t* __restrict__ force, SlotState st,
                                                                int32_t* __restrict__ codes) {
  __shared__ SampleShared sh;
  const int s = blockIdx.x, tid = threadIdx.x;
  int32_t* own = slot_of(st, s);
  uint32_t* seen = reinterpret_cast<uint32_t*>(own + kGroups);
  const int forced = force[s * kGroups + prm.group];
  int token = forced;
  if (forced < 0) {
    const bf16* l = logits + (int64_t)s * prm.vocab;
    const int frame = frames[s];
    const bool exempt_blocked = frame < prm.min_frames;
    float v[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int i = tid * kPer + j;
      float x = -INFINITY;
      if (i < prm.vocab) {
        x = __bfloat162float(l[i]);
        if (prm.penalize && (seen[i / 32] >> (i % 32) & 1u)) x = x > 0.f ? x / prm.penalty : x * prm.penalty;
        const bool in_range = i >= prm.suppress_lo && i < prm.suppress_hi;
        if ((in_range && i != prm.exempt) || (i == prm.exempt && exempt_blocked)) x = -INFINITY;
      }
      v[j] = x;
    }
    float u;
    if (prm.philox) {
      const uint64_t seed = *reinterpret_cast<const uint64_t*>(seen + prm.seen_words + (prm.seen_words & 1));
      u = philox_uniform(seed, (uint32_t)frame, (uint32_t)prm.group);
    } else {
      u = uniforms[s * kGroups + prm.group];
    }
    token = min(max(draw_token(v, prm.vocab, prm.temperature, prm.top_k, prm.top_p, u, sh), 0), prm.vocab - 1);
  }
  __syncthreads();
  if (tid == 0) {
    codes[s * kGroups + prm.group] = token;
    own[prm.group] = token;
    if (prm.penalize) seen[token / 32] |= 1u << (token % 32);
  }
}

cudaError_t launch_sample(const bf16* logits, const SampleParams& p, const int32_t* frames, const float* uniforms,
                          const int32_t* force, SlotState st, int32_t* codes, int rows, cudaStream_t s) {
  if (p.vocab > kSampleThreads * kPer || p.vocab < 1) return cudaErrorInvalidValue;
  sample_kernel<<<rows, kSampleThreads, 0, s>>>(logits, p, frames, uniforms, force, st, codes);
  return cudaGetLastError();
}

}  // namespace omni
