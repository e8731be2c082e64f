// Non-GEMM kernels of the duplex (PersonaPlex) token loop. Value semantics follow
// crates/omni-personaplex/kernels/lm.cu (line ranges at each kernel); ids, pages and slots outside their tables
// raise the device error word instead of reading out of bounds.
#include <cuda_fp8.h>

#include "duplex.h"

namespace omni {
namespace {

constexpr int kAttendWarps = 4;

__device__ __forceinline__ const int32_t* state_row(const void* state, const int32_t* lines, int s, int64_t stride) {
  return reinterpret_cast<const int32_t*>(static_cast<const char*>(state) + (int64_t)lines[s] * stride);
}

// Σ audio_emb[k][ids[1 + k]] over the 16 audio streams, then + text_emb[ids[0]]; every add rounded to bf16; an id
// of -1 contributes nothing (lm.cu:25-43).
__device__ __forceinline__ void embed_row(const int32_t* ids, const DuplexTables& t, bf16* out, int dim, uint32_t* err) {
  const int c = threadIdx.x * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < kDuplexStreams; ++k) {
    const int stream = k < kDuplexStreams - 1 ? k + 1 : 0;
    const int id = ids[stream];
    if (id < 0) continue;
    if (id >= (stream == 0 ? t.text_rows : t.card_rows)) {
      if (threadIdx.x == 0) raise(err, kErrBadIndex);
      continue;
    }
    const bf16* row = stream == 0 ? t.text_emb + (int64_t)id * dim : t.audio_emb + ((int64_t)k * t.card_rows + id) * dim;
    float e[8];
    ld8(row + c, e);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = bf16_round(acc[j] + e[j]);
  }
  st8(out + c, acc);
}

// `lm_embed_prompt` (lm.cu:47-59)
__global__ void lm_embed_ids_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ voice,
                                    const bf16* __restrict__ voices, int voice_rows, DuplexTables t,
                                    bf16* __restrict__ out, int dim, uint32_t* err) {
  const int64_t r = blockIdx.x;
  if (voice && voice[r] >= 0) {
    int v = voice[r];
    if (v >= voice_rows) {
      if (threadIdx.x == 0) raise(err, kErrBadIndex);
      v = 0;
    }
    const int c = threadIdx.x * 8;
    *reinterpret_cast<Pack8*>(out + r * dim + c) = *reinterpret_cast<const Pack8*>(voices + (int64_t)v * dim + c);
    return;
  }
  embed_row(ids + r * kDuplexStreams, t, out + r * dim, dim, err);
}

// `lm_embed_state` (lm.cu:62-70)
__global__ void lm_embed_state_kernel(const void* state, const int32_t* __restrict__ lines, int64_t stride,
                                      DuplexTables t, bf16* __restrict__ out, int32_t* __restrict__ rows_out, int dim,
                                      uint32_t* err) {
  const int s = blockIdx.x;
  const int32_t* row = state_row(state, lines, s, stride);
  if (threadIdx.x < kDuplexStreams) rows_out[s * kDuplexStreams + threadIdx.x] = row[threadIdx.x];
  embed_row(row, t, out + (int64_t)s * dim, dim, err);
}

// y = x * (alpha * rsqrt(eps + mean(x^2))) (lm.cu:74-84)
__device__ __forceinline__ void norm_row(const float* v, const bf16* alpha, bf16* out, int dim, float eps, float* scratch) {
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
  const float r = rsqrtf(block_add(ss, scratch) / dim + eps);
  float a[8], y[8];
  ld8(alpha + threadIdx.x * 8, a);
#pragma unroll
  for (int k = 0; k < 8; ++k) y[k] = v[k] * (a[k] * r);
  st8(out + threadIdx.x * 8, y);
}

__global__ void lm_norm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ alpha, bf16* __restrict__ out,
                               int dim, float eps) {
  __shared__ float scratch[32];
  const int64_t at = (int64_t)blockIdx.x * dim;
  float v[8];
  ld8(x + at + threadIdx.x * 8, v);
  norm_row(v, alpha, out + at, dim, eps, scratch);
}

// x = bf16(x + y), out = norm(x) over the rounded sum (lm.cu:95-106; out == nullptr: `lm_add`, lm.cu:109-120)
__global__ void lm_add_norm_kernel(const bf16* __restrict__ y, bf16* __restrict__ x, const bf16* __restrict__ alpha,
                                   bf16* __restrict__ out, int dim, float eps) {
  __shared__ float scratch[32];
  const int64_t at = (int64_t)blockIdx.x * dim + threadIdx.x * 8;
  float v[8], u[8];
  ld8(x + at, v);
  ld8(y + at, u);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = bf16_round(v[k] + u[k]);
  st8(x + at, v);
  if (out) norm_row(v, alpha, out + (int64_t)blockIdx.x * dim, dim, eps, scratch);
}

__device__ __forceinline__ uint8_t* page_head(void* kv, int64_t page, int heads, int h) {
  return static_cast<uint8_t*>(kv) + (page * heads + h) * (int64_t)kDuplexPageHeadBytes;
}

__device__ __forceinline__ float e4m3_scale(float amax) { return fmaxf(amax * (1.f / 448.f), 1e-12f); }

// `lm_rope` (lm.cu:129-184): a warp per head of the row.
__global__ void lm_rope_kv_kernel(bf16* __restrict__ qkv, const int32_t* __restrict__ pos,
                                  const int32_t* __restrict__ slots, void* kv, int heads, float coef, int kv_pages,
                                  uint32_t* err) {
  const int n = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (head >= 3 * heads) return;
  const int lane = threadIdx.x & 31;
  bf16* src = qkv + ((int64_t)n * 3 * heads + head) * kHeliumHeadDim;
  const float p = (float)pos[n];
  int64_t slot = slots[n];
  if (slot < 0 || (slot >> 4) >= kv_pages) {
    if (lane == 0) raise(err, kErrBadIndex);
    slot = 0;
  }
  const int tok = (int)(slot & 15);
  if (head < 2 * heads) {
    float out_r[2], out_i[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = lane + k * 32;
      const float freq = expf((float)i * coef);
      float s, c;
      sincosf(freq * p, &s, &c);
      const __nv_bfloat162 pair = *reinterpret_cast<const __nv_bfloat162*>(src + 2 * i);
      const float r = __bfloat162float(pair.x), im = __bfloat162float(pair.y);
      out_r[k] = r * c - im * s;
      out_i[k] = r * s + im * c;
    }
    if (head < heads) {  // q: rounded to bf16 in place
#pragma unroll
      for (int k = 0; k < 2; ++k)
        *reinterpret_cast<__nv_bfloat162*>(src + 2 * (lane + k * 32)) = __floats2bfloat162_rn(out_r[k], out_i[k]);
      return;
    }
    const int h = head - heads;
    const float amax = warp_fmax(fmaxf(fmaxf(fabsf(out_r[0]), fabsf(out_i[0])), fmaxf(fabsf(out_r[1]), fabsf(out_i[1]))));
    const float sc = e4m3_scale(amax), inv = 1.f / sc;
    uint8_t* block = page_head(kv, slot >> 4, heads, h);
    uint8_t* dst = block + tok * kHeliumHeadDim;
#pragma unroll
    for (int k = 0; k < 2; ++k)
      *reinterpret_cast<__nv_fp8x2_storage_t*>(dst + 2 * (lane + k * 32)) =
          __nv_cvt_float2_to_fp8x2(make_float2(out_r[k] * inv, out_i[k] * inv), __NV_SATFINITE, __NV_E4M3);
    if (lane == 0) reinterpret_cast<float*>(block + 2 * 16 * kHeliumHeadDim)[tok] = sc;
  } else {
    const int h = head - 2 * heads;
    float v[4];
    const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
    const float amax = warp_fmax(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
    const float sc = e4m3_scale(amax), inv = 1.f / sc;
    uint8_t* block = page_head(kv, slot >> 4, heads, h);
    uint8_t* dst = block + (16 + tok) * kHeliumHeadDim + lane * 4;
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(dst) = lo | hi << 16;
    if (lane == 0) reinterpret_cast<float*>(block + 2 * 16 * kHeliumHeadDim + 64)[tok] = sc;
  }
}

__device__ __forceinline__ float4 e4m3x4(uint32_t raw) {
  return static_cast<float4>(*reinterpret_cast<const __nv_fp8x4_e4m3*>(&raw));
}

// `lm_attend` / `attend_row_fp8` (lm.cu:197-290): a CTA per (row, head), four warps over tiles of 32 ring positions
// (a lane owns a key for the scores, then four output dims for the values), online softmax per warp, merged at the end.
__global__ void __launch_bounds__(kAttendWarps * 32)
    lm_attend_kernel(const bf16* __restrict__ qkv, const void* kv, const int32_t* __restrict__ pos,
                     const int32_t* __restrict__ seq, const int32_t* __restrict__ indptr,
                     const int32_t* __restrict__ pages, bf16* __restrict__ out, int heads, float scale, int context,
                     int kv_pages, uint32_t* err) {
  const int n = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = seq ? seq[n] : n;
  const int len = min(pos[n] + 1, context);
  const int32_t* my_pages = pages + indptr[s];
  __shared__ float qs[kHeliumHeadDim];
  __shared__ float ms[kAttendWarps], ls[kAttendWarps];
  __shared__ float os[kAttendWarps][kHeliumHeadDim];
  qs[threadIdx.x] = __bfloat162float(qkv[((int64_t)n * 3 * heads + h) * kHeliumHeadDim + threadIdx.x]);
  __syncthreads();
  float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int base = warp * 32; base < len; base += kAttendWarps * 32) {
    const int t = base + lane;
    const bool valid = t < len;
    const int tt = valid ? t : base;
    int64_t page = my_pages[tt >> 4];
    if (page < 0 || page >= kv_pages) {
      raise(err, kErrBadIndex);
      page = 0;
    }
    const uint8_t* block = page_head(const_cast<void*>(kv), page, heads, h);
    const int tok = tt & 15;
    const uint8_t* k = block + tok * kHeliumHeadDim;
    const float ks = reinterpret_cast<const float*>(block + 2 * 16 * kHeliumHeadDim)[tok];
    const float vs = reinterpret_cast<const float*>(block + 2 * 16 * kHeliumHeadDim + 64)[tok];
    float sc = 0.f;
#pragma unroll 2
    for (int c = 0; c < kHeliumHeadDim; c += 16) {
      const uint4 raw = *reinterpret_cast<const uint4*>(k + c);
      const float4 k0 = e4m3x4(raw.x), k1 = e4m3x4(raw.y), k2 = e4m3x4(raw.z), k3 = e4m3x4(raw.w);
      sc += qs[c + 0] * k0.x + qs[c + 1] * k0.y + qs[c + 2] * k0.z + qs[c + 3] * k0.w + qs[c + 4] * k1.x +
            qs[c + 5] * k1.y + qs[c + 6] * k1.z + qs[c + 7] * k1.w;
      sc += qs[c + 8] * k2.x + qs[c + 9] * k2.y + qs[c + 10] * k2.z + qs[c + 11] * k2.w + qs[c + 12] * k3.x +
            qs[c + 13] * k3.y + qs[c + 14] * k3.z + qs[c + 15] * k3.w;
    }
    const float sv = valid ? sc * (ks * scale) : -INFINITY;
    const float m2 = fmaxf(m, warp_fmax(sv));
    const float corr = __expf(m - m2);
    const float p = __expf(sv - m2);
    l = l * corr + warp_add(p);
#pragma unroll
    for (int d = 0; d < 4; ++d) acc[d] *= corr;
    m = m2;
    const float pv = p * vs;
    const int64_t vrow = (block - static_cast<const uint8_t*>(kv)) + (16 + tok) * kHeliumHeadDim;
    const int count = min(32, len - base);
    for (int j = 0; j < count; ++j) {
      const int64_t vj = __shfl_sync(0xffffffffu, vrow, j);
      const float pvj = __shfl_sync(0xffffffffu, pv, j);
      const float4 vf = e4m3x4(*reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(kv) + vj + lane * 4));
      acc[0] += pvj * vf.x, acc[1] += pvj * vf.y, acc[2] += pvj * vf.z, acc[3] += pvj * vf.w;
    }
  }
  if (lane == 0) {
    ms[warp] = m;
    ls[warp] = l;
  }
#pragma unroll
  for (int d = 0; d < 4; ++d) os[warp][lane * 4 + d] = acc[d];
  __syncthreads();
  const int d = threadIdx.x;
  float top = -INFINITY;
#pragma unroll
  for (int w = 0; w < kAttendWarps; ++w) top = fmaxf(top, ms[w]);
  float num = 0.f, den = 0.f;
#pragma unroll
  for (int w = 0; w < kAttendWarps; ++w) {
    const float e = ms[w] == -INFINITY ? 0.f : __expf(ms[w] - top);
    num += os[w][d] * e;
    den += ls[w] * e;
  }
  out[((int64_t)n * heads + h) * kHeliumHeadDim + d] = __float2bfloat16(num / den);
}

// `lm_dep_embed_norm` (lm.cu:301-313)
__global__ void lm_dep_embed_norm_kernel(const bf16* __restrict__ projected, int k, const bf16* __restrict__ table,
                                         int table_rows, const int32_t* __restrict__ drawn,
                                         const bf16* __restrict__ alpha, bf16* __restrict__ x, bf16* __restrict__ xn,
                                         int dim, float eps, uint32_t* err) {
  __shared__ float scratch[32];
  const int s = blockIdx.x, c = threadIdx.x * 8;
  int64_t id = drawn[s * kDuplexDrawn + k];
  if (id < 0 || id >= table_rows) {
    if (threadIdx.x == 0) raise(err, kErrBadIndex);
    id = 0;
  }
  float v[8], e[8];
  ld8(projected + ((int64_t)s * kDepSteps + k) * dim + c, v);
  ld8(table + id * dim + c, e);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = bf16_round(v[j] + e[j]);
  st8(x + (int64_t)s * dim + c, v);
  norm_row(v, alpha, xn + (int64_t)s * dim, dim, eps, scratch);
}

// `lm_dep_kv_attend` (lm.cu:319-366): a warp per (session, head), a lane owns two of the 64 dims; the step's own K
// and V stay in registers.
__global__ void lm_dep_kv_attend_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ ws, int step,
                                        bf16* __restrict__ out, int heads, float scale) {
  const int s = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= heads) return;
  const int width = heads * kDepHeadDim;
  const bf16* row = qkv + (int64_t)s * 3 * width;
  const int at = h * kDepHeadDim + lane * 2;
  const __nv_bfloat162 q2 = *reinterpret_cast<const __nv_bfloat162*>(row + at);
  const __nv_bfloat162 k2 = *reinterpret_cast<const __nv_bfloat162*>(row + width + at);
  const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(row + 2 * width + at);
  bf16* base = ws + (int64_t)s * kDepSteps * 2 * width;
  *reinterpret_cast<__nv_bfloat162*>(base + (int64_t)step * 2 * width + at) = k2;
  *reinterpret_cast<__nv_bfloat162*>(base + (int64_t)step * 2 * width + width + at) = v2;
  const float q0 = __bfloat162float(q2.x), q1 = __bfloat162float(q2.y);
  float m = -INFINITY, l = 0.f, a0 = 0.f, a1 = 0.f;
  for (int t = 0; t <= step; ++t) {
    __nv_bfloat162 kt = k2, vt = v2;
    if (t < step) {
      kt = *reinterpret_cast<const __nv_bfloat162*>(base + (int64_t)t * 2 * width + at);
      vt = *reinterpret_cast<const __nv_bfloat162*>(base + (int64_t)t * 2 * width + width + at);
    }
    const float sc = warp_add(q0 * __bfloat162float(kt.x) + q1 * __bfloat162float(kt.y)) * scale;
    const float m2 = fmaxf(m, sc);
    const float corr = __expf(m - m2);
    const float p = __expf(sc - m2);
    l = l * corr + p;
    a0 = a0 * corr + p * __bfloat162float(vt.x);
    a1 = a1 * corr + p * __bfloat162float(vt.y);
    m = m2;
  }
  const float inv_l = 1.f / l;
  *reinterpret_cast<__nv_bfloat162*>(out + (int64_t)s * width + at) = __floats2bfloat162_rn(a0 * inv_l, a1 * inv_l);
}

// ---- Gumbel-max draw over the top-k (lm.cu:368-537) ----------------------------------------------------------
// Every element's score depends only on (logit, seed, index): key = 16-bit order key of the bf16 logit, the k-th
// largest key found by a two-pass radix select (ties kept), score = logit / T - log(-log u) with
// u = ((mix(seed ^ mix(index)) >> 8) + 0.5) / 2^24, winner = largest (order_key(score), lowest index).

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ uint32_t order_key32(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t order_key16(bf16 v) {
  const uint16_t u = *reinterpret_cast<const uint16_t*>(&v);
  return (u & 0x8000u) ? (uint16_t)~u : (uint16_t)(u | 0x8000u);
}
__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

__global__ void __launch_bounds__(kSampleThreads)
    lm_sample_kernel(const bf16* __restrict__ logits, int vocab, int64_t ld, float temperature, int top_k,
                     const int32_t* __restrict__ force, const int32_t* __restrict__ seeds, int col,
                     int32_t* __restrict__ drawn) {
  const int s = blockIdx.x, tid = threadIdx.x;
  __shared__ uint32_t hist[256];
  __shared__ uint32_t sel_prefix, sel_left;
  __shared__ unsigned long long best;
  const int forced = force[s * kDuplexDrawn + col];
  if (forced >= 0) {
    if (tid == 0) drawn[s * kDuplexDrawn + col] = forced;
    return;
  }
  const bf16* l = logits + (int64_t)s * ld;
  const float inv_t = temperature > 0.f ? 1.f / temperature : 1.f;
  const int keep = top_k > 0 && top_k < vocab ? top_k : vocab;
  const uint32_t seed = mix32((uint32_t)seeds[2 * s] ^ mix32((uint32_t)seeds[2 * s + 1] + 0x9e3779b9u * (col + 1)));
  uint32_t prefix = 0;
  if (temperature > 0.f && keep < vocab) {
    uint32_t left = keep;
    for (int shift = 8; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      const uint32_t high = shift == 8 ? 0u : 0xff00u;
      for (int i = tid; i < vocab; i += kSampleThreads) {
        const uint32_t key = order_key16(l[i]);
        if (((key ^ prefix) & high) == 0) atomicAdd(&hist[(key >> shift) & 255], 1u);
      }
      __syncthreads();
      if (tid < 32) {  // lane t holds digits 8t..8t+7; keys in strictly higher digits via a suffix scan
        uint32_t c[8], mine = 0;
#pragma unroll
        for (int b = 0; b < 8; ++b) mine += c[b] = hist[tid * 8 + b];
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
            sel_prefix = prefix | (uint32_t)(tid * 8 + b) << shift;
            sel_left = left - above;
          }
          above += c[b];
        }
      }
      __syncthreads();
      prefix = sel_prefix;
      left = sel_left;
    }
  }
  if (tid == 0) best = 0ull;
  __syncthreads();
  unsigned long long mine = 0ull;
  for (int i = tid; i < vocab; i += kSampleThreads) {
    const bf16 val = l[i];
    if (order_key16(val) < prefix) continue;
    float score = __bfloat162float(val) * inv_t;
    if (temperature > 0.f) {
      const float u = ((mix32(seed ^ mix32((uint32_t)i)) >> 8) + 0.5f) * (1.f / 16777216.f);
      score -= __logf(-__logf(u));
    }
    const unsigned long long packed = (unsigned long long)order_key32(score) << 32 | (uint32_t)(0xffffffffu - i);
    mine = packed > mine ? packed : mine;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
    mine = other > mine ? other : mine;
  }
  if ((tid & 31) == 0) atomicMax(&best, mine);
  __syncthreads();
  if (tid == 0) drawn[s * kDuplexDrawn + col] = (int32_t)(0xffffffffu - (uint32_t)(best & 0xffffffffull));
}

// `lm_advance` (lm.cu:546-573): one thread per session.
__global__ void lm_advance_kernel(void* state, const int32_t* __restrict__ lines, int64_t stride,
                                  const int32_t* __restrict__ drawn, const int32_t* __restrict__ caller,
                                  const int32_t* __restrict__ force_caller, int32_t* __restrict__ emitted, int seqs) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= seqs) return;
  int32_t* row = const_cast<int32_t*>(state_row(state, lines, s, stride));
  int32_t* pending = row + kDuplexStreams;
  const int32_t* d = drawn + s * kDuplexDrawn;
  int32_t heard[kDuplexBooks];
#pragma unroll
  for (int k = 0; k < kDuplexBooks; ++k) {
    const int f = force_caller[s * kDuplexBooks + k];
    heard[k] = f >= 0 ? f : caller[s * kDuplexBooks + k];
  }
  emitted[s * kDuplexDrawn] = row[0];
  emitted[s * kDuplexDrawn + 1] = row[1];
#pragma unroll
  for (int k = 1; k < kDuplexBooks; ++k) emitted[s * kDuplexDrawn + 1 + k] = d[1 + k];
#pragma unroll
  for (int k = 0; k < kDuplexDrawn; ++k) row[k] = d[k];
  row[kDuplexDrawn] = heard[0];
#pragma unroll
  for (int k = 0; k < kDuplexBooks - 1; ++k) {
    row[kDuplexDrawn + 1 + k] = pending[k];
    pending[k] = heard[1 + k];
  }
}

// `lm_init` (lm.cu:576-581)
__global__ void lm_init_kernel(void* state, const int32_t* __restrict__ lines, int64_t stride,
                               const int32_t* __restrict__ init) {
  const int s = blockIdx.x;
  int32_t* own = const_cast<int32_t*>(state_row(state, lines, s, stride));
  if (threadIdx.x < kDuplexStateWords) own[threadIdx.x] = init[s * kDuplexStateWords + threadIdx.x];
}

// `lm_copy_kv` (lm.cu:584-593) for this library's layout: a warp per (token, head) moves the 128-byte key row, the
// 128-byte value row and the two scales.
__global__ void lm_copy_kv_kernel(void* kv, const int32_t* __restrict__ src_slot, const int32_t* __restrict__ dst_slot,
                                  int heads, int kv_pages, uint32_t* err) {
  const int r = blockIdx.x, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= heads) return;
  int64_t src = src_slot[r], dst = dst_slot[r];
  if (src < 0 || dst < 0 || (src >> 4) >= kv_pages || (dst >> 4) >= kv_pages) {
    if (lane == 0) raise(err, kErrBadIndex);
    return;
  }
  const uint8_t* from = page_head(kv, src >> 4, heads, h);
  uint8_t* to = page_head(kv, dst >> 4, heads, h);
  const int st = (int)(src & 15), dt = (int)(dst & 15);
  reinterpret_cast<uint32_t*>(to + dt * kHeliumHeadDim)[lane] = reinterpret_cast<const uint32_t*>(from + st * kHeliumHeadDim)[lane];
  reinterpret_cast<uint32_t*>(to + (16 + dt) * kHeliumHeadDim)[lane] =
      reinterpret_cast<const uint32_t*>(from + (16 + st) * kHeliumHeadDim)[lane];
  if (lane < 2)
    reinterpret_cast<float*>(to + 2 * 16 * kHeliumHeadDim + 64 * lane)[dt] =
        reinterpret_cast<const float*>(from + 2 * 16 * kHeliumHeadDim + 64 * lane)[st];
}

bool row_dim_ok(int dim) { return dim % 8 == 0 && dim / 8 <= 1024 && dim / 8 >= 32; }

}  // namespace

cudaError_t launch_lm_embed_ids(const int32_t* ids, const int32_t* voice, const bf16* voices, int voice_rows,
                                DuplexTables t, bf16* out, int rows, int dim, uint32_t* err, cudaStream_t s) {
  if (!row_dim_ok(dim)) return cudaErrorInvalidValue;
  lm_embed_ids_kernel<<<rows, dim / 8, 0, s>>>(ids, voice, voices, voice_rows, t, out, dim, err);
  return cudaGetLastError();
}

cudaError_t launch_lm_embed_state(const void* state, const int32_t* lines, int64_t stride, DuplexTables t, bf16* out,
                                  int32_t* rows_out, int rows, int dim, uint32_t* err, cudaStream_t s) {
  if (!row_dim_ok(dim)) return cudaErrorInvalidValue;
  lm_embed_state_kernel<<<rows, dim / 8, 0, s>>>(state, lines, stride, t, out, rows_out, dim, err);
  return cudaGetLastError();
}

cudaError_t launch_lm_norm(const bf16* x, const bf16* alpha, bf16* out, int rows, int dim, float eps, cudaStream_t s) {
  if (!row_dim_ok(dim)) return cudaErrorInvalidValue;
  lm_norm_kernel<<<rows, dim / 8, 0, s>>>(x, alpha, out, dim, eps);
  return cudaGetLastError();
}

cudaError_t launch_lm_add_norm(const bf16* y, bf16* x, const bf16* alpha, bf16* out, int rows, int dim, float eps,
                               cudaStream_t s) {
  if (!row_dim_ok(dim)) return cudaErrorInvalidValue;
  lm_add_norm_kernel<<<rows, dim / 8, 0, s>>>(y, x, alpha, out, dim, eps);
  return cudaGetLastError();
}

cudaError_t launch_lm_rope_kv(bf16* qkv, const int32_t* pos, const int32_t* slots, void* kv, int rows, int heads,
                              float coef, int kv_pages, uint32_t* err, cudaStream_t s) {
  lm_rope_kv_kernel<<<dim3(rows, (3 * heads + 7) / 8), 256, 0, s>>>(qkv, pos, slots, kv, heads, coef, kv_pages, err);
  return cudaGetLastError();
}

cudaError_t launch_lm_attend(const bf16* qkv, const void* kv, const int32_t* pos, const int32_t* seq,
                             const int32_t* indptr, const int32_t* pages, bf16* out, int rows, int heads, float scale,
                             int context, int kv_pages, uint32_t* err, cudaStream_t s) {
  lm_attend_kernel<<<dim3(rows, heads), kAttendWarps * 32, 0, s>>>(qkv, kv, pos, seq, indptr, pages, out, heads, scale,
                                                                  context, kv_pages, err);
  return cudaGetLastError();
}

cudaError_t launch_lm_dep_embed_norm(const bf16* projected, int k, const bf16* table, int table_rows,
                                     const int32_t* drawn, const bf16* alpha, bf16* x, bf16* xn, int rows, int dim,
                                     float eps, uint32_t* err, cudaStream_t s) {
  if (!row_dim_ok(dim)) return cudaErrorInvalidValue;
  lm_dep_embed_norm_kernel<<<rows, dim / 8, 0, s>>>(projected, k, table, table_rows, drawn, alpha, x, xn, dim, eps, err);
  return cudaGetLastError();
}

cudaError_t launch_lm_dep_kv_attend(const bf16* qkv, bf16* ws, int step, bf16* out, int rows, int heads, float scale,
                                    cudaStream_t s) {
  if (step < 0 || step >= kDepSteps) return cudaErrorInvalidValue;
  lm_dep_kv_attend_kernel<<<dim3(rows, (heads + 3) / 4), 128, 0, s>>>(qkv, ws, step, out, heads, scale);
  return cudaGetLastError();
}

cudaError_t launch_lm_sample(const bf16* logits, int vocab, int64_t ld, float temperature, int top_k,
                             const int32_t* force, const int32_t* seeds, int col, int32_t* drawn, int rows,
                             cudaStream_t s) {
  if (vocab < 1 || col < 0 || col >= kDuplexDrawn) return cudaErrorInvalidValue;
  lm_sample_kernel<<<rows, kSampleThreads, 0, s>>>(logits, vocab, ld, temperature, top_k, force, seeds, col, drawn);
  return cudaGetLastError();
}

cudaError_t launch_lm_advance(void* state, const int32_t* lines, int64_t stride, const int32_t* drawn,
                              const int32_t* caller, const int32_t* force_caller, int32_t* emitted, int rows,
                              cudaStream_t s) {
  lm_advance_kernel<<<(rows + 127) / 128, 128, 0, s>>>(state, lines, stride, drawn, caller, force_caller, emitted, rows);
  return cudaGetLastError();
}

cudaError_t launch_lm_copy_kv(void* kv, const int32_t* src_slot, const int32_t* dst_slot, int tokens, int heads,
                              int kv_pages, uint32_t* err, cudaStream_t s) {
  if (tokens < 1) return cudaSuccess;
  lm_copy_kv_kernel<<<dim3(tokens, (heads + 3) / 4), 128, 0, s>>>(kv, src_slot, dst_slot, heads, kv_pages, err);
  return cudaGetLastError();
}

cudaError_t launch_lm_init(void* state, const int32_t* lines, int64_t stride, const int32_t* init, int rows,
                           cudaStream_t s) {
  lm_init_kernel<<<rows, 32, 0, s>>>(state, lines, stride, init);
  return cudaGetLastError();
}

}  // namespace omni
