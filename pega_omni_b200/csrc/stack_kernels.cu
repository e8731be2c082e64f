// Decoder-stack kernels that are not GEMMs: RMSNorm with the residual stream,
// SwiGLU, per-head q/k norm + rotary embedding + KV write, and decode attention
// over the paged KV. Rounding points follow the reference's kernels
// (crates/omni-qwen3/kernels/qwen3.cu, crates/omni-kern/kernels/common.cuh):
// every tensor that crosses HBM is bf16, arithmetic is f32.
#include "attend.cuh"
#include "kernels.h"
#include "sampler.cuh"

namespace omni {

// ---- RMSNorm + residual ------------------------------------------------------

// One block of dim/8 threads per row. Semantics of `qwen3_norm_copy`
// (qwen3.cu:18-31).
__global__ void norm_copy_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ out,
                                 bf16* __restrict__ res, int dim, float eps) {
  __shared__ float scratch[32];
  const int64_t at = (int64_t)blockIdx.x * dim + threadIdx.x * 8;
  float v[8], g[8];
  ld8(x + at, v);
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) ss += v[k] * v[k];
  const float r = rsqrtf(block_add(ss, scratch) / dim + eps);
  st8(res + at, v);
  ld8(w + threadIdx.x * 8, g);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = v[k] * r * g[k];
  st8(out + at, v);
}

// Semantics of `qwen3_add_norm` (qwen3.cu:37-57): the residual is stored
// rounded, the norm is taken over the unrounded sum.
__global__ void add_norm_kernel(const bf16* __restrict__ x, bf16* __restrict__ res, const bf16* __restrict__ w,
                                bf16* __restrict__ out, int dim, float eps, int every, int which) {
  __shared__ float scratch[32];
  const int n = blockIdx.x;
  const int64_t at = (int64_t)n * dim + threadIdx.x * 8;
  float v[8], rv[8], g[8];
  ld8(x + at, v);
  ld8(res + at, rv);
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    v[k] += rv[k];
    ss += v[k] * v[k];
  }
  const float r = rsqrtf(block_add(ss, scratch) / dim + eps);
  st8(res + at, v);
  if (n % every != which) return;
  ld8(w + threadIdx.x * 8, g);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = v[k] * r * g[k];
  st8(out + (int64_t)(n / every) * dim + threadIdx.x * 8, v);
}

// `silu_mul` (common.cuh:66-76). With `interleaved` = g > 0, the fused row alternates g gate channels and the matching
// g up channels (the weight layout the tensor-core SwiGLU epilogue wants) instead of [all gate | all up].
__global__ void silu_mul_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ act, int inter, int total,
                                int interleaved) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int64_t n = i / (inter / 8), c = i % (inter / 8) * 8;
  float g[8], u[8];
  const int64_t g_at = interleaved ? (c / interleaved) * 2 * interleaved + c % interleaved : c;
  const int64_t u_at = interleaved ? g_at + interleaved : inter + c;
  ld8(gate_up + n * 2 * inter + g_at, g);
  ld8(gate_up + n * 2 * inter + u_at, u);
#pragma unroll
  for (int k = 0; k < 8; ++k) g[k] = bf16_round(g[k] / (1.f + __expf(-g[k]))) * u[k];
  st8(act + (int64_t)i * 8, g);
}

cudaError_t launch_norm_copy(const bf16* x, const bf16* w, bf16* out, bf16* res, int rows, int dim, float eps,
                             cudaStream_t s) {
  if (dim % 8 || dim / 8 > 1024) return cudaErrorInvalidValue;
  norm_copy_kernel<<<rows, dim / 8, 0, s>>>(x, w, out, res, dim, eps);
  return cudaGetLastError();
}

cudaError_t launch_add_norm(const bf16* x, bf16* res, const bf16* w, bf16* out, int rows, int dim, float eps,
                            int every, int which, cudaStream_t s) {
  if (dim % 8 || dim / 8 > 1024) return cudaErrorInvalidValue;
  add_norm_kernel<<<rows, dim / 8, 0, s>>>(x, res, w, out, dim, eps, every, which);
  return cudaGetLastError();
}

cudaError_t launch_silu_mul(const bf16* gate_up, bf16* act, int rows, int inter, int interleaved, cudaStream_t s) {
  const int total = rows * (inter / 8);
  if (interleaved && (inter % interleaved || interleaved % 8)) return cudaErrorInvalidValue;
  silu_mul_kernel<<<(total + 255) / 256, 256, 0, s>>>(gate_up, act, inter, total, interleaved);
  return cudaGetLastError();
}

// ---- row -> (sequence, position, page) -----------------------------------------

struct RowAt {
  int seq, pos;
  int64_t slot;            // page * 16 + pos % 16 of the row's own token
  const int32_t* pages;    // the sequence's page list, or nullptr when dense
};

__device__ __forceinline__ RowAt locate(const RowMap& m, int n) {
  RowAt r;
  if (m.pages) {
    r.seq = m.seq ? m.seq[n] : n;
    r.pos = m.pos[n];
    r.slot = m.slot ? m.slot[n] : 0;
    r.pages = m.pages + m.indptr[r.seq];
  } else {
    r.seq = n / m.per;
    r.pos = m.base + n % m.per;
    r.slot = (int64_t)r.seq * 16 + r.pos;
    r.pages = nullptr;
  }
  return r;
}

// ---- q/k norm + RoPE + KV write -------------------------------------------------

// One warp per (row, head) over the q, k and v heads of the fused qkv row.
// Semantics of `rope_kv` (qwen3.cu:66-107): RMSNorm over the head, the
// normalised value rounded to bf16 before the gain, half-rotation rotary
// embedding with inv_freq = theta^(-2i/D); q stays in place, k and v go to the
// row's slot.
template <int D>
__global__ void __launch_bounds__(256) rope_kv_kernel(bf16* __restrict__ qkv, const bf16* __restrict__ q_norm,
                                                      const bf16* __restrict__ k_norm, bf16* __restrict__ kv,
                                                      RowMap map, int hq, int hk, float eps, float theta,
                                                      int kv_pages, uint32_t* err) {
  constexpr int E = D / 64;  // elements of each half a lane owns
  const int n = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (head >= hq + 2 * hk) return;
  const RowAt at = locate(map, n);
  const int64_t page = at.slot >> 4;
  const int tok = (int)(at.slot & 15);
  if (page < 0 || page >= kv_pages) {
    if (lane == 0) raise(err, kErrBadIndex);
    return;
  }
  bf16* row = qkv + ((int64_t)n * (hq + 2 * hk) + head) * D;
  if (head >= hq + hk) {  // V: a plain copy
    bf16* dst = kv + kv_offset<D>(page, hk, head - hq - hk, 1, tok);
    for (int i = lane; i < D; i += 32) dst[i] = row[i];
    return;
  }
  const bool is_q = head < hq;
  const bf16* w = is_q ? q_norm : k_norm;
  bf16* dst = is_q ? row : kv + kv_offset<D>(page, hk, head - hq, 0, tok);
  float lo[E], hi[E], ss = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) {
    lo[e] = __bfloat162float(row[lane * E + e]);
    hi[e] = __bfloat162float(row[D / 2 + lane * E + e]);
    ss += lo[e] * lo[e] + hi[e] * hi[e];
  }
  const float r = rsqrtf(warp_add(ss) / D + eps);
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const int i = lane * E + e;
    const float a = bf16_round(lo[e] * r) * __bfloat162float(w[i]);
    const float b = bf16_round(hi[e] * r) * __bfloat162float(w[D / 2 + i]);
    const float inv_freq = 1.f / powf(theta, (float)(2 * i) / D);
    float sn, cs;
    sincosf((float)at.pos * inv_freq, &sn, &cs);
    dst[i] = __float2bfloat16(a * cs - b * sn);
    dst[D / 2 + i] = __float2bfloat16(b * cs + a * sn);
  }
}

cudaError_t launch_rope_kv(bf16* qkv, const bf16* q_norm, const bf16* k_norm, bf16* kv, const RowMap& map, int rows,
                           const AttnShape& a, int kv_pages, uint32_t* err, cudaStream_t s) {
  const int heads = a.q_heads + 2 * a.kv_heads;
  const dim3 grid(rows, (heads + 7) / 8);
  if (a.head_dim == 128)
    rope_kv_kernel<128><<<grid, 256, 0, s>>>(qkv, q_norm, k_norm, kv, map, a.q_heads, a.kv_heads, a.rms_eps,
                                             a.rope_theta, kv_pages, err);
  else if (a.head_dim == 64)
    rope_kv_kernel<64><<<grid, 256, 0, s>>>(qkv, q_norm, k_norm, kv, map, a.q_heads, a.kv_heads, a.rms_eps,
                                            a.rope_theta, kv_pages, err);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// ---- decode attention -------------------------------------------------------------
// The page loop lives in attend.cuh; here one CTA of four warps handles one (row, kv head). Every warp owns
// kAttnSlots staging slots in dynamic shared memory: its K|V blocks arrive through bulk copies, kAttnSlots of them
// ahead of the block it is working on.

constexpr int kAttnSlots = 1;

template <int D, int G>
__global__ void __launch_bounds__(kAttnWarps * 32) attend_kernel(const bf16* __restrict__ qkv,
                                                                 const bf16* __restrict__ kv, bf16* __restrict__ out,
                                                                 RowMap map, int hq, int hk, float scale, uint32_t* err) {
  extern __shared__ __align__(128) unsigned char attend_slots[];
  __shared__ AttnShared<D, G> sh;
  __shared__ __align__(8) uint64_t bars[kAttnWarps * kAttnSlots];
  const int n = blockIdx.x, kh = blockIdx.y;
  const RowAt at = locate(map, n);
  const bf16* q = qkv + ((int64_t)n * (hq + 2 * hk) + kh * G) * D;
  if (threadIdx.x < kAttnWarps * kAttnSlots) sm100::mbar_init(sm100::smem_addr(&bars[threadIdx.x]), 1);
  if (threadIdx.x == 0) sm100::mbar_init_fence();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) sh.qs[i / D][i % D] = __bfloat162float(q[i]);
  __syncthreads();
  const int warp = threadIdx.x >> 5;
  PageStage<kAttnSlots> stage{attend_slots + (size_t)warp * kAttnSlots * kv_block_bytes<D>(), bars + warp * kAttnSlots, 0u, err};
  attend_pages<D, G, kAttnWarps>(sh, kv, at.pages, at.seq, at.pos + 1, hk, kh, scale, out + ((int64_t)n * hq + kh * G) * D,
                                 threadIdx.x, sampler::CtaSync(), &stage);
}

template <int D, int G>
static cudaError_t launch_attend_dg(const bf16* qkv, const bf16* kv, bf16* out, const RowMap& map, int rows, int hq, int hk,
                                    uint32_t* err, cudaStream_t s) {
  constexpr size_t smem = (size_t)kAttnWarps * kAttnSlots * kv_block_bytes<D>();
  if (smem + sizeof(AttnShared<D, G>) > 40 * 1024) {  // per device and instantiation: above the default limit of dynamic shared memory
    static bool raised[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (!raised[device]) {
      const cudaError_t e = cudaFuncSetAttribute(attend_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      raised[device] = true;
    }
  }
  attend_kernel<D, G><<<dim3(rows, hk), kAttnWarps * 32, smem, s>>>(qkv, kv, out, map, hq, hk, 1.f / sqrtf((float)D), err);
  return cudaGetLastError();
}

template <int D>
static cudaError_t launch_attend_d(const bf16* qkv, const bf16* kv, bf16* out, const RowMap& map, int rows,
                                   const AttnShape& a, uint32_t* err, cudaStream_t s) {
  const int hq = a.q_heads, hk = a.kv_heads;
  switch (hq / hk) {
    case 1: return launch_attend_dg<D, 1>(qkv, kv, out, map, rows, hq, hk, err, s);
    case 2: return launch_attend_dg<D, 2>(qkv, kv, out, map, rows, hq, hk, err, s);
    case 4: return launch_attend_dg<D, 4>(qkv, kv, out, map, rows, hq, hk, err, s);
    case 5: return launch_attend_dg<D, 5>(qkv, kv, out, map, rows, hq, hk, err, s);
    case 8: return launch_attend_dg<D, 8>(qkv, kv, out, map, rows, hq, hk, err, s);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_attend(const bf16* qkv, const bf16* kv, bf16* out, const RowMap& map, int rows, const AttnShape& a,
                          uint32_t* err, cudaStream_t s) {
  if (a.q_heads % a.kv_heads) return cudaErrorInvalidValue;
  if (a.head_dim == 128) return launch_attend_d<128>(qkv, kv, out, map, rows, a, err, s);
  if (a.head_dim == 64) return launch_attend_d<64>(qkv, kv, out, map, rows, a, err, s);
  return cudaErrorInvalidValue;
}

}  // namespace omni
