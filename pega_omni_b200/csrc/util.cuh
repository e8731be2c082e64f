// Device helpers shared by every kernel of the library: bf16 packing, warp and
// block reductions, the device error word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace omni {

typedef __nv_bfloat16 bf16;

// Device error word: kernels OR a code into it instead of trapping, the host
// reads it after the call. Kernels that wait on hardware barriers return early
// once it is non-zero so one failure cannot stall a whole graph.
enum DeviceError : uint32_t {
  kErrNone = 0,
  kErrBarrierTimeout = 1u << 0,  // a bounded mbarrier wait ran out
  kErrBadIndex = 1u << 1,        // an id / page / slot outside its table
  kErrBadShape = 1u << 2,
};

__device__ __forceinline__ void raise(uint32_t* err, uint32_t code) { atomicOr(err, code); }

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

struct alignas(16) Pack8 {
  __nv_bfloat162 h[4];
};

// Eight bf16 (one 16-byte access) widened to f32.
__device__ __forceinline__ void unpack8(const Pack8& p, float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p.h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ Pack8 pack8(const float* v) {
  Pack8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return p;
}


// The same eight values moved as one 16-byte word: an access through uint4 is a single vector instruction wherever the
// struct copy above might be split into four.
__device__ __forceinline__ void unpack8v(const uint4& u, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint4 pack8v(const float* v) {
  uint4 u;
  __nv_bfloat162 t;
  t = __floats2bfloat162_rn(v[0], v[1]);
  u.x = *reinterpret_cast<const uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[2], v[3]);
  u.y = *reinterpret_cast<const uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[4], v[5]);
  u.z = *reinterpret_cast<const uint32_t*>(&t);
  t = __floats2bfloat162_rn(v[6], v[7]);
  u.w = *reinterpret_cast<const uint32_t*>(&t);
  return u;
}

__device__ __forceinline__ void ld8v(const bf16* src, float* v) { unpack8v(*reinterpret_cast<const uint4*>(src), v); }
__device__ __forceinline__ void st8v(bf16* dst, const float* v) { *reinterpret_cast<uint4*>(dst) = pack8v(v); }
// Eight bf16 at a 16-byte aligned address.
__device__ __forceinline__ void ld8(const bf16* src, float* v) { ld8v(src, v); }
__device__ __forceinline__ void st8(bf16* dst, const float* v) { st8v(dst, v); }

__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_fmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; `scratch` is 32 floats of shared memory. Ends with a
// barrier so `scratch` can be reused at once.
__device__ __forceinline__ float block_add(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_add(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  v = lane < nwarps ? scratch[lane] : 0.f;
  v = warp_add(v);
  __syncthreads();
  return v;
}

__device__ __forceinline__ float block_fmax(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_fmax(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  v = lane < nwarps ? scratch[lane] : -INFINITY;
  v = warp_fmax(v);
  __syncthreads();
  return v;
}

}  // namespace omni
