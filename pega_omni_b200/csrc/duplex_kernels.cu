// Non-GEMM kernels of the duplex (PersonaPlex) token loop. Value semantics follow
// crates/omni-personaplex/kernels/lm.cu (line ranges at each kernel); ids, pages and slots outside their tables
// raise the device error word instead of reading out of bounds.
#include <cuda_fp8.h>

#include "duplex.h"

#include "sm100.cuh"

namespace omni {
namespace {


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
    *reinterpret_cast<uint4*>(out + r * dim + c) = *reinterpret_cast<const uint4*>(voices + (int64_t)v * dim + c);
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

// ---- tensor-parallel pair: all-reduce of a projection's partial rows, fused with the add + norm that follows -----
// Two ranks (two GPUs, one process each) hold half of the attention heads and half of the MLP channels; after the o
// and down projections each has a partial row block y_r [rows, dim]. This kernel makes y = bf16(y_0 + y_1) on both
// ranks and goes on as lm_add_norm does (x = bf16(x + y), out = norm(x)). The exchange is plain peer-memory traffic:
//   - `mine` sits in this rank's exchange buffer (written by the GEMM launched before this kernel), `peer` is the same
//     buffer of the other rank, mapped into this process;
//   - one thread stores this exchange's number into the PEER's flag word (release, system scope), so each rank polls
//     a word in its own memory; thread 0 of every CTA waits (acquire, system scope, at most kTpWaitNs) until its own
//     flag has reached the number, then the CTA reads the peer's rows with system-scope loads that bypass L1;
//   - exchanges are numbered by a device-resident counter that the last CTA to finish advances, so a captured graph
//     replays the same launch with new numbers; two buffers alternate (o, down), and a rank can only overwrite a
//     buffer two exchanges later, after it has seen the peer's next flag, which the peer raises only when its
//     previous exchange kernel (the reader of that buffer) has completed.
// f32 addition commutes, so both ranks round the same sum: their rows stay bit-identical.
// A wait that runs out raises the error word, takes the peer's rows as zero and lets the kernel finish.
constexpr uint64_t kTpWaitNs = 2000ull * 1000 * 1000;

__global__ void lm_tp_add_norm_kernel(const bf16* __restrict__ mine, const bf16* peer, bf16* __restrict__ x,
                                      const bf16* __restrict__ alpha, bf16* __restrict__ out, int dim, float eps,
                                      uint32_t* my_flag, uint32_t* peer_flag, uint32_t* counter, uint32_t* finished,
                                      uint32_t* err) {
  __shared__ float scratch[32];
  __shared__ int peer_ready;
  const uint32_t number = *reinterpret_cast<volatile uint32_t*>(counter) + 1u;
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag), "r"(number) : "memory");
    }
    int ok = 1;
    if (*reinterpret_cast<volatile uint32_t*>(err) != 0) {
      ok = 0;  // an earlier kernel gave up: do not wait for a peer that may have given up as well
    } else {
      const uint64_t start = sm100::global_timer_ns();
      for (uint32_t spins = 0;; ++spins) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(my_flag) : "memory");
        if ((int32_t)(seen - number) >= 0) break;
        if ((spins & 63u) == 63u && sm100::global_timer_ns() - start > kTpWaitNs) {
          raise(err, kErrBarrierTimeout);
          ok = 0;
          break;
        }
      }
    }
    peer_ready = ok;
  }
  __syncthreads();
  const int64_t at = (int64_t)blockIdx.x * dim + threadIdx.x * 8;
  float v[8], a[8], b[8];
  ld8(x + at, v);
  ld8(mine + at, a);
  if (peer_ready) {
    Pack8 raw;
    uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                 : "l"(peer + at)
                 : "memory");
    unpack8(raw, b);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) b[k] = 0.f;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = bf16_round(v[k] + bf16_round(a[k] + b[k]));
  st8(x + at, v);
  if (out) norm_row(v, alpha, out + (int64_t)blockIdx.x * dim, dim, eps, scratch);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(finished, 1u) == gridDim.x - 1) {  // every CTA has read the counter: advance it for the next launch
      *finished = 0;
      *reinterpret_cast<volatile uint32_t*>(counter) = number;
      __threadfence();
    }
  }
}

__device__ __forceinline__ uint8_t* page_head(void* kv, int64_t page, int heads, int h) {
  return static_cast<uint8_t*>(kv) + (page * heads + h) * (int64_t)kDuplexPageHeadBytes;
}

__device__ __forceinline__ float e4m3_scale(float amax) { return fmaxf(amax * (1.f / 448.f), 1e-12f); }

// Interleaved rotary embedding + FP8 KV write of one row (value semantics of `lm_rope`, lm.cu:129-184). kRopeParts
// CTAs per row: the 64 rotation angles depend on the row's position alone, so a CTA computes them once into shared
// memory (freq_i = expf(i * coef), sincosf(freq_i * pos)) for all the heads it rotates; its eight warps then walk
// its share of the 3 * heads heads, a lane owning four consecutive elements of the head (two rotation pairs): one
// 8-byte load, and for k / v one 4-byte FP8 store. k and v are quantised per head to E4M3 with the scale
// max(amax / 448, 1e-12), kept as f32 beside the page's values.
constexpr int kRopeWarps = 8, kRopeParts = 4;

__global__ void __launch_bounds__(kRopeWarps * 32)
    lm_rope_kv_kernel(bf16* __restrict__ qkv, const int32_t* __restrict__ pos, const int32_t* __restrict__ slots, void* kv,
                      int heads, float coef, int kv_pages, uint32_t* err) {
  __shared__ float cs[kHeliumHeadDim / 2], sn[kHeliumHeadDim / 2];
  const int n = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < kHeliumHeadDim / 2) {
    const float freq = expf((float)threadIdx.x * coef);
    sincosf(freq * (float)pos[n], &sn[threadIdx.x], &cs[threadIdx.x]);
  }
  int64_t slot = slots[n];
  if (slot < 0 || (slot >> 4) >= kv_pages) {
    if (threadIdx.x == 0) raise(err, kErrBadIndex);
    slot = 0;
  }
  const int tok = (int)(slot & 15);
  __syncthreads();
  for (int head = blockIdx.y * kRopeWarps + warp; head < 3 * heads; head += kRopeWarps * kRopeParts) {
    bf16* src = qkv + ((int64_t)n * 3 * heads + head) * kHeliumHeadDim + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const float2 p0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 p1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float v[4] = {p0.x, p0.y, p1.x, p1.y};
    if (head < 2 * heads) {  // q and k: pairs (2i, 2i + 1) rotated by angle i
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const float c = cs[2 * lane + k], sv = sn[2 * lane + k];
        const float r = v[2 * k], im = v[2 * k + 1];
        v[2 * k] = r * c - im * sv;
        v[2 * k + 1] = r * sv + im * c;
      }
    }
    if (head < heads) {  // q: rounded to bf16 in place
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v[0], v[1]);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v[2], v[3]);
      *reinterpret_cast<uint2*>(src) = o;
      continue;
    }
    const bool is_v = head >= 2 * heads;
    const int h = head - (is_v ? 2 : 1) * heads;
    const float amax = warp_fmax(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
    const float sc = e4m3_scale(amax), inv = 1.f / sc;
    uint8_t* block = page_head(kv, slot >> 4, heads, h);
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint32_t*>(block + ((is_v ? 16 : 0) + tok) * kHeliumHeadDim + lane * 4) = lo | hi << 16;
    if (lane == 0) reinterpret_cast<float*>(block + 2 * 16 * kHeliumHeadDim + (is_v ? 64 : 0))[tok] = sc;
  }
}

__device__ __forceinline__ float4 e4m3x4(uint32_t raw) {
  return static_cast<float4>(*reinterpret_cast<const __nv_fp8x4_e4m3*>(&raw));
}

// Decode attention over the FP8 ring (value semantics of `lm_attend` / `attend_row_fp8`, lm.cu:197-290: f32 scores,
// score * (k_scale * scale), __expf, p * v_scale, bf16 out). One CTA per (row, head), four warps. A (page, head) block
// is 4,224 contiguous bytes (16 keys, 16 values, their scales), so a warp stages whole pages into its own two
// shared-memory slots with one bulk copy each (cp.async.bulk, completion on an mbarrier) and has the next page under
// way while it works on the current one. Inside a page a lane scores half a key (64 of the 128 FP8 dims; lanes t and
// t + 16 share key t), the online softmax advances one page (16 keys) at a time, then every lane adds its four output
// dims of the 16 values. The warps' states are merged at the end. Waits are bounded (the error word, then out).
constexpr int kAttendWarps = 4;
constexpr int kAttendSlotBytes = ((kDuplexPageHeadBytes + 127) / 128) * 128;

struct AttendShared {
  float q[kHeliumHeadDim];
  float ms[kAttendWarps], ls[kAttendWarps];
  float os[kAttendWarps][kHeliumHeadDim];
  uint64_t bar[kAttendWarps][2];
};

__global__ void __launch_bounds__(kAttendWarps * 32)
    lm_attend_kernel(const bf16* __restrict__ qkv, const void* kv, const int32_t* __restrict__ pos,
                     const int32_t* __restrict__ seq, const int32_t* __restrict__ indptr,
                     const int32_t* __restrict__ pages, bf16* __restrict__ out, int heads, float scale, int context,
                     int kv_pages, uint32_t* err) {
  extern __shared__ __align__(128) unsigned char attend_smem[];
  AttendShared& sh = *reinterpret_cast<AttendShared*>(attend_smem);
  unsigned char* slots = attend_smem + ((sizeof(AttendShared) + 127) & ~(size_t)127);
  const int n = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int s = seq ? seq[n] : n;
  const int len = min(pos[n] + 1, context), npages = (len + 15) >> 4;
  const int32_t* my_pages = pages + indptr[s];
  if (threadIdx.x < kHeliumHeadDim)
    sh.q[threadIdx.x] = __bfloat162float(qkv[((int64_t)n * 3 * heads + h) * kHeliumHeadDim + threadIdx.x]);
  if (lane == 0) {
    sm100::mbar_init(sm100::smem_addr(&sh.bar[warp][0]), 1);
    sm100::mbar_init(sm100::smem_addr(&sh.bar[warp][1]), 1);
  }
  sm100::mbar_init_fence();
  __syncthreads();

  unsigned char* mine = slots + (size_t)warp * 2 * kAttendSlotBytes;
  auto fetch = [&](int pi, int slot) {  // lane 0: one bulk copy of page pi's block for this head
    int64_t page = my_pages[pi];
    if (page < 0 || page >= kv_pages) {
      raise(err, kErrBadIndex);
      page = 0;
    }
    const uint32_t bar = sm100::smem_addr(&sh.bar[warp][slot]);
    sm100::mbar_expect_tx(bar, kDuplexPageHeadBytes);
    sm100::bulk_load(sm100::smem_addr(mine + (size_t)slot * kAttendSlotBytes),
                     page_head(const_cast<void*>(kv), page, heads, h), kDuplexPageHeadBytes, bar);
  };
  float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  const int tok = lane & 15, half = lane >> 4;
  if (warp < npages && lane == 0) fetch(warp, 0);
  uint32_t parity[2] = {0, 0};
  int slot = 0;
  for (int pi = warp; pi < npages; pi += kAttendWarps, slot ^= 1) {
    if (pi + kAttendWarps < npages && lane == 0) fetch(pi + kAttendWarps, slot ^ 1);  // (that slot was read a round ago)
    if (!sm100::mbar_wait(sm100::smem_addr(&sh.bar[warp][slot]), parity[slot], err)) break;
    parity[slot] ^= 1u;
    const unsigned char* blk = mine + (size_t)slot * kAttendSlotBytes;
    const int ntok = min(16, len - pi * 16);
    float dot = 0.f;
    {
      const uint4* krow = reinterpret_cast<const uint4*>(blk + tok * kHeliumHeadDim + half * 64);
      const float* qh = sh.q + half * 64;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 raw = krow[c];
        const float4 k0 = e4m3x4(raw.x), k1 = e4m3x4(raw.y), k2 = e4m3x4(raw.z), k3 = e4m3x4(raw.w);
        const float* qc = qh + c * 16;
        dot += qc[0] * k0.x + qc[1] * k0.y + qc[2] * k0.z + qc[3] * k0.w + qc[4] * k1.x + qc[5] * k1.y + qc[6] * k1.z +
               qc[7] * k1.w;
        dot += qc[8] * k2.x + qc[9] * k2.y + qc[10] * k2.z + qc[11] * k2.w + qc[12] * k3.x + qc[13] * k3.y +
               qc[14] * k3.z + qc[15] * k3.w;
      }
    }
    dot += __shfl_xor_sync(0xffffffffu, dot, 16);  // both halves of key `tok`
    const float ks = reinterpret_cast<const float*>(blk + 2 * 16 * kHeliumHeadDim)[tok];
    const float vs = reinterpret_cast<const float*>(blk + 2 * 16 * kHeliumHeadDim + 64)[tok];
    const float sv = tok < ntok ? dot * (ks * scale) : -INFINITY;
    const float m2 = fmaxf(m, warp_fmax(sv));
    const float corr = __expf(m - m2);
    const float p = __expf(sv - m2);
    float psum = p;  // over the 16 keys (both half-warps hold the same values)
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l = l * corr + psum;
#pragma unroll
    for (int d = 0; d < 4; ++d) acc[d] *= corr;
    m = m2;
    const float pv = p * vs;  // 0 for keys past the row's length
    const uint32_t* vrows = reinterpret_cast<const uint32_t*>(blk + 16 * kHeliumHeadDim) + lane;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pv, j);
      const float4 vf = e4m3x4(vrows[j * (kHeliumHeadDim / 4)]);
      acc[0] += pj * vf.x, acc[1] += pj * vf.y, acc[2] += pj * vf.z, acc[3] += pj * vf.w;
    }
    __syncwarp();  // every lane is done with this slot before lane 0 refills it in the next round
  }
  if (lane == 0) {
    sh.ms[warp] = m;
    sh.ls[warp] = l;
  }
#pragma unroll
  for (int d = 0; d < 4; ++d) sh.os[warp][lane * 4 + d] = acc[d];
  __syncthreads();
  if (threadIdx.x < kHeliumHeadDim) {
    const int d = threadIdx.x;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttendWarps; ++w) top = fmaxf(top, sh.ms[w]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < kAttendWarps; ++w) {
      const float e = sh.ms[w] == -INFINITY ? 0.f : __expf(sh.ms[w] - top);
      num += sh.os[w][d] * e;
      den += sh.ls[w] * e;
    }
    out[((int64_t)n * heads + h) * kHeliumHeadDim + d] = __float2bfloat16(num / den);
  }
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

// ---- Gumbel-max draw over the top-k (value semantics of `lm_sample`, lm.cu:368-537) ----------------------------
// Every element's score depends only on (logit, seed, index): key = 16-bit order key of the bf16 logit, the cut is
// the k-th largest key (ties kept), score = logit / T - log(-log u) with u = ((mix(seed ^ mix(index)) >> 8) + 0.5) /
// 2^24, winner = largest (order_key(score), lowest index).
//
// One CTA of 1024 threads per row. The row is read from memory ONCE: every thread keeps its share of the keys in
// registers (two per register, up to 64 per thread = a vocabulary of 65,536). The cut is then found by bisection on
// the key's 16 bits, most significant first: a bit stays set when at least k keys are >= the candidate, which takes
// one count per round over registers, a shuffle sum per warp and one block barrier (the per-warp counts are
// double-buffered in shared memory, so a round needs no second barrier). The survivors' scores are computed from the
// same registers and the winner is reduced by shuffles and one pass over the 32 warp results.

constexpr int kSampleThreads = 1024;
constexpr int kSampleRegs = 32;  // packed key pairs per thread

__device__ __forceinline__ uint32_t order_key32(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t order_key16(uint32_t bits) {  // bits: a bf16 in the low half
  return (bits & 0x8000u) ? (~bits & 0xffffu) : (bits | 0x8000u);
}
__device__ __forceinline__ float logit_of(uint32_t key) {  // the inverse of order_key16
  const uint32_t bits = (key & 0x8000u) ? (key & 0x7fffu) : (~key & 0xffffu);
  return __uint_as_float(bits << 16);
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
  const int s = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __shared__ uint32_t counts[2][kSampleThreads / 32];
  __shared__ unsigned long long best[kSampleThreads / 32];
  const int forced = force[s * kDuplexDrawn + col];
  if (forced >= 0) {
    if (tid == 0) drawn[s * kDuplexDrawn + col] = forced;
    return;
  }
  // element 2 * (r * 1024 + tid) + {0, 1} lives in the low / high half of reg[r]; 0 past the vocabulary (the smallest
  // key there is: -NaN with every mantissa bit set orders lowest, and no count ever includes index >= vocab)
  const uint16_t* row = reinterpret_cast<const uint16_t*>(logits + (int64_t)s * ld);
  uint32_t reg[kSampleRegs];
#pragma unroll
  for (int r = 0; r < kSampleRegs; ++r) {
    const int i = 2 * (r * kSampleThreads + tid);
    const uint32_t k0 = i < vocab ? order_key16(row[i]) : 0u, k1 = i + 1 < vocab ? order_key16(row[i + 1]) : 0u;
    reg[r] = k0 | k1 << 16;
  }
  const float inv_t = temperature > 0.f ? 1.f / temperature : 1.f;
  const int keep = top_k > 0 && top_k < vocab ? top_k : vocab;
  uint32_t cut = 0;
  if (temperature > 0.f && keep < vocab) {
    for (int bit = 15; bit >= 0; --bit) {
      const uint32_t cand = cut | 1u << bit;  // cand >= 1: the padding keys (0) never count
      uint32_t c = 0;
#pragma unroll
      for (int r = 0; r < kSampleRegs; ++r) c += ((reg[r] & 0xffffu) >= cand) + ((reg[r] >> 16) >= cand);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
      if (lane == 0) counts[bit & 1][warp] = c;
      __syncthreads();
      uint32_t total = 0;
#pragma unroll
      for (int w = 0; w < kSampleThreads / 32; ++w) total += counts[bit & 1][w];
      if (total >= (uint32_t)keep) cut = cand;
    }
  }
  const uint32_t seed = mix32((uint32_t)seeds[2 * s] ^ mix32((uint32_t)seeds[2 * s + 1] + 0x9e3779b9u * (col + 1)));
  unsigned long long mine = 0ull;
#pragma unroll
  for (int r = 0; r < kSampleRegs; ++r) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = 2 * (r * kSampleThreads + tid) + e;
      const uint32_t key = e ? reg[r] >> 16 : reg[r] & 0xffffu;
      if (i >= vocab || key < cut) continue;
      float score = logit_of(key) * inv_t;
      if (temperature > 0.f) {
        const float u = ((mix32(seed ^ mix32((uint32_t)i)) >> 8) + 0.5f) * (1.f / 16777216.f);
        score -= __logf(-__logf(u));
      }
      const unsigned long long packed = (unsigned long long)order_key32(score) << 32 | (uint32_t)(0xffffffffu - i);
      mine = packed > mine ? packed : mine;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
    mine = other > mine ? other : mine;
  }
  if (lane == 0) best[warp] = mine;
  __syncthreads();
  if (warp == 0) {
    mine = best[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, o);
      mine = other > mine ? other : mine;
    }
    if (lane == 0) drawn[s * kDuplexDrawn + col] = (int32_t)(0xffffffffu - (uint32_t)(mine & 0xffffffffull));
  }
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

cudaError_t launch_lm_tp_add_norm(const bf16* mine, const bf16* peer, bf16* x, const bf16* alpha, bf16* out, int rows,
                                  int dim, float eps, const TpLink& link, uint32_t* err, cudaStream_t s) {
  if (!row_dim_ok(dim) || !peer || !link.my_flag || !link.peer_flag) return cudaErrorInvalidValue;
  lm_tp_add_norm_kernel<<<rows, dim / 8, 0, s>>>(mine, peer, x, alpha, out, dim, eps, link.my_flag, link.peer_flag,
                                                 link.counter, link.finished, err);
  return cudaGetLastError();
}

cudaError_t launch_lm_rope_kv(bf16* qkv, const int32_t* pos, const int32_t* slots, void* kv, int rows, int heads,
                              float coef, int kv_pages, uint32_t* err, cudaStream_t s) {
  lm_rope_kv_kernel<<<dim3(rows, kRopeParts), kRopeWarps * 32, 0, s>>>(qkv, pos, slots, kv, heads, coef, kv_pages, err);
  return cudaGetLastError();
}

cudaError_t launch_lm_attend(const bf16* qkv, const void* kv, const int32_t* pos, const int32_t* seq,
                             const int32_t* indptr, const int32_t* pages, bf16* out, int rows, int heads, float scale,
                             int context, int kv_pages, uint32_t* err, cudaStream_t s) {
  const size_t smem = ((sizeof(AttendShared) + 127) & ~(size_t)127) + (size_t)kAttendWarps * 2 * kAttendSlotBytes;
  static bool raised[64] = {};  // per device: 70 KB of staging slots is above the default 48 KB of dynamic shared memory
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return cudaErrorInvalidDevice;
  if (!raised[device]) {
    const cudaError_t e = cudaFuncSetAttribute(lm_attend_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    raised[device] = true;
  }
  lm_attend_kernel<<<dim3(rows, heads), kAttendWarps * 32, smem, s>>>(qkv, kv, pos, seq, indptr, pages, out, heads, scale,
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
  if (vocab > 2 * kSampleRegs * kSampleThreads) return cudaErrorInvalidValue;  // a thread keeps 64 keys in registers
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
