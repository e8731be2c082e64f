// The persistent tick kernel (see tick.h): 11 warps per CTA, one CTA per SM, cooperative launch.
//   warp 0 / lane 0   weight producer: TMA loads of W tiles, runs ahead of the grid barriers
//   warp 1 / lane 0   activation producer: TMA loads of X tiles, gated by the barrier before its phase
//   warp 2 / lane 0   issues tcgen05.mma into one of two TMEM accumulators; whole warp owns the TMEM allocation
//   warps 3..10       workers: GEMM epilogues (TMEM -> partial tiles / SwiGLU) and every non-GEMM phase
//
// GEMM orientation. A tcgen05.mma occupies the tensor pipe for a fixed ~140 cycles whatever its M and N
// (measured on B200), so each instruction must carry as many weight bytes as possible: the activation
// rows (sessions, at most 128) sit on the MMA M dimension and 256 weight rows on N, 16 of K per
// instruction. D[session, weight row] lands with one session per TMEM lane, so a worker thread owns
// one output row and its 256 columns are contiguous in memory.
//
// Every wait (mbarrier, grid barrier, phase release) is bounded; on a timeout the device error word is
// raised, every CTA sees it within its next wait and the kernel unwinds.
#include "tick.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>

#include "attend.cuh"
#include "gemm.h"
#include "rope.cuh"
#include "sampler.cuh"
#include "sm100.cuh"

namespace omni {
namespace {

constexpr int kThreads = 352;  // 3 control warps + 8 worker warps: 186 registers per thread
constexpr int kWorkerThreads = 256;
constexpr int kFirstWorkerWarp = 3;
constexpr int kMaxStages = 16;
constexpr int kTileN = 256;  // weight rows per tile (the MMA N dimension)
constexpr int kTileK = 64;   // K elements per stage: one 128-byte swizzle row
constexpr int kTileM = 128;  // the MMA M dimension: activation rows, zero/garbage padded
constexpr int kMaxRingBytes = 192 * 1024;  // most shared memory the tile ring may take
constexpr int kGroupThreads = 128;

struct GroupBar {  // named barrier of one 128-thread worker group
  int id;
  __device__ __forceinline__ void sync() const { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
};
struct PairBar {  // named barrier of a two-warp attention team
  int id;
  __device__ __forceinline__ void sync() const { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }
};
using WorkerSync = sampler::NamedSync<1, kWorkerThreads>;

struct alignas(16) Control {
  uint64_t full_w[kMaxStages], full_x[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  volatile int released;  // phases [0, released) are complete on every CTA
  volatile int abort;
  float red[2][4];
  Phase phase[2];  // the workers' current and next phase records
};

union WorkerScratch {
  AttnShared<128, 4, 2> attn2[4];  // one per two-warp team
  AttnShared<128, 4, 1> attn1[8];  // one per worker warp
  sampler::Shared sample;
};

struct KernelArgs {
  const Phase* phases;
  int n_phases;
  const CUtensorMap* maps;
  float* partials;
  uint32_t* barrier;
  uint32_t barrier_base;  // arrivals counted by earlier launches (the counter is not reset between launches)
  uint32_t* err;
  int ring_bytes;                      // shared memory of the tile ring (a multiple of 1 KB): the rest of the SM's
                                       // array stays L1, which the row-wise phases live on
  int w_ahead;                         // phases the weight producer may run ahead of the grid barriers
  unsigned long long* trace;           // optional: four global-timer stamps per (phase, CTA), see tick_launch
  TickIo io;
};

__device__ __forceinline__ int first_item(const Phase& ph) {
  const int g = gridDim.x;
  return (int)((blockIdx.x + g - ph.cta_offset % g) % g);
}

// The tile ring of a GEMM phase: stages of [kbs activation k-blocks: bn rows each][kbs weight k-blocks: tile_n rows
// each], each row 128 bytes, as many stages as fit (at most kMaxStages); one TMA copy fills each half of a stage. The three pipeline roles of a CTA walk the stages in the same order and
// restart at stage 0 whenever the geometry changes; a stage's mbarrier parities are tracked per stage (one bit each),
// so a barrier that one geometry never reaches stays consistent for the next.
struct Ring {
  uint32_t x_slice = 0, w_slice = 0, x_bytes = 0, stage_bytes = 0;
  int kbs = 1, n = 0, stage = 0;
  uint32_t par = 0;  // bit s: parity of stage s's next wait
  // Returns true when the geometry changed (the caller may have to drain the old one first).
  __device__ __forceinline__ bool enter(const Phase& ph, int ring_bytes) {
    const uint32_t xs = ((uint32_t)ph.bn * kTileK * 2 + 1023u) & ~1023u, ws = (uint32_t)ph.tile_n * kTileK * 2;
    const int k = ph.i1 > 0 ? ph.i1 : 1;
    if (xs == x_slice && ws == w_slice && k == kbs) return false;
    x_slice = xs, w_slice = ws, kbs = k;
    x_bytes = xs * (uint32_t)k, stage_bytes = (xs + ws) * (uint32_t)k;
    n = min(kMaxStages, (int)((uint32_t)ring_bytes / stage_bytes));
    stage = 0;
    return true;
  }
  // k-block j of the stage's activation / weight tile
  __device__ __forceinline__ uint32_t x_off(int j = 0) const { return (uint32_t)stage * stage_bytes + (uint32_t)j * x_slice; }
  __device__ __forceinline__ uint32_t w_off(int j = 0) const {
    return (uint32_t)stage * stage_bytes + x_bytes + (uint32_t)j * w_slice;
  }
  __device__ __forceinline__ uint32_t parity() const { return par >> stage & 1u; }
  __device__ __forceinline__ void advance() {
    par ^= 1u << stage;
    if (++stage == n) stage = 0;
  }
};

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All CTAs arrive, then wait until `target` arrivals have been counted. Returns false on timeout / error.
// Called by one thread after a team barrier: the release on the counter is cumulative over the team's writes
// ordered before it by that barrier, and the acquire that sees the last arrival orders every CTA's writes before
// whatever the team does after its next barrier; no separate fence is needed on either side.
__device__ bool grid_barrier(uint32_t* counter, uint32_t target, uint32_t* err) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
  const uint64_t start = sm100::global_timer_ns();
  for (uint32_t spins = 0;; ++spins) {
    if (ld_acquire(counter) >= target) return true;
    if ((spins & 127u) == 127u) {
      if (*reinterpret_cast<volatile uint32_t*>(err) != 0) return false;
      if (sm100::global_timer_ns() - start > sm100::kWaitLimitNs) {
        raise(err, kErrBarrierTimeout);
        return false;
      }
    }
  }
}

// Split-K partial tiles: [split][tile][row (bn)][tile_n columns] f32, tile_n = 64, 128 or 256. Sums are taken in
// split order starting from zero, so the result does not depend on which CTA computed which split.
struct Partials {
  const float* base;
  int splits, tiles, bn, shift;  // shift = log2(tile_n)
  size_t split_stride;
  __device__ __forceinline__ Partials(const float* p, const Phase& ph)
      : base(p), splits(ph.splits), tiles(ph.tiles), bn(ph.bn), shift(ph.tile_n == 256 ? 8 : ph.tile_n == 128 ? 7 : 6),
        split_stride((size_t)ph.tiles * ph.bn * ph.tile_n) {}
  __device__ __forceinline__ uint32_t at(int m, int n) const {  // element offset inside split 0
    return (uint32_t)((((size_t)(n >> shift) * bn + m) << shift) + (n & ((1 << shift) - 1)));
  }
};

// NV groups of VEC consecutive columns of one row at once (a group never straddles a tile: cols[j] is a multiple
// of VEC). The split loop is outermost and unrolled so the loads of several splits are independent and in flight
// together: one L2 round trip per batch instead of one per element.
template <int VEC>
struct VecOf;
template <>
struct VecOf<1> { using T = float; };
template <>
struct VecOf<2> { using T = float2; };
template <>
struct VecOf<4> { using T = float4; };

template <int NV, int VEC>
__device__ __forceinline__ void reduce_vecs(const Partials& pt, int m, const int (&cols)[NV], float (&acc)[NV * VEC]) {
  using V = typename VecOf<VEC>::T;
  uint32_t off[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) off[j] = pt.at(m, cols[j]);
#pragma unroll
  for (int i = 0; i < NV * VEC; ++i) acc[i] = 0.f;
  const float* base = pt.base;
  constexpr int kBatch = NV * VEC <= 4 ? 8 : NV * VEC <= 16 ? 4 : 2;  // splits whose loads are issued before any is consumed
  for (int s0 = 0; s0 < pt.splits; s0 += kBatch, base += kBatch * pt.split_stride) {
    V f[kBatch][NV];
#pragma unroll
    for (int b = 0; b < kBatch; ++b)
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (s0 + b < pt.splits)
          f[b][j] = __ldcg(reinterpret_cast<const V*>(base + b * pt.split_stride + off[j]));
        else
          f[b][j] = V{};  // adding 0 for a missing split leaves the sum unchanged
      }
#pragma unroll
    for (int b = 0; b < kBatch; ++b)
#pragma unroll
      for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[j * VEC + e] += reinterpret_cast<const float*>(&f[b][j])[e];
  }
}

template <int N>
__device__ __forceinline__ void reduce_cols(const Partials& pt, int m, const int (&cols)[N], float (&acc)[N]) {
  reduce_vecs<N, 1>(pt, m, cols, acc);
}

// The row-wise phases' access pattern: a 128-thread group owns a row; thread j owns, for t < NV, the VEC
// consecutive columns starting at (t * 128 + j) * VEC. VEC = 4 reads the partial tiles 16 bytes at a time.
template <int NV, int VEC>
__device__ __forceinline__ int row_col(int t, int gtid) { return (t * kGroupThreads + gtid) * VEC; }

template <int NV, int VEC>
__device__ __forceinline__ void reduce_row(const Partials& pt, int m, int gtid, float (&acc)[NV * VEC]) {
  uint32_t off[NV];
#pragma unroll
  for (int t = 0; t < NV; ++t) off[t] = pt.at(m, row_col<NV, VEC>(t, gtid));
#pragma unroll
  for (int i = 0; i < NV * VEC; ++i) acc[i] = 0.f;
  const float* base = pt.base;
  constexpr int kBatch = NV * VEC <= 8 ? 8 : 4;  // splits whose loads are issued before any is consumed
  for (int s0 = 0; s0 < pt.splits; s0 += kBatch, base += kBatch * pt.split_stride) {
    if constexpr (VEC == 4) {
      float4 f[kBatch][NV];
#pragma unroll
      for (int b = 0; b < kBatch; ++b)
#pragma unroll
        for (int t = 0; t < NV; ++t)
          f[b][t] = s0 + b < pt.splits ? __ldcg(reinterpret_cast<const float4*>(base + b * pt.split_stride + off[t]))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int b = 0; b < kBatch; ++b)
#pragma unroll
        for (int t = 0; t < NV; ++t) {
          acc[4 * t] += f[b][t].x, acc[4 * t + 1] += f[b][t].y, acc[4 * t + 2] += f[b][t].z, acc[4 * t + 3] += f[b][t].w;
        }
    } else {
      float f[kBatch][NV];
#pragma unroll
      for (int b = 0; b < kBatch; ++b)
#pragma unroll
        for (int t = 0; t < NV; ++t) f[b][t] = s0 + b < pt.splits ? __ldcg(base + b * pt.split_stride + off[t]) : 0.f;
#pragma unroll
      for (int b = 0; b < kBatch; ++b)
#pragma unroll
        for (int t = 0; t < NV; ++t) acc[t] += f[b][t];
    }
  }
}

// VEC consecutive bf16 at p, widened / narrowed.
template <int VEC>
__device__ __forceinline__ void ld_bf16(const bf16* p, float* v) {
  if constexpr (VEC == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
  } else {
    v[0] = __bfloat162float(*p);
  }
}

template <int VEC>
__device__ __forceinline__ void st_bf16(bf16* p, const float* v) {
  if constexpr (VEC == 4) {
    uint2 u;
    *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = u;
  } else {
    *p = __float2bfloat16(v[0]);
  }
}

__device__ __forceinline__ float group_sum(float v, int gtid, float* red, const GroupBar& bar) {
  v = warp_add(v);
  if ((gtid & 31) == 0) red[gtid >> 5] = v;
  bar.sync();
  const float s = red[0] + red[1] + red[2] + red[3];
  bar.sync();
  return s;
}

struct Team {  // a 128-thread worker group
  int group, n_groups, gtid;
  float* red;
  GroupBar bar;
};

// ---- row-wise phases: one 128-thread group per row of hidden size NV * VEC * 128 -----------------------------

// res = v; x = bf16(v * rsqrt(mean(v^2) + eps) * gain)   (v already holds bf16-representable values)
// This thread's columns of the norm gain, as raw bf16 (fetched before the row's sums are waited on).
template <int NV, int VEC>
struct Gain {
  bf16 g[NV * VEC];
  __device__ __forceinline__ Gain(const bf16* gain, int gtid) {
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      if constexpr (VEC == 4)
        *reinterpret_cast<uint2*>(&g[t * 4]) = __ldg(reinterpret_cast<const uint2*>(gain + row_col<NV, VEC>(t, gtid)));
      else
        g[t] = gain[row_col<NV, VEC>(t, gtid)];
    }
  }
};

template <int NV, int VEC>
__device__ __forceinline__ void norm_store(const float (&v)[NV * VEC], float ss, int dim, float eps,
                                           const Gain<NV, VEC>& gain, bf16* res_row, bf16* out_row, const Team& tm) {
  const float r = rsqrtf(group_sum(ss, tm.gtid, tm.red, tm.bar) / dim + eps);
#pragma unroll
  for (int t = 0; t < NV; ++t) {
    const int col = row_col<NV, VEC>(t, tm.gtid);
    float g[VEC], o[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) g[e] = __bfloat162float(gain.g[t * VEC + e]);
#pragma unroll
    for (int e = 0; e < VEC; ++e) o[e] = v[t * VEC + e] * r * g[e];
    if (res_row) st_bf16<VEC>(res_row + col, &v[t * VEC]);
    if (out_row) st_bf16<VEC>(out_row + col, o);
  }
}

template <int NV, int VEC>
__device__ __noinline__ void embed_norm_rows(const Phase& ph, const TickIo& io, const Team& tm, uint32_t* err) {
  const int dim = ph.N;
  const bf16 *pad = (const bf16*)ph.src0, *codec_emb = (const bf16*)ph.src1, *p_emb = (const bf16*)ph.src2;
  if (tm.group >= ph.rows) return;
  const Gain<NV, VEC> gain((const bf16*)ph.src3, tm.gtid);
  for (int row = tm.group; row < ph.rows; row += tm.n_groups) {
    const int32_t* codes =
        reinterpret_cast<const int32_t*>(static_cast<const char*>(io.state) + (int64_t)io.lines[row] * io.stride);
    float v[NV * VEC];
#pragma unroll
    for (int t = 0; t < NV; ++t) ld_bf16<VEC>(pad + row_col<NV, VEC>(t, tm.gtid), &v[t * VEC]);
    // f32 sum in the reference's order: pad, codebook 0, codebooks 1.. (talker.cu:76-96)
    for (int g = 0; g < ph.i2; ++g) {
      int c = codes[g];
      if (c < 0 || c >= (g == 0 ? ph.i0 : ph.i1)) {
        if (tm.gtid == 0) raise(err, kErrBadIndex);
        c = 0;
      }
      const bf16* rowp = g == 0 ? codec_emb + (int64_t)c * dim : p_emb + ((int64_t)(g - 1) * ph.i1 + c) * dim;
#pragma unroll
      for (int t = 0; t < NV; ++t) {
        float e[VEC];
        ld_bf16<VEC>(rowp + row_col<NV, VEC>(t, tm.gtid), e);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v[t * VEC + k] += e[k];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV * VEC; ++i) {
      v[i] = bf16_round(v[i]);
      ss += v[i] * v[i];
    }
    norm_store<NV, VEC>(v, ss, dim, ph.f0, gain, (bf16*)ph.dst0 + (int64_t)row * dim,
                        (bf16*)ph.dst1 + (int64_t)row * dim, tm);
  }
}

template <int NV, int VEC>
__device__ __noinline__ void reduce_norm_rows(const Phase& ph, const float* partials, const Team& tm) {
  const int dim = ph.N;
  const bf16* bias = (const bf16*)ph.src0;
  const Partials pt(partials, ph);
  if (tm.group >= ph.rows) return;
  const Gain<NV, VEC> gain((const bf16*)ph.src3, tm.gtid);
  for (int row = tm.group; row < ph.rows; row += tm.n_groups) {
    float v[NV * VEC], ss = 0.f;
    reduce_row<NV, VEC>(pt, row, tm.gtid, v);
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      float b[VEC];
      if (bias) ld_bf16<VEC>(bias + row_col<NV, VEC>(t, tm.gtid), b);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float a = bf16_round(v[t * VEC + e]);
        if (bias) a = bf16_round(a + b[e]);
        v[t * VEC + e] = a;
        ss += a * a;
      }
    }
    norm_store<NV, VEC>(v, ss, dim, ph.f0, gain, (bf16*)ph.dst0 + (int64_t)row * dim,
                        (bf16*)ph.dst1 + (int64_t)row * dim, tm);
  }
}

template <int NV, int VEC>
__device__ __noinline__ void add_norm_rows(const Phase& ph, const float* partials, const Team& tm) {
  const int dim = ph.N, every = ph.i0, which = ph.i1;
  bf16 *res = (bf16*)ph.dst0, *out = (bf16*)ph.dst1;
  const Partials pt(partials, ph);
  if (tm.group >= ph.rows) return;
  const Gain<NV, VEC> gain((const bf16*)ph.src3, tm.gtid);
  for (int row = tm.group; row < ph.rows; row += tm.n_groups) {
    float v[NV * VEC], old[NV * VEC], ss = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) ld_bf16<VEC>(res + (int64_t)row * dim + row_col<NV, VEC>(t, tm.gtid), &old[t * VEC]);
    reduce_row<NV, VEC>(pt, row, tm.gtid, v);
#pragma unroll
    for (int i = 0; i < NV * VEC; ++i) {
      v[i] = bf16_round(v[i]) + old[i];  // the norm runs over the unrounded sum (qwen3.cu:34)
      ss += v[i] * v[i];
    }
    const bool keep = row % every == which;
    norm_store<NV, VEC>(v, ss, dim, ph.f0, gain, res + (int64_t)row * dim,
                        keep ? out + (int64_t)(row / every) * dim : nullptr, tm);
  }
}

// AddNorm of a 1024- or 2048-wide row by all 256 workers of a CTA (one row per CTA, when the phase has no more rows
// than the grid has CTAs): a thread owns columns 4 (256 j + t) .. + 3 for j < kDim / 1024, so the partial tiles of up
// to eight K splits are one batch of at most sixteen 16-byte loads per thread (a 128-thread group needs two batches,
// two L2 round trips, for a 2048-wide row). The splits are summed in split order per element, as everywhere.
template <int kDim>
__device__ __noinline__ void add_norm_rows_wide(const Phase& ph, const float* partials, int wtid, float* red) {
  constexpr int NJ = kDim / (kWorkerThreads * 4);
  const int row = blockIdx.x, every = ph.i0, which = ph.i1;
  if (row >= ph.rows) return;
  bf16 *res = (bf16*)ph.dst0 + (int64_t)row * kDim, *out = (bf16*)ph.dst1;
  const bf16* gain = (const bf16*)ph.src3;
  const Partials pt(partials, ph);
  int col[NJ];
  uint32_t off[NJ];
  uint2 graw[NJ];
  float v[4 * NJ], old[4 * NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    col[j] = (j * kWorkerThreads + wtid) * 4;
    off[j] = pt.at(row, col[j]);
    graw[j] = __ldg(reinterpret_cast<const uint2*>(gain + col[j]));
    ld_bf16<4>(res + col[j], &old[j * 4]);
  }
#pragma unroll
  for (int i = 0; i < 4 * NJ; ++i) v[i] = 0.f;
  const float* base = pt.base;
  for (int s0 = 0; s0 < pt.splits; s0 += 8, base += 8 * pt.split_stride) {
    float4 f[8][NJ];
#pragma unroll
    for (int b = 0; b < 8; ++b)
#pragma unroll
      for (int j = 0; j < NJ; ++j)
        f[b][j] = s0 + b < pt.splits ? __ldcg(reinterpret_cast<const float4*>(base + b * pt.split_stride + off[j]))
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int b = 0; b < 8; ++b)
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        v[4 * j] += f[b][j].x, v[4 * j + 1] += f[b][j].y, v[4 * j + 2] += f[b][j].z, v[4 * j + 3] += f[b][j].w;
      }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4 * NJ; ++i) {
    v[i] = bf16_round(v[i]) + old[i];  // the norm runs over the unrounded sum (qwen3.cu:34)
    ss += v[i] * v[i];
  }
  ss = warp_add(ss);
  if ((wtid & 31) == 0) red[wtid >> 5] = ss;
  WorkerSync::sync();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < kWorkerThreads / 32; ++w) total += red[w];
  WorkerSync::sync();
  const float r = rsqrtf(total / kDim + ph.f0);
  const bool keep = row % every == which;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw[j].x));
    const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw[j].y));
    const float g[4] = {g0.x, g0.y, g1.x, g1.y};
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = v[4 * j + e] * r * g[e];
    st_bf16<4>(res + col[j], &v[4 * j]);
    if (keep) st_bf16<4>(out + (int64_t)(row / every) * kDim + col[j], o);
  }
}

// Hidden sizes the decoder stacks use: 128 and 256 column by column, 512 .. 2048 four columns at a time.
#define OMNI_ROW_DISPATCH(fn, dim, ...)        \
  switch (dim) {                               \
    case 128: fn<1, 1>(__VA_ARGS__); break;    \
    case 256: fn<2, 1>(__VA_ARGS__); break;    \
    case 512: fn<1, 4>(__VA_ARGS__); break;    \
    case 1024: fn<2, 4>(__VA_ARGS__); break;   \
    case 2048: fn<4, 4>(__VA_ARGS__); break;   \
    default: break;                            \
  }

// SwiGLU over split-K partials of the gate|up GEMM (each tile holds tile_n/2 gate channels then the matching up
// channels): act[m, c] = bf16(bf16(silu(bf16(gate))) * bf16(up)). One group per (row, 512-channel chunk).
__device__ __noinline__ void reduce_silu_rows(const Phase& ph, const float* partials, const Team& tm) {
  const int inter = ph.i0, chunks = (inter + 4 * kGroupThreads - 1) / (4 * kGroupThreads), half = ph.tile_n >> 1;
  bf16* act = (bf16*)ph.dst0;
  const Partials pt(partials, ph);
  for (int it = tm.group; it < ph.rows * chunks; it += tm.n_groups) {
    const int row = it % ph.rows, c0 = (it / ph.rows) * 4 * kGroupThreads;
    int cols[8];
    float v[8];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int c = min(c0 + q * kGroupThreads + tm.gtid, inter - 1);
      cols[q] = (c / half) * ph.tile_n + c % half;  // gate
      cols[4 + q] = cols[q] + half;                 // up
    }
    reduce_cols<8>(pt, row, cols, v);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int c = c0 + q * kGroupThreads + tm.gtid;
      if (c < inter) {
        const float g = bf16_round(v[q]), u = bf16_round(v[4 + q]);
        act[(int64_t)row * inter + c] = __float2bfloat16(bf16_round(g / (1.f + __expf(-g))) * u);
      }
    }
  }
}

// ---- rope + KV write + attention --------------------------------------------------------------------------------
// A team of W warps per (sequence, kv head): two warps for the talker's paged KV (pages alternate between the
// warps), one warp for the code predictor's single-page frames (so all eight worker warps of a CTA hold an item).

template <int D, int G, int W, typename TeamSync>
__device__ __noinline__ void rope_attend_item(const Phase& ph, const TickIo& io, const float* partials, int seq, int kh,
                                              int tid, AttnShared<D, G, W>& sh, const TeamSync& team, uint32_t* err,
                                              unsigned long long* stamp = nullptr) {
  constexpr int E = D / 64, VE = D / 32;
  const int hq = ph.i0, hk = ph.i1, per = ph.i3, base = ph.i4;
  const bool paged = ph.i5 != 0;
  const bf16 *q_norm = (const bf16*)ph.src0, *k_norm = (const bf16*)ph.src1;
  bf16 *kv = (bf16*)ph.dst0, *out = (bf16*)ph.dst1;
  const int lane = tid & 31, warp = tid >> 5;
  const float scale = rsqrtf((float)D);
  const Partials pt(partials, ph);
  float qwl[E], qwh[E], kwl[E], kwh[E];  // this lane's q/k norm gains, fetched before any partial sum is waited on
#pragma unroll
  for (int e = 0; e < E; ++e) {
    qwl[e] = __bfloat162float(q_norm[lane * E + e]), qwh[e] = __bfloat162float(q_norm[D / 2 + lane * E + e]);
    kwl[e] = __bfloat162float(k_norm[lane * E + e]), kwh[e] = __bfloat162float(k_norm[D / 2 + lane * E + e]);
  }
  for (int r = 0; r < per; ++r) {
    const int n = seq * per + r;
    const int pos = paged ? io.d_pos[n] : base + r;
    float cs[E], sn[E];
    // (the two-warp path takes its angles after it has asked for its partial sums: the row's position is a load there)
    if constexpr (!(G == 2 && W == 2 && D == 128)) rope_angles<D>(lane, pos, ph.f1, cs, sn);
    const int64_t slot = paged ? io.d_slot[n] : (int64_t)seq * 16 + pos;
    int64_t page = slot >> 4;
    const int tok = (int)(slot & 15);
    if (page < 0 || page >= ph.i6) {
      if (tid == 0) raise(err, kErrBadIndex);
      page = 0;
    }
    bf16* kdst = kv + kv_offset<D>(page, hk, kh, 0, tok);
    bf16* vdst = kv + kv_offset<D>(page, hk, kh, 1, tok);
    if constexpr (W == 1) {
      // one warp does the G query heads, the key head and the value head; all their partial sums in one batch,
      // E consecutive columns per load (a lane owns value dims lane * VE .. + VE)
      constexpr int NG = (G + 1) * 2 + VE / E;
      int cols[NG];
      float val[NG * E];
#pragma unroll
      for (int j = 0; j <= G; ++j) {
        const int col0 = (j < G ? kh * G + j : hq + kh) * D;
        cols[j * 2] = col0 + lane * E;
        cols[j * 2 + 1] = col0 + D / 2 + lane * E;
      }
#pragma unroll
      for (int g = 0; g < VE / E; ++g) cols[(G + 1) * 2 + g] = (hq + hk + kh) * D + lane * VE + g * E;
      if (ph.src2) {
        // the row's q | k | v were computed at load for every code (a pass's first-layer input is a function of the
        // code drawn before it alone): read the code's row instead of summing partial tiles of a GEMM
        const int code = io.codes[n * 16 + ph.i7];
        const bf16* qkv_row = (const bf16*)ph.src2 + (int64_t)code * ph.i8;
#pragma unroll
        for (int j = 0; j < NG; ++j) {
          if constexpr (E == 2) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(qkv_row + cols[j]));
            val[j * E] = f.x, val[j * E + 1] = f.y;
          } else {
            val[j] = __bfloat162float(qkv_row[cols[j]]);
          }
        }
      } else {
        reduce_vecs<NG, E>(pt, n, cols, val);
      }
#pragma unroll
      for (int j = 0; j <= G; ++j) {
        float lo[E], hi[E];
#pragma unroll
        for (int e = 0; e < E; ++e) lo[e] = bf16_round(val[j * 2 * E + e]), hi[e] = bf16_round(val[j * 2 * E + E + e]);
        if (j < G) rope_head<D>(lo, hi, qwl, qwh, cs, sn, ph.f0);
        else rope_head<D>(lo, hi, kwl, kwh, cs, sn, ph.f0);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int i = lane * E + e;
          if (j < G) {
            sh.qs[j][i] = lo[e], sh.qs[j][D / 2 + i] = hi[e];
          } else {
            kdst[i] = __float2bfloat16(lo[e]), kdst[D / 2 + i] = __float2bfloat16(hi[e]);
          }
        }
      }
#pragma unroll
      for (int e = 0; e < VE; ++e) vdst[lane * VE + e] = __float2bfloat16(val[(G + 1) * 2 * E + e]);
    } else if constexpr (G == 2 && W == 2 && D == 128) {
      // two query heads, the key head and the value head over two warps: each warp takes one query head and one of
      // key / value, and asks for all its partial sums in one batch (one L2 round trip instead of two)
      const int qcol = (kh * G + warp) * D, kcol = (hq + kh) * D, vcol = (hq + hk + kh) * D;
      int cols[4];
      cols[0] = qcol + lane * E, cols[1] = qcol + D / 2 + lane * E;
      if (warp == 0) cols[2] = kcol + lane * E, cols[3] = kcol + D / 2 + lane * E;
      else cols[2] = vcol + lane * VE, cols[3] = vcol + lane * VE + E;
      float val[4 * E], lo[E], hi[E];
      reduce_vecs<4, E>(pt, n, cols, val);
      rope_angles<D>(lane, pos, ph.f1, cs, sn);
#pragma unroll
      for (int e = 0; e < E; ++e) lo[e] = bf16_round(val[e]), hi[e] = bf16_round(val[E + e]);
      rope_head<D>(lo, hi, qwl, qwh, cs, sn, ph.f0);
#pragma unroll
      for (int e = 0; e < E; ++e) sh.qs[warp][lane * E + e] = lo[e], sh.qs[warp][D / 2 + lane * E + e] = hi[e];
      if (warp == 0) {
#pragma unroll
        for (int e = 0; e < E; ++e) lo[e] = bf16_round(val[2 * E + e]), hi[e] = bf16_round(val[3 * E + e]);
        rope_head<D>(lo, hi, kwl, kwh, cs, sn, ph.f0);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          kdst[lane * E + e] = __float2bfloat16(lo[e]);
          kdst[D / 2 + lane * E + e] = __float2bfloat16(hi[e]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < VE; ++e) vdst[lane * VE + e] = __float2bfloat16(val[2 * E + e]);
      }
    } else {
      for (int job = warp; job < G + 2; job += W) {
        if (job == G + 1) {  // value: plain copy
          int cols[1] = {(hq + hk + kh) * D + lane * VE};
          float val[VE];
          reduce_vecs<1, VE>(pt, n, cols, val);
#pragma unroll
          for (int e = 0; e < VE; ++e) vdst[lane * VE + e] = __float2bfloat16(val[e]);
          continue;
        }
        const bool is_q = job < G;
        const int col0 = (is_q ? kh * G + job : hq + kh) * D;
        int cols[2] = {col0 + lane * E, col0 + D / 2 + lane * E};
        float val[2 * E], lo[E], hi[E];
        reduce_vecs<2, E>(pt, n, cols, val);
#pragma unroll
        for (int e = 0; e < E; ++e) lo[e] = bf16_round(val[e]), hi[e] = bf16_round(val[E + e]);
        if (is_q) rope_head<D>(lo, hi, qwl, qwh, cs, sn, ph.f0);
        else rope_head<D>(lo, hi, kwl, kwh, cs, sn, ph.f0);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const int i = lane * E + e;
          if (is_q) {
            sh.qs[job][i] = lo[e], sh.qs[job][D / 2 + i] = hi[e];
          } else {
            kdst[i] = __float2bfloat16(lo[e]), kdst[D / 2 + i] = __float2bfloat16(hi[e]);
          }
        }
      }
    }
    __threadfence_block();
    team.sync();
    if (stamp && tid == 0) stamp[0] = sm100::global_timer_ns();  // q/k/v summed, normed, rotated, K/V written
    attend_pages<D, G, W>(sh, kv, paged ? io.pages + io.indptr[n] : nullptr, seq, pos + 1, hk, kh, scale,
                          out + ((int64_t)n * hq + kh * G) * D, tid, team);
    if (stamp && tid == 0) stamp[1] = sm100::global_timer_ns();  // attention of the item's row done
  }
}

template <int D, int G>
__device__ __forceinline__ void rope_attn_dg(const Phase& ph, const TickIo& io, const float* partials, const Team& tm,
                                             int wtid, WorkerScratch& scratch, uint32_t* err, unsigned long long* stamp) {
  const int hk = ph.i1, per = ph.i3;
  const int items = (ph.rows / per) * hk;
  if (ph.i5) {  // paged: a two-warp team per item, so one round covers 4 x (number of CTAs) items
    const int team = wtid >> 6;
    auto& sh = reinterpret_cast<AttnShared<D, G, 2>&>(scratch.attn2[team]);
    const int first = team * (int)gridDim.x + (int)blockIdx.x, n_teams = 4 * (int)gridDim.x;
    for (int it = first; it < items; it += n_teams)
      rope_attend_item<D, G, 2>(ph, io, partials, it / hk, it % hk, wtid & 63, sh, PairBar{4 + team}, err,
                                wtid == 0 ? stamp : nullptr);
  } else {  // one page per sequence: a warp per item
    auto& sh = reinterpret_cast<AttnShared<D, G, 1>&>(scratch.attn1[wtid >> 5]);
    // warp ids run over the CTAs first, so a phase with few items spreads over as many SMs as it has items
    const int wid = (wtid >> 5) * (int)gridDim.x + (int)blockIdx.x, n_warps = (int)gridDim.x * (kWorkerThreads / 32);
    for (int it = wid; it < items; it += n_warps)
      rope_attend_item<D, G, 1>(ph, io, partials, it / hk, it % hk, wtid & 31, sh, WarpSync(), err, wtid == 0 ? stamp : nullptr);
  }
}

__device__ __forceinline__ void phase_rope_attn(const Phase& ph, const TickIo& io, const float* partials, const Team& tm,
                                                int wtid, WorkerScratch& scratch, uint32_t* err, unsigned long long* stamp) {
  const int D = ph.i2, G = ph.i0 / ph.i1;
  if (D == 128) {
    if (G == 1) rope_attn_dg<128, 1>(ph, io, partials, tm, wtid, scratch, err, stamp);
    else if (G == 2) rope_attn_dg<128, 2>(ph, io, partials, tm, wtid, scratch, err, stamp);
    else rope_attn_dg<128, 4>(ph, io, partials, tm, wtid, scratch, err, stamp);
  } else {
    if (G == 1) rope_attn_dg<64, 1>(ph, io, partials, tm, wtid, scratch, err, stamp);
    else if (G == 2) rope_attn_dg<64, 2>(ph, io, partials, tm, wtid, scratch, err, stamp);
    else rope_attn_dg<64, 4>(ph, io, partials, tm, wtid, scratch, err, stamp);
  }
}

// The next predictor pass's input when the code embeddings were sent through the input projection at load: the drawn
// code's projected row IS the pass's residual start, and its RMSNorm the first layer's input (what the projection GEMM
// and the ReduceNorm phase after it would produce, without either phase). One 128-thread group.
template <int NV, int VEC>
__device__ __forceinline__ void projected_input_row(const bf16* table_row, const bf16* gain_ptr, float eps, int dim,
                                                    bf16* res_row, bf16* out_row, const Team& tm) {
  const Gain<NV, VEC> gain(gain_ptr, tm.gtid);
  float v[NV * VEC], ss = 0.f;
#pragma unroll
  for (int t = 0; t < NV; ++t) ld_bf16<VEC>(table_row + row_col<NV, VEC>(t, tm.gtid), &v[t * VEC]);
#pragma unroll
  for (int i = 0; i < NV * VEC; ++i) ss += v[i] * v[i];
  norm_store<NV, VEC>(v, ss, dim, eps, gain, res_row, out_row, tm);
}

// ---- head reduce + draw + next predictor input: one row per CTA (all 256 workers) -----------------------------

__device__ __noinline__ void phase_sample(const Phase& ph, const TickIo& io, const float* partials, int wtid, sampler::Shared& sh,
                                          unsigned long long* stamp, const Team& tm) {
  using Team = sampler::Team<kWorkerThreads, WorkerSync>;
  const int g = gridDim.x;
  bf16* logits_out = (bf16*)ph.dst0;
  sampler::Params prm;
  prm.vocab = ph.N;
  prm.temperature = ph.f0;
  prm.top_p = ph.f1;
  prm.penalty = ph.f2;
  prm.top_k = ph.i1;
  prm.suppress_lo = ph.i2;
  prm.suppress_hi = ph.i3;
  prm.exempt = ph.i4;
  prm.min_frames = ph.i5;
  prm.penalize = ph.i6;
  prm.group = ph.i7;
  prm.philox = ph.i10;
  prm.seen_words = io.seen_words;
  for (int row = first_item(ph); row < ph.rows; row += g) {
    int32_t* slot = reinterpret_cast<int32_t*>(static_cast<char*>(io.state) + (int64_t)io.lines[row] * io.stride);
    // everything the draw needs besides the logits is fetched before the partial sums are waited on
    const int forced = io.force[row * 16 + prm.group], frame = io.frames[row];
    const float uniform = io.uniforms[row * 16 + prm.group];
    const uint32_t seen_bits = Team::seen_word(slot, prm, wtid);
    // The head's split-K partials are summed with every warp reading whole 512-byte runs of a tile row (thread t takes
    // columns 4 (256 j + t) .. + 3), rounded and published from there; a thread's own PER consecutive logits then
    // come back through shared memory (the nucleus arrays, idle until the draw needs them).
    float mine[Team::PER];
    {
      float* stage = reinterpret_cast<float*>(sh.cand_idx);  // cand_idx | cand_p | sorted_idx | sorted_p: kVocabMax floats
      static_assert(offsetof(sampler::Shared, sorted_p) - offsetof(sampler::Shared, cand_idx) == 3 * sampler::kMaxNucleus * 4 &&
                        4 * sampler::kMaxNucleus >= sampler::kVocabMax,
                    "the four nucleus arrays are contiguous and hold a row of logits");
      const Partials pt(partials, ph);
#pragma unroll
      for (int j0 = 0; j0 < Team::PER / 4; j0 += 2) {
        if ((j0 * kWorkerThreads) * 4 >= prm.vocab) break;  // CTA-uniform: no column of this round is inside the vocabulary
        int cols[2];
        float sum[8];
#pragma unroll
        for (int j = 0; j < 2; ++j) cols[j] = min(((j0 + j) * kWorkerThreads + wtid) * 4, prm.vocab - 4);
        reduce_vecs<2, 4>(pt, row, cols, sum);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int col = ((j0 + j) * kWorkerThreads + wtid) * 4;
          if (col < prm.vocab) {
            float r[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) r[e] = bf16_round(sum[j * 4 + e]);
            *reinterpret_cast<float4*>(stage + col) = make_float4(r[0], r[1], r[2], r[3]);
            st_bf16<4>(logits_out + (int64_t)row * ph.i0 + col, r);
          }
        }
      }
      WorkerSync::sync();
#pragma unroll
      for (int j = 0; j < Team::PER; j += 4) {
        const int col = wtid * Team::PER + j;
        const float4 v = col < prm.vocab ? *reinterpret_cast<const float4*>(stage + col) : make_float4(0.f, 0.f, 0.f, 0.f);
        mine[j] = v.x, mine[j + 1] = v.y, mine[j + 2] = v.z, mine[j + 3] = v.w;
      }
      WorkerSync::sync();  // the staging rows are the draw's nucleus arrays again
    }
    if (stamp && wtid == 0) stamp[0] = sm100::global_timer_ns();  // the row's logits are summed
    const int token = Team::sample_row([&](int, int j) { return mine[j]; }, prm, frame, uniform, forced, slot, seen_bits,
                                       io.codes + row * 16 + prm.group, wtid, sh);
    if (stamp && wtid == 0) stamp[1] = sm100::global_timer_ns();  // the token is drawn
    // the next predictor pass reads the embedding of the code just drawn
    const int dim = ph.i9;
    if (ph.i8 == kNextHiddenAndCode) {
      const bf16 *table = (const bf16*)ph.src0, *hidden = (const bf16*)ph.src1;
      bf16* dst = (bf16*)ph.dst1;
      for (int i = wtid * 8; i < dim; i += kWorkerThreads * 8) {
        *reinterpret_cast<uint4*>(dst + ((int64_t)2 * row) * dim + i) =
            *reinterpret_cast<const uint4*>(hidden + (int64_t)row * dim + i);
        *reinterpret_cast<uint4*>(dst + ((int64_t)2 * row + 1) * dim + i) =
            *reinterpret_cast<const uint4*>(table + (int64_t)token * dim + i);
      }
    } else if (ph.i8 == kNextCode) {
      const bf16* table = (const bf16*)ph.src0;
      bf16* dst = (bf16*)ph.dst1;
      for (int i = wtid * 8; i < dim; i += kWorkerThreads * 8)
        *reinterpret_cast<uint4*>(dst + (int64_t)row * dim + i) =
            *reinterpret_cast<const uint4*>(table + (int64_t)token * dim + i);
    } else if (ph.i8 == kNextProjected && wtid < kGroupThreads) {
      // the next pass's first attention phase reads the code's q | k | v row (src1, i11 bytes): ask it into L2 now
      if (wtid == 0 && ph.src1) sm100::prefetch_l2((const char*)ph.src1 + (int64_t)token * ph.i11, (uint32_t)ph.i11);
      const bf16* src = (const bf16*)ph.src0 + (int64_t)token * dim;
      bf16 *res = (bf16*)ph.dst1 + (int64_t)row * dim, *out = (bf16*)ph.dst2 + (int64_t)row * dim;
      switch (dim) {
        case 256: projected_input_row<2, 1>(src, (const bf16*)ph.src3, ph.f3, dim, res, out, tm); break;
        case 512: projected_input_row<1, 4>(src, (const bf16*)ph.src3, ph.f3, dim, res, out, tm); break;
        case 1024: projected_input_row<2, 4>(src, (const bf16*)ph.src3, ph.f3, dim, res, out, tm); break;
        case 2048: projected_input_row<4, 4>(src, (const bf16*)ph.src3, ph.f3, dim, res, out, tm); break;
        default: projected_input_row<1, 1>(src, (const bf16*)ph.src3, ph.f3, dim, res, out, tm); break;  // 128
      }
    }
    WorkerSync::sync();
  }
}

// ---- GEMM epilogue: a worker thread owns one activation row (its TMEM lane) and half of the tile's columns -------

__device__ __noinline__ void gemm_epilogue(const Phase& ph, float* partials, int tile, int split, uint32_t tmem_acc,
                                           int row_base, int wwarp, int lane) {
  // a warp may only touch the TMEM lanes of its quadrant, (warp index in the CTA) % 4
  const int quad = (wwarp + kFirstWorkerWarp) & 3, half = wwarp >> 2;
  const int m = row_base + quad * 32 + lane, tn = ph.tile_n;  // row_base: 128 for the second half of a 256-row tile
  if (row_base + quad * 32 >= ph.rows) return;  // no live row in this warp's quadrant (warp-uniform)
  const uint32_t lane_addr = tmem_acc + ((uint32_t)(quad * 32) << 16);
  if (ph.mode == kGemmPartials) {
    float* rowp = partials + (((size_t)split * ph.tiles + tile) * ph.bn + min(m, ph.bn - 1)) * tn;
    // 32 columns per round: both loads are under way before the one wait (tn / 2 is 32, 64 or 128 here)
#pragma unroll 1
    for (int c0 = half * (tn / 2); c0 < (half + 1) * (tn / 2); c0 += 32) {
      uint32_t a[16], b[16];
      sm100::tmem_ld16_issue(lane_addr + c0, a);
      sm100::tmem_ld16_issue(lane_addr + c0 + 16, b);
      sm100::tmem_ld_fence(a, b);
      if (m < ph.rows) {
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<uint4*>(rowp + c0 + j) = make_uint4(a[j], a[j + 1], a[j + 2], a[j + 3]);
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<uint4*>(rowp + c0 + 16 + j) = make_uint4(b[j], b[j + 1], b[j + 2], b[j + 3]);
      }
    }
  } else {
    // SwiGLU: columns [0, tn/2) are gate channels tile*tn/2.., columns [tn/2, tn) the matching up channels
    bf16* act = (bf16*)ph.dst0;
    // (16-column chunks alternate between the two warps of a quadrant: hc is 32, 48, 64 or 128)
    const int inter = ph.i0, hc = tn / 2;
#pragma unroll 1
    for (int c0 = half * 16; c0 < hc; c0 += 32) {
      float g[16], u[16];
      {
        uint32_t gr[16], ur[16];
        sm100::tmem_ld16_issue(lane_addr + c0, gr);
        sm100::tmem_ld16_issue(lane_addr + hc + c0, ur);
        sm100::tmem_ld_fence(gr, ur);
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = __uint_as_float(gr[j]), u[j] = __uint_as_float(ur[j]);
      }
      const int ch = tile * hc + c0;
      if (m < ph.rows && ch < inter) {
        float o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float gg = bf16_round(g[j]);
          // the fast division differs from the IEEE one by at most 2 ulp of an f32 that is rounded to bf16 next
          o[j] = bf16_round(__fdividef(gg, 1.f + __expf(-gg))) * bf16_round(u[j]);
        }
        st8(act + (int64_t)m * inter + ch, o);
        st8(act + (int64_t)m * inter + ch + 8, o + 8);
      }
    }
  }
}

// After an abort: waits (bounded) until the last copy this producer issued into each stage it ever used has landed, so
// that no TMA write is in flight when the CTA gives its shared memory back. bit s of `par` is the parity of stage
// s's NEXT use, i.e. the last issued use has the opposite parity; a phase that completed earlier reads as complete.
__device__ __noinline__ void drain_copies(uint64_t* full, uint32_t touched, uint32_t par, uint32_t* err) {
  for (int s = 0; s < kMaxStages; ++s)
    if (touched >> s & 1u) sm100::mbar_wait(sm100::smem_addr(&full[s]), (par >> s & 1u) ^ 1u, err);
}

// kWide: the program has GEMM phases of more than 128 activation rows (buckets above 64: two accumulators per item).
// The narrow instantiation carries none of that code: the 64-session tick is sensitive to the kernel's size.
template <bool kWide>
__global__ void __launch_bounds__(kThreads, 1) tick_kernel(const __grid_constant__ KernelArgs a) {
  using namespace sm100;
  extern __shared__ unsigned char tick_smem_raw[];
  const uint32_t raw = smem_addr(tick_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = tick_smem_raw + (base - raw);
  Control& ctl = *reinterpret_cast<Control*>(base_ptr + a.ring_bytes);
  WorkerScratch& scratch = *reinterpret_cast<WorkerScratch*>(base_ptr + a.ring_bytes + ((sizeof(Control) + 127) & ~127));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;
  constexpr uint32_t kTmemCols = 512;  // two accumulators of 256 f32 columns

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_addr(&ctl.full_w[s]), 1);
      mbar_init(smem_addr(&ctl.full_x[s]), 1);
      mbar_init(smem_addr(&ctl.empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_addr(&ctl.acc_full[b]), 1);
      mbar_init(smem_addr(&ctl.acc_empty[b]), 1);
    }
    ctl.released = 0;
    ctl.abort = *reinterpret_cast<volatile uint32_t*>(a.err) != 0 ? 1 : 0;
    ctl.phase[0] = a.phases[0];
    mbar_init_fence();
  }
  if (warp == 2) tmem_alloc(smem_addr(&ctl.tmem_base), kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;

  if (warp == 0) {
    if (lane == 0) {  // ---- weight producer ----
      Ring ring;
      uint32_t touched = 0;  // stages this thread has issued a copy into
      for (int p = 0; p < a.n_phases && !ctl.abort; ++p) {
        const Phase& ph = a.phases[p];
        if (ph.type != kPhGemm) continue;
        const int items = ph.tiles * ph.splits, nkb = ph.K / kTileK;
        const CUtensorMap* map = a.maps + ph.wmap;
        if (first_item(ph) >= items) continue;
        prefetch_tensormap(map);  // this producer runs ahead of the phase: both descriptors are warm when needed
        prefetch_tensormap(a.maps + ph.xmap);
        {  // weights do not depend on activations, but how far ahead of the barriers they are fetched is bounded
          const uint64_t start = global_timer_ns();
          while (ctl.released < p - a.w_ahead && !ctl.abort) {
            __nanosleep(40);
            if (global_timer_ns() - start > kWaitLimitNs) {
              raise(a.err, kErrBarrierTimeout);
              ctl.abort = 1;
            }
          }
        }
        const int old_n = ring.n;
        if (ring.enter(ph, a.ring_bytes)) {
          // new stage boundaries: every tile of the old geometry must have been consumed before one is overwritten
          for (int s = 0; s < old_n && !ctl.abort; ++s)
            if (!mbar_wait(smem_addr(&ctl.empty[s]), (ring.par >> s & 1u) ^ 1u, a.err)) ctl.abort = 1;
        }
        for (int it = first_item(ph); it < items && !ctl.abort; it += G) {
          const int tile = it % ph.tiles, split = it / ph.tiles;
          const int kb0 = (int)((int64_t)nkb * split / ph.splits), kb1 = (int)((int64_t)nkb * (split + 1) / ph.splits);
          for (int kb = kb0; kb < kb1; kb += ring.kbs) {
            if (!mbar_wait(smem_addr(&ctl.empty[ring.stage]), ring.parity() ^ 1u, a.err)) {
              ctl.abort = 1;
              break;
            }
            const uint32_t bar = smem_addr(&ctl.full_w[ring.stage]);
            mbar_expect_tx(bar, ring.w_slice * (uint32_t)ring.kbs);
            if (ring.kbs == 1)  // rank-2 map: the plain tile copy is about 10 % cheaper than a rank-3 one
              tma_load_2d(base + ring.w_off(), map, bar, kb * kTileK, tile * ph.tile_n, kEvictFirst);
            else
              tma_load_3d(base + ring.w_off(), map, bar, 0, tile * ph.tile_n, kb, kEvictFirst);
            touched |= 1u << ring.stage;
            ring.advance();
          }
        }
      }
      if (ctl.abort) drain_copies(ctl.full_w, touched, ring.par, a.err);
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- activation producer ----
      Ring ring;
      uint32_t touched = 0;
      for (int p = 0; p < a.n_phases && !ctl.abort; ++p) {
        const Phase& ph = a.phases[p];
        if (ph.type != kPhGemm) continue;
        const int items = ph.tiles * ph.splits, nkb = ph.K / kTileK;
        if (first_item(ph) >= items) continue;
        // the rows this phase multiplies were written by earlier phases: wait until those are complete everywhere
        // (by then this CTA's earlier GEMM phases are over too, so a change of stage geometry needs no further wait)
        const uint64_t start = global_timer_ns();
        while (ctl.released < p && !ctl.abort) {
          __nanosleep(40);
          if (global_timer_ns() - start > kWaitLimitNs) {
            raise(a.err, kErrBarrierTimeout);
            ctl.abort = 1;
          }
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");  // generic-proxy writes of other CTAs -> async-proxy reads
        ring.enter(ph, a.ring_bytes);
        const CUtensorMap* map = a.maps + ph.xmap;
        const uint32_t xbytes = (uint32_t)ph.bn * kTileK * 2 * (uint32_t)ring.kbs;
        for (int it = first_item(ph); it < items && !ctl.abort; it += G) {
          const int split = it / ph.tiles;
          const int kb0 = (int)((int64_t)nkb * split / ph.splits), kb1 = (int)((int64_t)nkb * (split + 1) / ph.splits);
          for (int kb = kb0; kb < kb1; kb += ring.kbs) {
            if (!mbar_wait(smem_addr(&ctl.empty[ring.stage]), ring.parity() ^ 1u, a.err)) {
              ctl.abort = 1;
              break;
            }
            const uint32_t bar = smem_addr(&ctl.full_x[ring.stage]);
            mbar_expect_tx(bar, xbytes);
            if (ring.kbs == 1)
              tma_load_2d(base + ring.x_off(), map, bar, kb * kTileK, 0, kEvictLast);
            else
              tma_load_3d(base + ring.x_off(), map, bar, 0, 0, kb, kEvictLast);
            touched |= 1u << ring.stage;
            ring.advance();
          }
        }
      }
      if (ctl.abort) drain_copies(ctl.full_x, touched, ring.par, a.err);
    }
  } else if (warp == 2) {
    if (lane == 0) {  // ---- MMA issuer ----
      Ring ring;
      int buf = 0;
      uint32_t empty_par[2] = {0, 0};
      // A = the activation tile (rows beyond the phase's bn read whatever follows in the ring; those TMEM
      // lanes are never read back), B = tile_n weight rows, both K-major with the 128-byte swizzle
      for (int p = 0; p < a.n_phases && !ctl.abort; ++p) {
        const Phase& ph = a.phases[p];
        if (ph.type != kPhGemm) continue;
        const int items = ph.tiles * ph.splits, nkb = ph.K / kTileK;
        if (first_item(ph) >= items) continue;
        ring.enter(ph, a.ring_bytes);
        const uint32_t idesc = idesc_bf16_f32(kTileM, ph.tile_n);
        if (kWide && ph.bn > kTileM) {
          // 129..256 activation rows: two M = 128 halves per k-block, one into each accumulator (no double buffering)
          for (int it = first_item(ph); it < items && !ctl.abort; it += G) {
            const int split = it / ph.tiles;
            const int kb0 = (int)((int64_t)nkb * split / ph.splits), kb1 = (int)((int64_t)nkb * (split + 1) / ph.splits);
            for (int h = 0; h < 2; ++h) {
              if (!mbar_wait(smem_addr(&ctl.acc_empty[h]), empty_par[h] ^ 1u, a.err)) ctl.abort = 1;
              empty_par[h] ^= 1u;
            }
            if (ctl.abort) break;
            tc_fence_after_sync();
            for (int kb = kb0; kb < kb1; kb += ring.kbs) {
              if (!mbar_wait(smem_addr(&ctl.full_w[ring.stage]), ring.parity(), a.err) ||
                  !mbar_wait(smem_addr(&ctl.full_x[ring.stage]), ring.parity(), a.err)) {
                ctl.abort = 1;
                break;
              }
              tc_fence_after_sync();
              if (a.trace && kb == kb0 && it == first_item(ph)) a.trace[((size_t)p * G + blockIdx.x) * 4] = global_timer_ns();
              for (int j = 0; j < ring.kbs; ++j) {
                const uint64_t bdesc = kmajor_sw128_desc(base + ring.w_off(j));
                for (int h = 0; h < 2; ++h) {
                  const uint64_t adesc = kmajor_sw128_desc(base + ring.x_off(j) + (uint32_t)(h * kTileM * kTileK * 2));
#pragma unroll
                  for (int k = 0; k < kTileK / 16; ++k)
                    mma_bf16(tmem_base + (uint32_t)(h * kTileN), adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                             (kb > kb0 || j > 0 || k > 0) ? 1u : 0u);
                }
              }
              mma_commit(smem_addr(&ctl.empty[ring.stage]));
              ring.advance();
            }
            if (ctl.abort) break;
            mma_commit(smem_addr(&ctl.acc_full[0]));
            mma_commit(smem_addr(&ctl.acc_full[1]));
          }
          continue;
        }
        for (int it = first_item(ph); it < items && !ctl.abort; it += G) {
          const int split = it / ph.tiles;
          const int kb0 = (int)((int64_t)nkb * split / ph.splits), kb1 = (int)((int64_t)nkb * (split + 1) / ph.splits);
          if (!mbar_wait(smem_addr(&ctl.acc_empty[buf]), empty_par[buf] ^ 1u, a.err)) {
            ctl.abort = 1;
            break;
          }
          empty_par[buf] ^= 1u;
          tc_fence_after_sync();
          const uint32_t tmem_d = tmem_base + (uint32_t)(buf * kTileN);
          for (int kb = kb0; kb < kb1; kb += ring.kbs) {
            if (!mbar_wait(smem_addr(&ctl.full_w[ring.stage]), ring.parity(), a.err) ||
                !mbar_wait(smem_addr(&ctl.full_x[ring.stage]), ring.parity(), a.err)) {
              ctl.abort = 1;
              break;
            }
            tc_fence_after_sync();
            if (a.trace && kb == kb0 && it == first_item(ph)) a.trace[((size_t)p * G + blockIdx.x) * 4] = global_timer_ns();
            {
              const uint64_t adesc = kmajor_sw128_desc(base + ring.x_off()), bdesc = kmajor_sw128_desc(base + ring.w_off());
#pragma unroll
              for (int k = 0; k < kTileK / 16; ++k)
                mma_bf16(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
            for (int j = 1; j < ring.kbs; ++j) {
              const uint64_t adesc = kmajor_sw128_desc(base + ring.x_off(j)), bdesc = kmajor_sw128_desc(base + ring.w_off(j));
#pragma unroll
              for (int k = 0; k < kTileK / 16; ++k) mma_bf16(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, 1u);
            }
            mma_commit(smem_addr(&ctl.empty[ring.stage]));
            ring.advance();
          }
          if (ctl.abort) break;
          mma_commit(smem_addr(&ctl.acc_full[buf]));
          buf ^= 1;
        }
      }
    }
  } else if (warp >= kFirstWorkerWarp) {
    // ---- workers ----
    const int wtid = threadIdx.x - kFirstWorkerWarp * 32, wwarp = warp - kFirstWorkerWarp;
    const int grp = wtid >> 7;
    // group ids run over the CTAs first, so a phase with few rows spreads over as many SMs as it has rows
    const Team tm{grp * G + (int)blockIdx.x, G * 2, wtid & 127, ctl.red[grp], GroupBar{2 + grp}};
    int buf = 0;
    uint32_t full_par[2] = {0, 0};
    for (int p = 0; p < a.n_phases; ++p) {
      if (ctl.abort) break;
      // the phase record was copied to shared memory during the previous phase; fetch the next one now
      const Phase& ph = ctl.phase[p & 1];
      if (wtid >= 32 && wtid < 32 + (int)(sizeof(Phase) / 16) && p + 1 < a.n_phases)
        reinterpret_cast<uint4*>(&ctl.phase[(p + 1) & 1])[wtid - 32] =
            __ldg(reinterpret_cast<const uint4*>(a.phases + p + 1) + (wtid - 32));
      switch (ph.type) {
        case kPhGemm: {
          const int items = ph.tiles * ph.splits;
          if (kWide && ph.bn > kTileM) {  // two accumulators per item: rows 0..127 and 128..255
            for (int it = first_item(ph); it < items && !ctl.abort; it += G) {
              for (int h = 0; h < 2; ++h) {
                const bool ok = mbar_wait(smem_addr(&ctl.acc_full[h]), full_par[h], a.err);
                if (!ok) ctl.abort = 1;
                full_par[h] ^= 1u;
                tc_fence_after_sync();
                if (ok)
                  gemm_epilogue(ph, a.partials, it % ph.tiles, it / ph.tiles, tmem_base + (uint32_t)(h * kTileN), h * kTileM,
                                wwarp, lane);
                tc_fence_before_sync();
                WorkerSync::sync();
                if (wtid == 0) mbar_arrive(smem_addr(&ctl.acc_empty[h]));
              }
            }
            break;
          }
          for (int it = first_item(ph); it < items; it += G) {
            const bool ok = mbar_wait(smem_addr(&ctl.acc_full[buf]), full_par[buf], a.err);
            if (!ok) ctl.abort = 1;
            full_par[buf] ^= 1u;
            tc_fence_after_sync();
            if (a.trace && wtid == 0 && it == first_item(ph)) a.trace[((size_t)p * G + blockIdx.x) * 4 + 1] = global_timer_ns();
            if (ok) gemm_epilogue(ph, a.partials, it % ph.tiles, it / ph.tiles, tmem_base + (uint32_t)(buf * kTileN), 0, wwarp, lane);
            tc_fence_before_sync();
            WorkerSync::sync();
            if (wtid == 0) mbar_arrive(smem_addr(&ctl.acc_empty[buf]));
            buf ^= 1;
            if (ctl.abort) break;
          }
          break;
        }
        case kPhEmbedNorm: OMNI_ROW_DISPATCH(embed_norm_rows, ph.N, ph, a.io, tm, a.err); break;
        case kPhReduceNorm: OMNI_ROW_DISPATCH(reduce_norm_rows, ph.N, ph, a.partials, tm); break;
        case kPhAddNorm:
          if (ph.N == 2048 && ph.rows <= G) add_norm_rows_wide<2048>(ph, a.partials, wtid, &ctl.red[0][0]);
          else if (ph.N == 1024 && ph.rows <= G) add_norm_rows_wide<1024>(ph, a.partials, wtid, &ctl.red[0][0]);
          else OMNI_ROW_DISPATCH(add_norm_rows, ph.N, ph, a.partials, tm);
          break;
        case kPhReduceSilu: reduce_silu_rows(ph, a.partials, tm); break;
        case kPhRopeAttn:
          phase_rope_attn(ph, a.io, a.partials, tm, wtid, scratch, a.err, a.trace ? a.trace + ((size_t)p * G + blockIdx.x) * 4 : nullptr);
          break;
        case kPhSample:
          phase_sample(ph, a.io, a.partials, wtid, scratch.sample, a.trace ? a.trace + ((size_t)p * G + blockIdx.x) * 4 : nullptr, tm);
          break;
        default: break;
      }
      // end of phase: the team barrier orders every worker's writes before thread 0's gpu-scope fence and arrival
      // (fences are cumulative), then everyone waits for thread 0 to see all CTAs arrive
      WorkerSync::sync();
      if (wtid == 0) {
        if (a.trace) a.trace[((size_t)p * G + blockIdx.x) * 4 + 2] = global_timer_ns();  // this CTA's share is done
        if (!ctl.abort && !grid_barrier(a.barrier, a.barrier_base + (uint32_t)(p + 1) * (uint32_t)G, a.err)) ctl.abort = 1;
        ctl.released = p + 1;
        if (a.trace) a.trace[((size_t)p * G + blockIdx.x) * 4 + 3] = global_timer_ns();  // every CTA has arrived
      }
      WorkerSync::sync();
    }
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, kTmemCols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static_assert(1024 + kMaxRingBytes + ((sizeof(Control) + 127) & ~127) + sizeof(WorkerScratch) <= 227 * 1024,
              "ring + control + scratch exceed the shared memory of an SM");

size_t tick_smem_bytes(int ring_bytes) {
  // 1 KB of slack to align the ring to the swizzle atom; an activation descriptor spans 128 rows whatever bn is,
  // so the last stage's reads run into the control block and scratch that follow the ring (and are never used)
  return 1024 + (size_t)ring_bytes + ((sizeof(Control) + 127) & ~127) + sizeof(WorkerScratch);
}

// The ring's size. 128 KB by default: with the control block and scratch the CTA then takes the 164 KB shared-memory
// carve-out and 92 KB of the SM's array stay L1. With one k-block per stage 104 KB (132 KB carve-out, 124 KB L1) was
// the faster trade; stages of several k-blocks need the room (two stages of 48 KB for the 128-row weight tiles).
// Measured with multi-k-block stages: 104 / 112 / 120 / 128 / 136 KB -> 6.25 / 6.32 / 6.26 / 6.17 / 6.17 ms per tick.
int tick_ring_bytes() { return 128 * 1024; }

}  // namespace

int tick_ring_size() { return tick_ring_bytes(); }

int tick_add_map(TickProgram* prog, const bf16* base, int rows, int K, int box_rows, int kbs) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return -1;
  // kbs == 1: rank 2, {column, row}, a box of 64 columns x box_rows rows. Otherwise rank 3, {element in a 64-wide
  // k-block, row, k-block}: one copy moves kbs k-blocks of box_rows rows, each landing as its own [box_rows x 128 B]
  // swizzled block.
  const bool flat = kbs == 1;
  const cuuint64_t dims[3] = {(cuuint64_t)(flat ? K : kTileK), (cuuint64_t)rows, (cuuint64_t)(K / kTileK)};
  const cuuint64_t strides[2] = {(cuuint64_t)K * sizeof(bf16), (cuuint64_t)kTileK * sizeof(bf16)};
  const cuuint32_t box[3] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows, (cuuint32_t)kbs};
  const cuuint32_t elem[3] = {1, 1, 1};
  CUtensorMap map;
  const CUresult r = reinterpret_cast<EncodeTiledFn>(fn)(
      &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, flat ? 2 : 3, const_cast<bf16*>(base), dims, strides, box, elem,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -1;
  prog->maps.push_back(map);
  return (int)prog->maps.size() - 1;
}

bool tick_supports(int hidden, int head_dim, int q_heads, int kv_heads, int rows_max) {
  const int g = kv_heads > 0 ? q_heads / kv_heads : 0;
  const bool dim_ok = hidden == 128 || hidden == 256 || hidden == 512 || hidden == 1024 || hidden == 2048;
  return dim_ok && (head_dim == 64 || head_dim == 128) && (g == 1 || g == 2 || g == 4) && rows_max <= 2 * kTileM;
}

int tick_upload(TickProgram* prog) {
  tick_free(prog);
  if (cudaMalloc((void**)&prog->d_phases, prog->phases.size() * sizeof(Phase)) != cudaSuccess) return -1;
  if (cudaMalloc((void**)&prog->d_maps, prog->maps.size() * sizeof(CUtensorMap)) != cudaSuccess) return -1;
  if (cudaMemcpy(prog->d_phases, prog->phases.data(), prog->phases.size() * sizeof(Phase), cudaMemcpyHostToDevice) !=
      cudaSuccess)
    return -1;
  if (cudaMemcpy(prog->d_maps, prog->maps.data(), prog->maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice) !=
      cudaSuccess)
    return -1;
  return 0;
}

void tick_free(TickProgram* prog) {
  if (prog->d_phases) cudaFree(prog->d_phases);
  if (prog->d_maps) cudaFree(prog->d_maps);
  prog->d_phases = nullptr;
  prog->d_maps = nullptr;
}

int tick_configure(int device) {
  const size_t smem = tick_smem_bytes(kMaxRingBytes);
  if (cudaFuncSetAttribute(tick_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
      cudaFuncSetAttribute(tick_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return 0;
  int per_sm = 0, per_sm_wide = 0, sms = 0, coop = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tick_kernel<false>, kThreads, smem) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_wide, tick_kernel<true>, kThreads, smem) != cudaSuccess)
    return 0;
  per_sm = std::min(per_sm, per_sm_wide);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device) != cudaSuccess || !coop) return 0;
  return per_sm >= 1 ? sms : 0;
}

cudaError_t tick_launch(const TickProgram& prog, const TickIo& io, float* partials, uint32_t* barrier,
                        uint32_t* barrier_base, uint32_t* err, int ctas, cudaStream_t stream, unsigned long long* trace) {
  KernelArgs a;
  a.trace = trace;
  a.phases = prog.d_phases;
  a.n_phases = (int)prog.phases.size();
  a.maps = prog.d_maps;
  a.partials = partials;
  a.barrier = barrier;
  a.err = err;
  a.ring_bytes = tick_ring_bytes();
  a.w_ahead = 1 << 20;  // unbounded: limiting the run-ahead to 0 / 1 / 2 phases measured 6.23 / 6.08 / 6.06 ms against 6.06
  a.io = io;
  // the arrival counter runs on from launch to launch (one memset less per tick); it restarts from zero when the
  // next launch could overflow it. After a launch that raised the error word the caller passes *barrier_base = ~0u.
  const uint32_t arrivals = (uint32_t)a.n_phases * (uint32_t)ctas;
  if (*barrier_base > 0xffffffffu - 2u * arrivals) {
    const cudaError_t e = cudaMemsetAsync(barrier, 0, sizeof(uint32_t), stream);
    if (e != cudaSuccess) return e;
    *barrier_base = 0;
  }
  a.barrier_base = *barrier_base;
  *barrier_base += arrivals;
  void* args[] = {&a};
  const void* kernel = prog.max_bn > kTileM ? (const void*)tick_kernel<true> : (const void*)tick_kernel<false>;
  return cudaLaunchCooperativeKernel(kernel, dim3(ctas), dim3(kThreads), args, tick_smem_bytes(a.ring_bytes), stream);
}

}  // namespace omni
