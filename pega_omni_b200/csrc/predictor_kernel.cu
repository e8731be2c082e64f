// The cluster predictor kernel (see predictor.h): 10 warps per CTA, C CTAs per cluster, one cluster per group of at
// most 16 sessions, no communication between clusters.
//   warp 0 / lane 0   weight producer: TMA loads of weight boxes into the stage ring, never waits for activations
//   warp 1 / lane 0   activation producer: TMA loads of activation k-blocks written by the cluster's other CTAs
//   warps 2..9        consumers: thread 0 issues tcgen05.mma (weight rows on M = 128 or 64, the cluster's 16 session rows
//                     on N, accumulator in TMEM; the legacy mma.sync path was measured at a quarter of the rate the
//                     weight stream needs); all eight warps read the accumulator back and run every epilogue, norm,
//                     attention and draw
// Every wait is bounded; a wait that runs out raises the device error word and the CTA unwinds.
#include "predictor.h"

#include <algorithm>

#include "attend.cuh"
#include "rope.cuh"
#include "sampler.cuh"
#include "sm100.cuh"

namespace omni {
namespace {

constexpr int kThreads = 320, kConsumers = 256, kFirstConsumerWarp = 2;
constexpr int kStageW = 32 * 1024;           // weight part of a stage: 128 rows x 2 k-blocks or 64 rows x 4
constexpr int kStageX = 8 * 1024;            // activation part: 16 rows x up to 4 k-blocks
constexpr int kStageBytes = kStageW + kStageX;
constexpr int kStages = 4;
constexpr uint32_t kTmemCols = 32;           // one accumulator of 16 f32 columns (the smallest allocation is 32)
constexpr int kOutPitch = 132;               // floats per row of the epilogue tile (128 columns + 4 of padding)

constexpr int64_t kPrefetchAhead = 1 << 20;   // bytes of a CTA's future weight boxes asked into L2
constexpr int kPrefetchChunk = 64 * 1024;

using ConsumerSync = sampler::NamedSync<1, kConsumers>;
using DrawTeam = sampler::Team<kConsumers, ConsumerSync>;

struct alignas(16) Control {
  uint64_t full_w[kStages], full_x[kStages], empty[kStages];
  uint64_t acc_full;       // the entry's accumulator is complete in TMEM
  uint64_t cbar[2];        // the cluster barrier: every CTA's elected thread arrives on every peer's
  uint32_t tmem_base;
  volatile int bars_done;  // cluster barriers this CTA has passed
  volatile int abort;
};

struct EpilogueTiles {
  float out[1][kPredRows][kOutPitch];  // the accumulator as [session row][weight row of the box]
  float q[kPredRows][128];             // the CTA's query head after norm + RoPE
};
union Scratch {
  EpilogueTiles t;
  sampler::Shared draw;
};

struct KernelArgs {
  const PredEntry* entries;
  int n_entries;
  const CUtensorMap* maps;
  PredConfig cfg;
  int rows, per_cluster;
  TickIo io;
  float* vbuf;  // [rows][hidden] f32: the residual sums the norm runs over, exchanged through L2
  uint32_t* err;
  unsigned long long* trace;  // optional: per entry, the global timer at its start, after its main loop and at its end (cluster 0, rank 0)
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void hw_cluster_sync() {  // every thread of every CTA of the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void remote_arrive(uint32_t local_bar, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_bar), "r"(rank));
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}
__device__ __forceinline__ bool try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// Bounded wait on one of the CTA's own mbarriers; gives up at once when this CTA or any other raised an error.
// `where`: which wait gave up, kept in the upper bits of the error word for the log (the host tests bit 0).
enum WaitSite : uint32_t { kAtWeightEmpty = 1u << 8, kAtRowsReady = 1u << 9, kAtRowsEmpty = 1u << 10, kAtWeightFull = 1u << 11,
                           kAtRowsFull = 1u << 12, kAtClusterBarrier = 1u << 13 };

template <bool kCluster>
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, Control& ctl, uint32_t* err, uint32_t where) {
  uint64_t start = 0;
  for (uint32_t spins = 0;; ++spins) {
    if (kCluster ? try_wait_cluster(bar, parity) : sm100::mbar_try_wait(bar, parity)) return true;
    if ((spins & 255u) == 255u) {
      if (ctl.abort || *reinterpret_cast<volatile uint32_t*>(err) != 0) {
        ctl.abort = 1;
        return false;
      }
      const uint64_t now = sm100::global_timer_ns();
      if (start == 0) start = now;
      if (now - start > sm100::kWaitLimitNs) {
        raise(err, kErrBarrierTimeout | where);
        ctl.abort = 1;
        return false;
      }
    }
  }
}

struct StageWalk {  // the three pipeline roles walk the ring in the same order
  int stage = 0;
  uint32_t par = 0;  // bit s: parity of stage s's next wait
  __device__ __forceinline__ uint32_t parity() const { return par >> stage & 1u; }
  __device__ __forceinline__ void advance() {
    par ^= 1u << stage;
    if (++stage == kStages) stage = 0;
  }
};

__device__ __forceinline__ int weight_row(const PredEntry& e, int rank) {
  if (e.epi == kPeKv) return ((rank & 1) ? e.wrow2 : e.wrow) + (rank >> 1) * e.rows;
  return e.wrow + rank * e.cta_stride;
}

// This thread's TMEM lane, 8 consecutive f32 columns starting at the column encoded in `taddr`.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
  uint32_t r[8];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// Byte offset of element k (a multiple of 8) of row n inside a [rows][64] bf16 block stored with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(int n, int k) { return (uint32_t)(n * 128 + ((((k >> 3) ^ (n & 7)) << 4))); }

// The cluster barrier of the consumer warps: orders everything the cluster's consumers wrote (shared or global
// memory) before everything they read afterwards. Two mbarriers used alternately, so an early arrival for the next
// barrier can never be counted into one a slow peer is still waiting on.
__device__ __forceinline__ bool cluster_barrier(Control& ctl, int& n_bars, int C, int ctid, uint32_t* err) {
  ConsumerSync::sync();
  const uint32_t bar = sm100::smem_addr(&ctl.cbar[n_bars & 1]);
  if (ctid < 32) {
    if (ctid < C) remote_arrive(bar, (uint32_t)ctid);  // lane p arrives on peer p's barrier (C <= 16)
    if (ctid == 0) {  // one thread watches the barrier; the team barrier below passes its acquire on to the others
      wait_bar<true>(bar, (uint32_t)(n_bars >> 1) & 1u, ctl, err, kAtClusterBarrier);
      ctl.bars_done = n_bars + 1;
    }
  }
  ++n_bars;
  ConsumerSync::sync();
  return !ctl.abort;
}

__device__ __forceinline__ void ld_bf16x4(const bf16* p, float* v) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  v[0] = lo.x, v[1] = lo.y, v[2] = hi.x, v[3] = hi.y;
}

// x = bf16(v * rsqrt(mean(v^2) + eps) * gain) for the cluster's rows, v from the exchange buffer, into the resident
// activation tile (k-blocks of [16 rows][64] bf16, swizzled like a TMA box). A warp per row, rows w and w + 8; both
// rows' loads are issued before either is summed (one L2 round trip), and a row is read once. NV = hidden / 128.
template <int NV>
__device__ __forceinline__ void norm_rows(const float* vbuf, const bf16* gain, float eps, int s0, int live, unsigned char* xs,
                                          int cwarp, int lane) {
  constexpr int hidden = NV * 128;
  float4 v[2][NV];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int n = cwarp + 8 * r;
    if (n < live) {
      const float* row = vbuf + (int64_t)(s0 + n) * hidden;
#pragma unroll
      for (int t = 0; t < NV; ++t) v[r][t] = __ldcg(reinterpret_cast<const float4*>(row + t * 128 + lane * 4));
    }
  }
  float g[NV][4];
#pragma unroll
  for (int t = 0; t < NV; ++t) ld_bf16x4(gain + t * 128 + lane * 4, g[t]);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int n = cwarp + 8 * r;
    if (n >= live) continue;  // warp-uniform
    float ss = 0.f;
#pragma unroll
    for (int t = 0; t < NV; ++t) ss += v[r][t].x * v[r][t].x + v[r][t].y * v[r][t].y + v[r][t].z * v[r][t].z + v[r][t].w * v[r][t].w;
    const float rn = rsqrtf(warp_add(ss) / hidden + eps);
#pragma unroll
    for (int t = 0; t < NV; ++t) {
      const int k = t * 128 + lane * 4;
      uint2 u;
      *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(v[r][t].x * rn * g[t][0], v[r][t].y * rn * g[t][1]);
      *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(v[r][t].z * rn * g[t][2], v[r][t].w * rn * g[t][3]);
      *reinterpret_cast<uint2*>(xs + (k >> 6) * (kPredRows * 128) + swz(n, k & 63) + (k & 7) * 2) = u;
    }
  }
}

__device__ __forceinline__ void norm_to_tile(const float* vbuf, const bf16* gain, int hidden, float eps, int s0, int live,
                                             unsigned char* xs, int cwarp, int lane) {
  switch (hidden) {  // 64 * C
    case 128: norm_rows<1>(vbuf, gain, eps, s0, live, xs, cwarp, lane); break;
    case 256: norm_rows<2>(vbuf, gain, eps, s0, live, xs, cwarp, lane); break;
    case 512: norm_rows<4>(vbuf, gain, eps, s0, live, xs, cwarp, lane); break;
    default: norm_rows<8>(vbuf, gain, eps, s0, live, xs, cwarp, lane); break;
  }
}

__global__ void __launch_bounds__(kThreads, 1) pred_kernel(const __grid_constant__ KernelArgs a) {
  using namespace sm100;
  extern __shared__ unsigned char pred_smem_raw[];
  const uint32_t raw = smem_addr(pred_smem_raw);
  unsigned char* base_ptr = pred_smem_raw + (((raw + 1023u) & ~1023u) - raw);
  const uint32_t ring = smem_addr(base_ptr);
  const int xs_bytes = (a.cfg.hidden / 64) * kPredRows * 128;
  unsigned char* xs = base_ptr + kStages * kStageBytes;
  Scratch& scratch = *reinterpret_cast<Scratch*>(xs + xs_bytes);
  float(*res)[64] = reinterpret_cast<float(*)[64]>(reinterpret_cast<unsigned char*>(&scratch) + sizeof(Scratch));
  Control& ctl = *reinterpret_cast<Control*>(reinterpret_cast<unsigned char*>(res) + kPredRows * 64 * sizeof(float));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int C = a.cfg.C, rank = (int)cluster_rank();
  const int s0 = (int)cluster_id() * a.per_cluster;
  const int live = max(0, min(a.per_cluster, a.rows - s0));  // this cluster's sessions

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_addr(&ctl.full_w[s]), 1);
      mbar_init(smem_addr(&ctl.full_x[s]), 1);
      mbar_init(smem_addr(&ctl.empty[s]), 1);
    }
    mbar_init(smem_addr(&ctl.acc_full), 1);
    mbar_init(smem_addr(&ctl.cbar[0]), (uint32_t)C);
    mbar_init(smem_addr(&ctl.cbar[1]), (uint32_t)C);
    ctl.bars_done = 0;
    ctl.abort = *reinterpret_cast<volatile uint32_t*>(a.err) != 0 ? 1 : 0;
    mbar_init_fence();
  }
  // rows past the cluster's sessions stay zero in the resident tile for the whole launch
  for (int i = threadIdx.x * 16; i < xs_bytes; i += kThreads * 16) *reinterpret_cast<uint4*>(xs + i) = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == kFirstConsumerWarp) tmem_alloc(smem_addr(&ctl.tmem_base), kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_acc = ctl.tmem_base;
  hw_cluster_sync();  // every peer's barriers exist before anyone arrives on them

  if (live > 0 && warp == 0) {
    if (lane == 0) {  // ---- weight producer ----
      StageWalk w;
      // Every cluster reads the same weights at about the same time, so the distinct bytes under way from HBM are one
      // cluster's rings (2 MB). Each CTA therefore asks for its own boxes (contiguous: whole rows) into L2 about
      // 1 MB before it loads them (measured: 7 % on the main loops).
      int pf = 0;
      int64_t ahead = 0;
      for (int i = 0; i < a.n_entries && !ctl.abort; ++i) {
        const PredEntry& e = a.entries[i];
        while (pf < a.n_entries && (ahead < kPrefetchAhead || pf <= i)) {
          const PredEntry& f = a.entries[pf];
          const int64_t box_bytes = (int64_t)f.rows * f.nkb * 128;
          const char* src = static_cast<const char*>(f.w) + (int64_t)weight_row(f, rank) * f.nkb * 128;
          for (int64_t off = 0; off < box_bytes; off += kPrefetchChunk)
            sm100::prefetch_l2(src + off, (uint32_t)min((int64_t)kPrefetchChunk, box_bytes - off));
          ahead += box_bytes;
          ++pf;
        }
        ahead -= (int64_t)e.rows * e.nkb * 128;
        const CUtensorMap* map = a.maps + e.wmap;
        const int row = weight_row(e, rank);
        const uint32_t bytes = (uint32_t)e.rows * 128u * (uint32_t)e.kbs;
        for (int kb = 0; kb < e.nkb; kb += e.kbs) {
          if (!wait_bar<false>(smem_addr(&ctl.empty[w.stage]), w.parity() ^ 1u, ctl, a.err, kAtWeightEmpty)) break;
          const uint32_t bar = smem_addr(&ctl.full_w[w.stage]);
          mbar_expect_tx(bar, bytes);
          tma_load_3d(ring + (uint32_t)w.stage * kStageBytes, map, bar, 0, row, kb, kEvictLast);
          w.advance();
        }
      }
    }
  } else if (live > 0 && warp == 1) {
    if (lane == 0) {  // ---- activation producer ----
      StageWalk w;
      for (int i = 0; i < a.n_entries && !ctl.abort; ++i) {
        const PredEntry& e = a.entries[i];
        const int chunks = e.nkb / e.kbs;
        if (e.xmap < 0) {  // the operand is resident: these stages carry weights only
          for (int c = 0; c < chunks; ++c) w.advance();
          continue;
        }
        {  // the rows were written by the cluster's CTAs before cluster barrier number need_bars
          uint64_t start = 0;
          for (uint32_t spins = 0; ctl.bars_done < e.need_bars && !ctl.abort; ++spins) {
            if ((spins & 255u) == 255u) {
              const uint64_t now = global_timer_ns();
              if (start == 0) start = now;
              if (now - start > kWaitLimitNs) {
                raise(a.err, kErrBarrierTimeout | kAtRowsReady);
                ctl.abort = 1;
              }
            }
          }
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");  // generic-proxy writes of other CTAs -> async-proxy reads
        const CUtensorMap* map = a.maps + e.xmap;
        const uint32_t bytes = (uint32_t)kPredRows * 128u * (uint32_t)e.kbs;
        for (int kb = 0; kb < e.nkb && !ctl.abort; kb += e.kbs) {
          if (!wait_bar<false>(smem_addr(&ctl.empty[w.stage]), w.parity() ^ 1u, ctl, a.err, kAtRowsEmpty)) break;
          const uint32_t bar = smem_addr(&ctl.full_x[w.stage]);
          mbar_expect_tx(bar, bytes);
          tma_load_3d(ring + (uint32_t)w.stage * kStageBytes + kStageW, map, bar, 0, s0, e.xz0 + kb, kEvictLast);
          w.advance();
        }
      }
    }
  } else if (live > 0 && warp >= kFirstConsumerWarp) {
    // ---- consumers ----
    const int ctid = threadIdx.x - kFirstConsumerWarp * 32, cw = warp - kFirstConsumerWarp;
    StageWalk w;
    uint32_t xpar = 0;  // bit s: parity of stage s's next activation wait (only some uses of a stage carry activations)
    int n_bars = 0;
    const int hidden = a.cfg.hidden;
    for (int i = 0; i < a.n_entries && !ctl.abort; ++i) {
      const PredEntry& e = a.entries[i];
      const bool tracing = a.trace && ctid == 0 && rank == 0 && s0 == 0;
      if (tracing) a.trace[3 * i] = global_timer_ns();
      // ---- main loop: thread 0 issues the entry's MMAs, D[weight row, session] accumulates in TMEM ----
      const bool narrow = e.rows == 64;
      if (ctid == 0) {
        const uint32_t idesc = idesc_bf16_f32(e.rows, kPredRows);
        bool ok = true;
        for (int kb = 0; kb < e.nkb; kb += e.kbs) {
          const uint32_t stage_base = ring + (uint32_t)w.stage * kStageBytes;
          ok = wait_bar<false>(smem_addr(&ctl.full_w[w.stage]), w.parity(), ctl, a.err, kAtWeightFull);
          if (ok && e.xmap >= 0) {
            ok = wait_bar<false>(smem_addr(&ctl.full_x[w.stage]), xpar >> w.stage & 1u, ctl, a.err, kAtRowsFull);
            xpar ^= 1u << w.stage;
          }
          if (!ok) break;
          tc_fence_after_sync();
          for (int j = 0; j < e.kbs; ++j) {
            const uint64_t adesc = kmajor_sw128_desc(stage_base + (uint32_t)j * (uint32_t)e.rows * 128u);
            const uint64_t bdesc = kmajor_sw128_desc(e.xmap >= 0 ? stage_base + kStageW + (uint32_t)j * (kPredRows * 128)
                                                                 : smem_addr(xs) + (uint32_t)(kb + j) * (kPredRows * 128));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              mma_bf16(tmem_acc, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb > 0 || j > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit(smem_addr(&ctl.empty[w.stage]));  // the stage is free once these MMAs have read it
          w.advance();
        }
        if (ok) mma_commit(smem_addr(&ctl.acc_full));
      }
      if (!wait_bar<false>(smem_addr(&ctl.acc_full), (uint32_t)i & 1u, ctl, a.err, kAtWeightFull)) break;
      tc_fence_after_sync();
      if (tracing) a.trace[3 * i + 1] = global_timer_ns();
      // ---- accumulator -> out[session][weight row]: a warp reads the TMEM lanes of its quadrant (warp index % 4), the two
      // warps of a quadrant eight sessions each. M = 64 keeps rows 16q .. 16q + 15 in the first 16 lanes of quadrant q.
      {
        const int quad = warp & 3, half = cw >> 2;
        float v[8];
        tmem_ld8(tmem_acc + ((uint32_t)(quad * 32) << 16) + (uint32_t)(half * 8), v);
        const int c = narrow ? quad * 16 + lane : quad * 32 + lane;
        if (!narrow || lane < 16) {
#pragma unroll
          for (int x = 0; x < 8; ++x) scratch.t.out[0][half * 8 + x][c] = v[x];
        }
        tc_fence_before_sync();
      }
      ConsumerSync::sync();
      const float(*o0)[kOutPitch] = scratch.t.out[0];

      switch (e.epi) {
        case kPeBiasNorm:
        case kPeAddNorm: {
          // this CTA's 64 columns of the residual stream; the unrounded sum goes to the exchange buffer
          const bf16* bias = (const bf16*)e.p0;
          const int col0 = rank * 64;
          for (int idx = ctid; idx < kPredRows * 64; idx += kConsumers) {
            const int n = idx >> 6, c = idx & 63;
            const float y = bf16_round(o0[n][c]);
            float v;
            if (e.epi == kPeBiasNorm) v = bias ? bf16_round(y + __bfloat162float(bias[col0 + c])) : y;
            else v = y + res[n][c];  // the norm runs over the unrounded sum (qwen3.cu:34)
            res[n][c] = bf16_round(v);
            if (n < live) a.vbuf[(int64_t)(s0 + n) * hidden + col0 + c] = v;
          }
          if (!cluster_barrier(ctl, n_bars, C, ctid, a.err)) break;
          norm_to_tile(a.vbuf, (const bf16*)e.p1, hidden, e.eps, s0, live, xs, cw, lane);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these stores are read by tcgen05.mma
          ConsumerSync::sync();
          break;
        }
        case kPeQ:
        case kPeKv: {
          // one head of 128: rows cw and cw + 8
          const bool is_q = e.epi == kPeQ, is_v = !is_q && (rank & 1);
          const int kh = rank >> 1, hk = a.cfg.kv_heads;
          bf16* kv = (bf16*)e.q0;
          float cs[2], sn[2], wl[2], wh[2];
          if (!is_v) {
            const bf16* g = (const bf16*)e.p0;
            rope_angles<128>(lane, e.pos, e.theta, cs, sn);
#pragma unroll
            for (int x = 0; x < 2; ++x) wl[x] = __bfloat162float(g[lane * 2 + x]), wh[x] = __bfloat162float(g[64 + lane * 2 + x]);
          }
          for (int n = cw; n < live; n += 8) {
            if (is_v) {
              bf16* dst = kv + kv_offset<128>(s0 + n, hk, kh, 1, e.pos) + lane * 4;
              uint2 u;
              *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(o0[n][lane * 4], o0[n][lane * 4 + 1]);
              *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(o0[n][lane * 4 + 2], o0[n][lane * 4 + 3]);
              *reinterpret_cast<uint2*>(dst) = u;
              continue;
            }
            float lo[2], hi[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) lo[x] = bf16_round(o0[n][lane * 2 + x]), hi[x] = bf16_round(o0[n][64 + lane * 2 + x]);
            rope_head<128>(lo, hi, wl, wh, cs, sn, e.eps);
            if (is_q) {
#pragma unroll
              for (int x = 0; x < 2; ++x) scratch.t.q[n][lane * 2 + x] = lo[x], scratch.t.q[n][64 + lane * 2 + x] = hi[x];
            } else {
              bf16* dst = kv + kv_offset<128>(s0 + n, hk, kh, 0, e.pos);
              *reinterpret_cast<__nv_bfloat162*>(dst + lane * 2) = __floats2bfloat162_rn(lo[0], lo[1]);
              *reinterpret_cast<__nv_bfloat162*>(dst + 64 + lane * 2) = __floats2bfloat162_rn(hi[0], hi[1]);
            }
          }
          if (is_q) {
            ConsumerSync::sync();  // the epilogue tile is free for the next box; q stays
            break;
          }
          if (!cluster_barrier(ctl, n_bars, C, ctid, a.err)) break;  // the partner's half of this position's K/V
          // attention of query head `rank` over positions 0 .. pos of the frame (one page): f32 scores, __expf,
          // one softmax over at most 16 keys (qwen3.cu:123-207 with a single key tile), bf16 out
          {
            const int len = e.pos + 1;
            const float scale = rsqrtf(128.f);
            bf16* out = (bf16*)e.q1;
            for (int n = cw; n < live; n += 8) {
              const bf16* kpage = kv + kv_offset<128>(s0 + n, hk, kh, 0, 0);
              const bf16* vpage = kpage + 16 * 128;
              // every load of the page is issued before any is used: lane j holds key row j, and every lane its four
              // output dims of all 16 value rows (rows past the frame's length are never read)
              uint4 kraw[16];
              uint2 vraw[16];
#pragma unroll
              for (int c = 0; c < 16; ++c)
                kraw[c] = lane < len ? __ldcg(reinterpret_cast<const uint4*>(kpage + lane * 128 + c * 8)) : make_uint4(0, 0, 0, 0);
#pragma unroll
              for (int j = 0; j < 16; ++j)
                vraw[j] = j < len ? __ldcg(reinterpret_cast<const uint2*>(vpage + j * 128 + lane * 4)) : make_uint2(0, 0);
              float dot = 0.f;
#pragma unroll
              for (int c = 0; c < 16; ++c) {
                float kf[8];
                unpack8(*reinterpret_cast<const Pack8*>(&kraw[c]), kf);
#pragma unroll
                for (int x = 0; x < 8; ++x) dot = fmaf(scratch.t.q[n][c * 8 + x], kf[x], dot);
              }
              const float s = lane < len ? dot * scale : -INFINITY;
              const float mx = warp_fmax(s);
              const float p = lane < len ? __expf(s - mx) : 0.f;
              const float l = warp_add(p);
              float acc4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);  // 0 past the frame's length
                const float2 v0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vraw[j].x));
                const float2 v1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vraw[j].y));
                acc4[0] = fmaf(pj, v0.x, acc4[0]), acc4[1] = fmaf(pj, v0.y, acc4[1]);
                acc4[2] = fmaf(pj, v1.x, acc4[2]), acc4[3] = fmaf(pj, v1.y, acc4[3]);
              }
              uint2 u;
              *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(acc4[0] / l, acc4[1] / l);
              *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(acc4[2] / l, acc4[3] / l);
              *reinterpret_cast<uint2*>(out + (int64_t)(s0 + n) * (a.cfg.q_heads * 128) + rank * 128 + lane * 4) = u;
            }
          }
          cluster_barrier(ctl, n_bars, C, ctid, a.err);
          break;
        }
        case kPeSwiglu: {
          // the box holds whole granules: gr gate rows followed by the gr matching up rows
          const int gr = a.cfg.granule, inter = a.cfg.inter, box_row = weight_row(e, rank);
          bf16* act = (bf16*)e.q0;
          for (int idx = ctid; idx < kPredRows * 64; idx += kConsumers) {
            const int n = idx >> 6, cc = idx & 63;
            const int cg = (cc / gr) * 2 * gr + cc % gr;
            const int ch = ((box_row + cg) / (2 * gr)) * gr + cc % gr;
            if (n < live && ch < inter) {
              const float g = bf16_round(o0[n][cg]), u = bf16_round(o0[n][cg + gr]);
              act[(int64_t)(s0 + n) * inter + ch] = __float2bfloat16(bf16_round(g / (1.f + __expf(-g))) * u);
            }
          }
          if (e.last) cluster_barrier(ctl, n_bars, C, ctid, a.err);
          else ConsumerSync::sync();
          break;
        }
        case kPeHead: {
          bf16* logits = (bf16*)e.q0;
          const int vocab = a.cfg.vocab, col = e.col0 + rank * e.cta_stride;
          for (int idx = ctid; idx < kPredRows * e.rows; idx += kConsumers) {
            const int n = idx / e.rows, c = idx % e.rows;
            if (n < live && col + c < vocab) {
              const float y = o0[n][c];
              logits[(int64_t)(s0 + n) * vocab + col + c] = __float2bfloat16(y);
            }
          }
          if (!e.last) {
            ConsumerSync::sync();
            break;
          }
          if (!cluster_barrier(ctl, n_bars, C, ctid, a.err)) break;
          // the draw of row n by CTA n % C (talker.cu:171-293 through sampler.cuh), then the next sub-step's input row
          sampler::Params prm;
          prm.vocab = vocab;
          prm.temperature = a.cfg.temperature;
          prm.top_p = a.cfg.top_p;
          prm.penalty = 1.f;
          prm.top_k = a.cfg.top_k;
          prm.suppress_lo = 0, prm.suppress_hi = 0, prm.exempt = -1, prm.min_frames = 0, prm.penalize = 0;
          prm.group = e.group;
          prm.philox = a.cfg.philox;
          prm.seen_words = a.io.seen_words;
          for (int n = rank; n < live; n += C) {
            const int s = s0 + n;
            int32_t* slot = reinterpret_cast<int32_t*>(static_cast<char*>(a.io.state) + (int64_t)a.io.lines[s] * a.io.stride);
            const int forced = a.io.force[s * 16 + prm.group], frame = a.io.frames[s];
            const float uniform = a.io.uniforms[s * 16 + prm.group];
            float mine[DrawTeam::PER];
            if (ctid * DrawTeam::PER < vocab) {
              const uint4* src = reinterpret_cast<const uint4*>(logits + (int64_t)s * vocab + ctid * DrawTeam::PER);
#pragma unroll
              for (int j = 0; j < DrawTeam::PER / 8; ++j) {
                const uint4 raw = __ldcg(src + j);
                unpack8(*reinterpret_cast<const Pack8*>(&raw), mine + 8 * j);
              }
            } else {
#pragma unroll
              for (int j = 0; j < DrawTeam::PER; ++j) mine[j] = 0.f;
            }
            const int token = DrawTeam::sample_row([&](int, int j) { return mine[j]; }, prm, frame, uniform, forced, slot, 0u,
                                                   a.io.codes + s * 16 + prm.group, ctid, scratch.draw);
            if (e.next_dim > 0) {
              const bf16* table = (const bf16*)e.p0;
              bf16* dst = (bf16*)e.q1 + (int64_t)s * a.cfg.next_stride;
              for (int k = ctid * 8; k < e.next_dim; k += kConsumers * 8)
                *reinterpret_cast<uint4*>(dst + k) = *reinterpret_cast<const uint4*>(table + (int64_t)token * e.next_dim + k);
            }
            ConsumerSync::sync();
          }
          cluster_barrier(ctl, n_bars, C, ctid, a.err);
          break;
        }
        default: break;
      }
      if (tracing) a.trace[3 * i + 2] = global_timer_ns();
    }
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kFirstConsumerWarp) tmem_dealloc(tmem_acc, kTmemCols);
  hw_cluster_sync();  // no CTA leaves while a peer may still arrive on its barriers
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

size_t pred_smem_bytes(int hidden) {
  return 1024 + (size_t)kStages * kStageBytes + (size_t)(hidden / 64) * kPredRows * 128 + sizeof(Scratch) +
         kPredRows * 64 * sizeof(float) + sizeof(Control);
}

}  // namespace

int pred_add_map(PredProgram* prog, const bf16* base, int64_t rows, int K, int64_t row_stride, int box_rows, int kbs) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return -1;
  const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)row_stride * sizeof(bf16), (cuuint64_t)64 * sizeof(bf16)};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, (cuuint32_t)kbs};
  const cuuint32_t elem[3] = {1, 1, 1};
  CUtensorMap map;
  const CUresult r = reinterpret_cast<EncodeTiledFn>(fn)(
      &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<bf16*>(base), dims, strides, box, elem,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -1;
  prog->maps.push_back(map);
  return (int)prog->maps.size() - 1;
}

int pred_configure(int C) {
  if (C != 2 && C != 4 && C != 8 && C != 16) return 0;
  const size_t smem = pred_smem_bytes(64 * C);
  if (smem > 227 * 1024) return 0;
  if (cudaFuncSetAttribute(pred_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return 0;
  if (C > 8 && cudaFuncSetAttribute(pred_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(C);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = C, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, pred_kernel, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return clusters;
}

int pred_upload(PredProgram* prog) {
  pred_free(prog);
  if (cudaMalloc((void**)&prog->d_entries, prog->entries.size() * sizeof(PredEntry)) != cudaSuccess) return -1;
  if (cudaMalloc((void**)&prog->d_maps, prog->maps.size() * sizeof(CUtensorMap)) != cudaSuccess) return -1;
  if (cudaMemcpy(prog->d_entries, prog->entries.data(), prog->entries.size() * sizeof(PredEntry), cudaMemcpyHostToDevice) !=
      cudaSuccess)
    return -1;
  if (cudaMemcpy(prog->d_maps, prog->maps.data(), prog->maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice) != cudaSuccess)
    return -1;
  return 0;
}

void pred_free(PredProgram* prog) {
  if (prog->d_entries) cudaFree(prog->d_entries);
  if (prog->d_maps) cudaFree(prog->d_maps);
  prog->d_entries = nullptr;
  prog->d_maps = nullptr;
}

cudaError_t pred_launch(const PredProgram& prog, const TickIo& io, float* vbuf, uint32_t* err, cudaStream_t stream,
                        unsigned long long* trace) {
  KernelArgs a;
  a.entries = prog.d_entries;
  a.n_entries = (int)prog.entries.size();
  a.maps = prog.d_maps;
  a.cfg = prog.cfg;
  a.rows = prog.rows;
  a.per_cluster = prog.per_cluster;
  a.io = io;
  a.vbuf = vbuf;
  a.err = err;
  a.trace = trace;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(prog.clusters * prog.cfg.C);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pred_smem_bytes(prog.cfg.hidden);
  cfg.stream = stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = prog.cfg.C, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, pred_kernel, a);
}

}  // namespace omni
