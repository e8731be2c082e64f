// The persistent tick kernel (see tick.h): 12 warps per CTA, one CTA per SM, cooperative launch.
//   warp 0 / lane 0   weight producer: TMA loads of W tiles, runs ahead of the grid barriers
//   warp 1 / lane 0   activation producer: TMA loads of X tiles, gated by the barrier before its phase
//   warp 2 / lane 0   issues tcgen05.mma into one of two TMEM accumulators; whole warp owns the TMEM allocation
//   warp 3            idle
//   warps 4..11       workers: GEMM epilogues (TMEM -> partial tiles / SwiGLU) and every non-GEMM phase
// Every wait (mbarrier, grid barrier, phase release) is bounded; on a timeout the device error word is
// raised, every CTA sees it within its next wait and the kernel unwinds.
#include "tick.h"

#include <algorithm>
#include <cstdio>

#include "attend.cuh"
#include "gemm.h"
#include "sampler.cuh"
#include "sm100.cuh"

namespace omni {
namespace {

constexpr int kThreads = 384;
constexpr int kWorkerThreads = 256;
constexpr int kFirstWorkerWarp = 4;
constexpr int kMaxStages = 8;
constexpr int kTileW = 128, kTileK = 64;
constexpr int kWBytes = kTileW * kTileK * 2;
constexpr int kMaxPerThread = 32;  // row-wise phases: hidden <= 32 * 128

struct GroupBar {  // named barrier of one 128-thread worker group
  int id;
  __device__ __forceinline__ void sync() const { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
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
  AttnShared<128, 4> attn[2];
  sampler::Shared sample;
};

struct KernelArgs {
  const Phase* phases;
  int n_phases;
  const CUtensorMap* maps;
  float* partials;
  uint32_t* barrier;
  uint32_t* err;
  int n_stages, stage_bytes, acc_stride;  // acc_stride: TMEM columns per accumulator
  int n_acc;                              // independent accumulators per buffer (K steps rotate over them)
  int tmem_cols;
  unsigned long long* trace;  // optional: CTA 0 stamps the global timer after every phase's barrier
  TickIo io;
};

__device__ __forceinline__ int first_item(const Phase& ph) {
  const int g = gridDim.x;
  return (int)((blockIdx.x + g - ph.cta_offset % g) % g);
}

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All CTAs arrive, then wait until `target` arrivals have been counted. Returns false on timeout / error.
__device__ bool grid_barrier(uint32_t* counter, uint32_t target, uint32_t* err) {
  __threadfence();
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
  const uint64_t start = sm100::global_timer_ns();
  for (uint32_t spins = 0;; ++spins) {
    if (ld_acquire(counter) >= target) {
      __threadfence();
      return true;
    }
    if ((spins & 127u) == 127u) {
      if (*reinterpret_cast<volatile uint32_t*>(err) != 0) return false;
      if (sm100::global_timer_ns() - start > sm100::kWaitLimitNs) {
        raise(err, kErrBarrierTimeout);
        return false;
      }
    }
  }
}

// Sums of K-split partials are taken in split order, starting from zero, exactly as the per-op GEMM's last CTA does.
// N columns of one row at once: the split loop is outermost so the N loads of a split are
// independent and in flight together (one L2 round trip per split instead of one per element).
template <int N>
__device__ __forceinline__ void reduce_partial_n(const float* __restrict__ partials, int splits, int tiles, int bn,
                                                 int m, const int (&cols)[N], float (&acc)[N]) {
  const float* p[N];
#pragma unroll
  for (int j = 0; j < N; ++j) {
    p[j] = partials + ((size_t)(cols[j] >> 7) * bn + m) * kTileW + (cols[j] & 127);
    acc[j] = 0.f;
  }
  const size_t stride = (size_t)tiles * bn * kTileW;
  for (int s = 0; s < splits; ++s) {
    float f[N];
#pragma unroll
    for (int j = 0; j < N; ++j) f[j] = __ldcg(p[j] + s * stride);
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] += f[j];
  }
}

// Row r, columns t*128 + gtid for t < nt (nt <= kMaxPerThread): the row-wise phases' access pattern.
__device__ __forceinline__ void reduce_row(const float* __restrict__ partials, int splits, int tiles, int bn, int m,
                                           int gtid, int nt, float (&acc)[kMaxPerThread]) {
  const float* p = partials + (size_t)m * kTileW + gtid;
  const size_t tile_stride = (size_t)bn * kTileW, stride = (size_t)tiles * bn * kTileW;
#pragma unroll
  for (int t = 0; t < kMaxPerThread; ++t) acc[t] = 0.f;
  for (int s = 0; s < splits; ++s) {
    float f[kMaxPerThread];
#pragma unroll
    for (int t = 0; t < kMaxPerThread; ++t)
      if (t < nt) f[t] = __ldcg(p + s * stride + t * tile_stride);
#pragma unroll
    for (int t = 0; t < kMaxPerThread; ++t)
      if (t < nt) acc[t] += f[t];
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

// ---- row-wise phases: one 128-thread group per row, thread j owns columns t*128 + j -------------------------

__device__ void phase_embed_norm(const Phase& ph, const TickIo& io, int group, int n_groups, int gtid, float* red,
                                 const GroupBar& bar, uint32_t* err) {
  const int dim = ph.N, nt = dim / kTileW;
  const bf16 *pad = (const bf16*)ph.src0, *codec_emb = (const bf16*)ph.src1, *p_emb = (const bf16*)ph.src2,
             *gain = (const bf16*)ph.src3;
  bf16 *res = (bf16*)ph.dst0, *x = (bf16*)ph.dst1;
  for (int row = group; row < ph.rows; row += n_groups) {
    const int32_t* codes =
        reinterpret_cast<const int32_t*>(static_cast<const char*>(io.state) + (int64_t)io.lines[row] * io.stride);
    int c[16];
#pragma unroll
    for (int g = 0; g < 16; ++g) {
      c[g] = g < ph.i2 ? codes[g] : 0;
      const int limit = g == 0 ? ph.i0 : ph.i1;
      if (c[g] < 0 || c[g] >= limit) {
        if (gtid == 0) raise(err, kErrBadIndex);
        c[g] = 0;
      }
    }
    float v[kMaxPerThread], ss = 0.f;
#pragma unroll
    for (int t = 0; t < kMaxPerThread; ++t) {
      if (t < nt) {
        const int col = t * kTileW + gtid;
        float acc = __bfloat162float(pad[col]);
        acc += __bfloat162float(codec_emb[(int64_t)c[0] * dim + col]);
#pragma unroll
        for (int g = 1; g < 16; ++g)
          if (g < ph.i2) acc += __bfloat162float(p_emb[((int64_t)(g - 1) * ph.i1 + c[g]) * dim + col]);
        v[t] = bf16_round(acc);
        ss += v[t] * v[t];
      }
    }
    const float r = rsqrtf(group_sum(ss, gtid, red, bar) / dim + ph.f0);
#pragma unroll
    for (int t = 0; t < kMaxPerThread; ++t) {
      if (t < nt) {
        const int col = t * kTileW + gtid;
        res[(int64_t)row * dim + col] = __float2bfloat16(v[t]);
        x[(int64_t)row * dim + col] = __float2bfloat16(v[t] * r * __bfloat162float(gain[col]));
      }
    }
  }
}

__device__ void phase_reduce_norm(const Phase& ph, const float* partials, int group, int n_groups, int gtid, float* red,
                                  const GroupBar& bar) {
  const int dim = ph.N, nt = dim / kTileW;
  const bf16 *bias = (const bf16*)ph.src0, *gain = (const bf16*)ph.src3;
  bf16 *res = (bf16*)ph.dst0, *x = (bf16*)ph.dst1;
  for (int row = group; row < ph.rows; row += n_groups) {
    float v[kMaxPerThread], ss = 0.f;
    reduce_row(partials, ph.splits, ph.tiles, ph.bn, row, gtid, nt, v);
#pragma unroll
    for (int t = 0; t < kMaxPerThread; ++t) {
      if (t < nt) {
        const int col = t * kTileW + gtid;
        float a = bf16_round(v[t]);
        if (bias) a = bf16_round(a + __bfloat162float(bias[col]));
        v[t] = a;
        ss += a * a;
      }
    }
    const float r = rsqrtf(group_sum(ss, gtid, red, bar) / dim + ph.f0);
#pragma unroll
    for (int t = 0; t < kMaxPerThread; ++t) {
      if (t < nt) {
        const int col = t * kTileW + gtid;
        res[(int64_t)row * dim + col] = __float2bfloat16(v[t]);
        x[(int64_t)row * dim + col] = __float2bfloat16(v[t] * r * __bfloat162float(gain[col]));
      }
    }
  }
}

__device__ void phase_add_norm(const Phase& ph, const float* partials, int group, int n_groups, int gtid, float* red,
                               const GroupBar& bar) {
  const int dim = ph.N, nt = dim / kTileW, every = ph.i0, which = ph.i1;
  const bf16* gain = (const bf16*)ph.src3;
  bf16 *res = (bf16*)ph.dst0, *out = (bf16*)ph.dst1;
  for (int row = group; row < ph.rows; row += n_groups) {
    float v[kMaxPerThread], ss = 0.f;
    reduce_row(partials, ph.splits, ph.tiles, ph.bn, row, gtid, nt, v);
#pragma unroll
    for (int t = 0; t < kMaxPerThread; ++t) {
      if (t < nt) {
        const int col = t * kTileW + gtid;
        v[t] = bf16_round(v[t]) + __bfloat162float(res[(int64_t)row * dim + col]);
        ss += v[t] * v[t];
      }
    }
    const float r = rsqrtf(group_sum(ss, gtid, red, bar) / dim + ph.f0);
    const bool keep = row % every == which;
#pragma unroll
    for (int t = 0; t < kMaxPerThread; ++t) {
      if (t < nt) {
        const int col = t * kTileW + gtid;
        res[(int64_t)row * dim + col] = __float2bfloat16(v[t]);
        if (keep) out[(int64_t)(row / every) * dim + col] = __float2bfloat16(v[t] * r * __bfloat162float(gain[col]));
      }
    }
  }
}

// ---- rope + KV write + attention: one group per (sequence, kv head) ---------------------------------------------

template <int D, int G>
__device__ void rope_attend_item(const Phase& ph, const TickIo& io, const float* partials, int seq, int kh, int gtid,
                                 AttnShared<128, 4>& shraw, const GroupBar& bar, uint32_t* err) {
  AttnShared<D, G>& sh = reinterpret_cast<AttnShared<D, G>&>(shraw);
  constexpr int E = D / 64;
  const int hq = ph.i0, hk = ph.i1, per = ph.i3, base = ph.i4;
  const bool paged = ph.i5 != 0;
  const bf16 *q_norm = (const bf16*)ph.src0, *k_norm = (const bf16*)ph.src1;
  bf16 *kv = (bf16*)ph.dst0, *out = (bf16*)ph.dst1;
  const int lane = gtid & 31, warp = gtid >> 5;
  const float scale = rsqrtf((float)D);
  for (int r = 0; r < per; ++r) {
    const int n = seq * per + r;
    const int pos = paged ? io.d_pos[n] : base + r;
    const int64_t slot = paged ? io.d_slot[n] : (int64_t)seq * 16 + pos;
    int64_t page = slot >> 4;
    const int tok = (int)(slot & 15);
    if (page < 0 || page >= ph.i6) {
      if (gtid == 0) raise(err, kErrBadIndex);
      page = 0;
    }
    // G query heads, the key head and the value head of this row, a warp per head
    for (int job = warp; job < G + 2; job += kAttnWarps) {
      if (job == G + 1) {  // value: plain copy
        bf16* dst = kv + kv_offset<D>(page, hk, kh, 1, tok);
        const int col0 = (hq + hk + kh) * D;
        int cols[D / 32];
        float val[D / 32];
#pragma unroll
        for (int e = 0; e < D / 32; ++e) cols[e] = col0 + lane + 32 * e;
        reduce_partial_n(partials, ph.splits, ph.tiles, ph.bn, n, cols, val);
#pragma unroll
        for (int e = 0; e < D / 32; ++e) dst[lane + 32 * e] = __float2bfloat16(val[e]);
        continue;
      }
      const bool is_q = job < G;
      const int col0 = (is_q ? kh * G + job : hq + kh) * D;
      const bf16* w = is_q ? q_norm : k_norm;
      float lo[E], hi[E], ss = 0.f;
      {
        int cols[2 * E];
        float val[2 * E];
#pragma unroll
        for (int e = 0; e < E; ++e) cols[e] = col0 + lane * E + e, cols[E + e] = col0 + D / 2 + lane * E + e;
        reduce_partial_n(partials, ph.splits, ph.tiles, ph.bn, n, cols, val);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          lo[e] = bf16_round(val[e]);
          hi[e] = bf16_round(val[E + e]);
          ss += lo[e] * lo[e] + hi[e] * hi[e];
        }
      }
      const float rn = rsqrtf(warp_add(ss) / D + ph.f0);
      bf16* kdst = kv + kv_offset<D>(page, hk, kh, 0, tok);
#pragma unroll
      for (int e = 0; e < E; ++e) {
        const int i = lane * E + e;
        const float a = bf16_round(lo[e] * rn) * __bfloat162float(w[i]);
        const float b = bf16_round(hi[e] * rn) * __bfloat162float(w[D / 2 + i]);
        const float inv_freq = 1.f / powf(ph.f1, (float)(2 * i) / D);
        float sn, cs;
        sincosf((float)pos * inv_freq, &sn, &cs);
        const bf16 o_lo = __float2bfloat16(a * cs - b * sn), o_hi = __float2bfloat16(b * cs + a * sn);
        if (is_q) {
          sh.qs[job][i] = __bfloat162float(o_lo);
          sh.qs[job][D / 2 + i] = __bfloat162float(o_hi);
        } else {
          kdst[i] = o_lo;
          kdst[D / 2 + i] = o_hi;
        }
      }
    }
    __threadfence_block();
    bar.sync();
    attend_pages<D, G>(sh, kv, paged ? io.pages + io.indptr[n] : nullptr, seq, pos + 1, hk, kh, scale,
                       out + ((int64_t)n * hq + kh * G) * D, gtid, bar);
  }
}

__device__ void phase_rope_attn(const Phase& ph, const TickIo& io, const float* partials, int group, int n_groups,
                                int gtid, AttnShared<128, 4>& sh, const GroupBar& bar, uint32_t* err) {
  const int hq = ph.i0, hk = ph.i1, D = ph.i2, per = ph.i3, G = hq / hk;
  const int seqs = ph.rows / per, items = seqs * hk;
  for (int it = group; it < items; it += n_groups) {
    const int seq = it / hk, kh = it % hk;
    if (D == 128) {
      if (G == 1) rope_attend_item<128, 1>(ph, io, partials, seq, kh, gtid, sh, bar, err);
      else if (G == 2) rope_attend_item<128, 2>(ph, io, partials, seq, kh, gtid, sh, bar, err);
      else rope_attend_item<128, 4>(ph, io, partials, seq, kh, gtid, sh, bar, err);
    } else {
      if (G == 1) rope_attend_item<64, 1>(ph, io, partials, seq, kh, gtid, sh, bar, err);
      else if (G == 2) rope_attend_item<64, 2>(ph, io, partials, seq, kh, gtid, sh, bar, err);
      else rope_attend_item<64, 4>(ph, io, partials, seq, kh, gtid, sh, bar, err);
    }
  }
}

// ---- head reduce + draw + next predictor input: one row per CTA (all 256 workers) -----------------------------

__device__ void phase_sample(const Phase& ph, const TickIo& io, const float* partials, int wtid, sampler::Shared& sh,
                             uint32_t* err) {
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
    // this thread's PER consecutive logits: reduce the head's split-K partials, round, publish
    float mine[Team::PER];
    {
      int cols[Team::PER];
#pragma unroll
      for (int j = 0; j < Team::PER; ++j) cols[j] = min(wtid * Team::PER + j, prm.vocab - 1);
      reduce_partial_n(partials, ph.splits, ph.tiles, ph.bn, row, cols, mine);
#pragma unroll
      for (int j = 0; j < Team::PER; ++j) {
        const bf16 b = __float2bfloat16(mine[j]);
        mine[j] = __bfloat162float(b);
        if (wtid * Team::PER + j < prm.vocab) logits_out[(int64_t)row * ph.i0 + wtid * Team::PER + j] = b;
      }
    }
    const int forced = io.force[row * 16 + prm.group];
    const int token = Team::sample_row([&](int, int j) { return mine[j]; }, prm, io.frames[row],
                                       io.uniforms[row * 16 + prm.group], forced, slot,
                                       io.codes + row * 16 + prm.group, wtid, sh);
    // the next predictor pass reads the embedding of the code just drawn
    const int dim = ph.i9;
    if (ph.i8 == kNextHiddenAndCode) {
      const bf16 *table = (const bf16*)ph.src0, *hidden = (const bf16*)ph.src1;
      bf16* dst = (bf16*)ph.dst1;
      for (int i = wtid * 8; i < dim; i += kWorkerThreads * 8) {
        *reinterpret_cast<Pack8*>(dst + ((int64_t)2 * row) * dim + i) =
            *reinterpret_cast<const Pack8*>(hidden + (int64_t)row * dim + i);
        *reinterpret_cast<Pack8*>(dst + ((int64_t)2 * row + 1) * dim + i) =
            *reinterpret_cast<const Pack8*>(table + (int64_t)token * dim + i);
      }
    } else if (ph.i8 == kNextCode) {
      const bf16* table = (const bf16*)ph.src0;
      bf16* dst = (bf16*)ph.dst1;
      for (int i = wtid * 8; i < dim; i += kWorkerThreads * 8)
        *reinterpret_cast<Pack8*>(dst + (int64_t)row * dim + i) =
            *reinterpret_cast<const Pack8*>(table + (int64_t)token * dim + i);
    }
    WorkerSync::sync();
  }
  (void)err;
}

// ---- GEMM epilogue: this worker warp's TMEM quadrant, every other 16-column chunk ---------------------------------

// Reads 16 columns of this lane from every accumulator of the buffer and sums them in accumulator order.
__device__ __forceinline__ void load_acc16(uint32_t addr, int n_acc, int acc_stride, float* v) {
  sm100::tmem_ld16(addr, v);
  for (int a = 1; a < n_acc; ++a) {
    float w[16];
    sm100::tmem_ld16(addr + (uint32_t)(a * acc_stride), w);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] += w[j];
  }
}

__device__ void gemm_epilogue(const Phase& ph, float* partials, int tile, int split, uint32_t tmem_acc, int n_acc,
                              int acc_stride, int wwarp, int lane) {
  const int quad = wwarp & 3, half = wwarp >> 2;
  const uint32_t lane_addr = tmem_acc + ((uint32_t)(quad * 32) << 16);
  if (ph.mode == kGemmPartials) {
    float* tile_base = partials + ((size_t)split * ph.tiles + tile) * ph.bn * kTileW + quad * 32 + lane;
    for (int c0 = half * 16; c0 < ph.bn; c0 += 32) {
      float v[16];
      load_acc16(lane_addr + c0, n_acc, acc_stride, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) tile_base[(size_t)(c0 + j) * kTileW] = v[j];
    }
  } else {
    // SwiGLU: the tile's rows alternate 16 gate channels / 16 up channels, so a lane's partner is lane ^ 16
    bf16* act = (bf16*)ph.dst0;
    const int inter = ph.i0;
    const int ch = tile * 64 + quad * 16 + (lane & 15);
    for (int c0 = half * 16; c0 < ph.bn; c0 += 32) {
      float v[16];
      load_acc16(lane_addr + c0, n_acc, acc_stride, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float mine = bf16_round(v[j]);
        const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
        const int m = c0 + j;
        if (lane < 16 && m < ph.rows && ch < inter) {
          const float silu = bf16_round(mine / (1.f + __expf(-mine)));
          act[(int64_t)m * inter + ch] = __float2bfloat16(silu * other);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) tick_kernel(const __grid_constant__ KernelArgs a) {
  using namespace sm100;
  extern __shared__ unsigned char tick_smem_raw[];
  const uint32_t raw = smem_addr(tick_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = tick_smem_raw + (base - raw);
  Control& ctl = *reinterpret_cast<Control*>(base_ptr + (size_t)a.n_stages * a.stage_bytes);
  WorkerScratch& scratch =
      *reinterpret_cast<WorkerScratch*>(base_ptr + (size_t)a.n_stages * a.stage_bytes + ((sizeof(Control) + 127) & ~127));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;

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
  if (warp == 2) tmem_alloc(smem_addr(&ctl.tmem_base), (uint32_t)a.tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl.tmem_base;
  auto stage_addr = [&](int s) { return base + (uint32_t)(s * a.stage_bytes); };

  if (warp == 0) {
    if (lane == 0) {  // ---- weight producer ----
      int stage = 0;
      uint32_t par = 0;
      for (int p = 0; p < a.n_phases && !ctl.abort; ++p) {
        const Phase& ph = a.phases[p];
        if (ph.type != kPhGemm) continue;
        const int items = ph.tiles * ph.splits, nkb = ph.K / kTileK;
        const CUtensorMap* map = a.maps + ph.wmap;
        for (int it = first_item(ph); it < items && !ctl.abort; it += G) {
          const int tile = it % ph.tiles, split = it / ph.tiles;
          const int kb0 = (int)((int64_t)nkb * split / ph.splits), kb1 = (int)((int64_t)nkb * (split + 1) / ph.splits);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(smem_addr(&ctl.empty[stage]), par ^ 1u, a.err)) {
              ctl.abort = 1;
              break;
            }
            const uint32_t bar = smem_addr(&ctl.full_w[stage]);
            mbar_expect_tx(bar, kWBytes);
            tma_load_2d(stage_addr(stage), map, bar, kb * kTileK, tile * kTileW, kEvictFirst);
            if (++stage == a.n_stages) stage = 0, par ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ---- activation producer ----
      int stage = 0;
      uint32_t par = 0;
      for (int p = 0; p < a.n_phases && !ctl.abort; ++p) {
        const Phase& ph = a.phases[p];
        if (ph.type != kPhGemm) continue;
        const int items = ph.tiles * ph.splits, nkb = ph.K / kTileK;
        if (first_item(ph) >= items) continue;
        // the rows this phase multiplies were written by earlier phases: wait until those are complete everywhere
        const uint64_t start = global_timer_ns();
        while (ctl.released < p && !ctl.abort) {
          __nanosleep(40);
          if (global_timer_ns() - start > kWaitLimitNs) {
            raise(a.err, kErrBarrierTimeout);
            ctl.abort = 1;
          }
        }
        asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy writes of other CTAs -> async-proxy reads
        const CUtensorMap* map = a.maps + ph.xmap;
        const uint32_t xbytes = (uint32_t)ph.bn * kTileK * 2;
        for (int it = first_item(ph); it < items && !ctl.abort; it += G) {
          const int split = it / ph.tiles;
          const int kb0 = (int)((int64_t)nkb * split / ph.splits), kb1 = (int)((int64_t)nkb * (split + 1) / ph.splits);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(smem_addr(&ctl.empty[stage]), par ^ 1u, a.err)) {
              ctl.abort = 1;
              break;
            }
            const uint32_t bar = smem_addr(&ctl.full_x[stage]);
            mbar_expect_tx(bar, xbytes);
            tma_load_2d(stage_addr(stage) + kWBytes, map, bar, kb * kTileK, 0, kEvictLast);
            if (++stage == a.n_stages) stage = 0, par ^= 1u;
          }
        }
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {  // ---- MMA issuer ----
      int stage = 0, buf = 0;
      uint32_t par = 0, empty_par[2] = {0, 0};
      for (int p = 0; p < a.n_phases && !ctl.abort; ++p) {
        const Phase& ph = a.phases[p];
        if (ph.type != kPhGemm) continue;
        const int items = ph.tiles * ph.splits, nkb = ph.K / kTileK;
        const uint32_t idesc = idesc_bf16_f32(kTileW, ph.bn);
        for (int it = first_item(ph); it < items && !ctl.abort; it += G) {
          const int split = it / ph.tiles;
          const int kb0 = (int)((int64_t)nkb * split / ph.splits), kb1 = (int)((int64_t)nkb * (split + 1) / ph.splits);
          if (!mbar_wait(smem_addr(&ctl.acc_empty[buf]), empty_par[buf] ^ 1u, a.err)) {
            ctl.abort = 1;
            break;
          }
          empty_par[buf] ^= 1u;
          tc_fence_after_sync();
          const uint32_t tmem_d = tmem_base + (uint32_t)(buf * a.n_acc * a.acc_stride);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(smem_addr(&ctl.full_w[stage]), par, a.err) ||
                !mbar_wait(smem_addr(&ctl.full_x[stage]), par, a.err)) {
              ctl.abort = 1;
              break;
            }
            tc_fence_after_sync();
            const uint64_t adesc = kmajor_sw128_desc(stage_addr(stage)),
                           bdesc = kmajor_sw128_desc(stage_addr(stage) + kWBytes);
            // consecutive MMAs into one accumulator serialise on its latency: rotate the K steps over n_acc of them
#pragma unroll
            for (int k = 0; k < kTileK / 16; ++k)
              mma_bf16(tmem_d + (uint32_t)((k % a.n_acc) * a.acc_stride), adesc + (uint64_t)(k * 2),
                       bdesc + (uint64_t)(k * 2), idesc, (kb > kb0 || k >= a.n_acc) ? 1u : 0u);
            mma_commit(smem_addr(&ctl.empty[stage]));
            if (++stage == a.n_stages) stage = 0, par ^= 1u;
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
    const int grp = wtid >> 7, gtid = wtid & 127;
    const GroupBar gbar{2 + grp};
    const int group = blockIdx.x * 2 + grp, n_groups = G * 2;
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
          for (int it = first_item(ph); it < items; it += G) {
            const bool ok = mbar_wait(smem_addr(&ctl.acc_full[buf]), full_par[buf], a.err);
            if (!ok) ctl.abort = 1;
            full_par[buf] ^= 1u;
            tc_fence_after_sync();
            if (ok)
              gemm_epilogue(ph, a.partials, it % ph.tiles, it / ph.tiles,
                            tmem_base + (uint32_t)(buf * a.n_acc * a.acc_stride), a.n_acc, a.acc_stride, wwarp, lane);
            tc_fence_before_sync();
            WorkerSync::sync();
            if (wtid == 0) mbar_arrive(smem_addr(&ctl.acc_empty[buf]));
            buf ^= 1;
            if (ctl.abort) break;
          }
          break;
        }
        case kPhEmbedNorm: phase_embed_norm(ph, a.io, group, n_groups, gtid, ctl.red[grp], gbar, a.err); break;
        case kPhReduceNorm: phase_reduce_norm(ph, a.partials, group, n_groups, gtid, ctl.red[grp], gbar); break;
        case kPhAddNorm: phase_add_norm(ph, a.partials, group, n_groups, gtid, ctl.red[grp], gbar); break;
        case kPhRopeAttn:
          phase_rope_attn(ph, a.io, a.partials, group, n_groups, gtid, scratch.attn[grp], gbar, a.err);
          break;
        case kPhSample: phase_sample(ph, a.io, a.partials, wtid, scratch.sample, a.err); break;
        default: break;
      }
      // end of phase: the team barrier orders every worker's writes before thread 0's gpu-scope fence and arrival
      // (fences are cumulative), then everyone waits for thread 0 to see all CTAs arrive
      WorkerSync::sync();
      if (wtid == 0) {
        if (!ctl.abort && !grid_barrier(a.barrier, (uint32_t)(p + 1) * (uint32_t)G, a.err)) ctl.abort = 1;
        ctl.released = p + 1;
        if (a.trace && blockIdx.x == 0) a.trace[p] = global_timer_ns();
      }
      WorkerSync::sync();
    }
  }
  __syncwarp();
  if (ctl.abort) __nanosleep(20000);  // let copies still in flight land before the shared memory is released
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem_base, (uint32_t)a.tmem_cols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

size_t tick_smem_bytes(int n_stages, int stage_bytes) {
  return 1024 + (size_t)n_stages * stage_bytes + ((sizeof(Control) + 127) & ~127) + sizeof(WorkerScratch);
}

void stage_plan(int max_bn, int* n_stages, int* stage_bytes) {
  *stage_bytes = kWBytes + max_bn * kTileK * 2;
  *n_stages = std::min(kMaxStages, (188 * 1024) / *stage_bytes);
}

}  // namespace

int tick_add_map(TickProgram* prog, const bf16* base, int rows, int K, int box_rows) {
  if (tc_init() != 0) return -1;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return -1;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(bf16)};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  CUtensorMap map;
  const CUresult r = reinterpret_cast<EncodeTiledFn>(fn)(
      &map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<bf16*>(base), dims, strides, box, elem,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -1;
  prog->maps.push_back(map);
  return (int)prog->maps.size() - 1;
}

bool tick_supports(int hidden, int head_dim, int q_heads, int kv_heads, int rows_max) {
  const int g = kv_heads > 0 ? q_heads / kv_heads : 0;
  return hidden % kTileW == 0 && hidden <= kMaxPerThread * kTileW && (head_dim == 64 || head_dim == 128) &&
         (g == 1 || g == 2 || g == 4) && rows_max <= 256;
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
  int n_stages, stage_bytes;
  stage_plan(256, &n_stages, &stage_bytes);
  size_t worst = tick_smem_bytes(n_stages, stage_bytes);
  stage_plan(64, &n_stages, &stage_bytes);
  worst = std::max(worst, tick_smem_bytes(n_stages, stage_bytes));
  if (cudaFuncSetAttribute(tick_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)worst) != cudaSuccess) return 0;
  int per_sm = 0, sms = 0, coop = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tick_kernel, kThreads, worst) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device) != cudaSuccess || !coop) return 0;
  return per_sm >= 1 ? sms : 0;
}

cudaError_t tick_launch(const TickProgram& prog, const TickIo& io, float* partials, uint32_t* barrier, uint32_t* err,
                        int ctas, cudaStream_t stream, unsigned long long* trace) {
  KernelArgs a;
  a.trace = trace;
  a.phases = prog.d_phases;
  a.n_phases = (int)prog.phases.size();
  a.maps = prog.d_maps;
  a.partials = partials;
  a.barrier = barrier;
  a.err = err;
  stage_plan(prog.max_bn, &a.n_stages, &a.stage_bytes);
  a.acc_stride = prog.max_bn < 32 ? 32 : prog.max_bn;
  a.n_acc = std::max(1, std::min(4, 512 / (2 * a.acc_stride)));
  int cols = 2 * a.n_acc * a.acc_stride;
  a.tmem_cols = cols <= 32 ? 32 : cols <= 64 ? 64 : cols <= 128 ? 128 : cols <= 256 ? 256 : 512;
  a.io = io;
  cudaError_t e = cudaMemsetAsync(barrier, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return e;
  void* args[] = {&a};
  return cudaLaunchCooperativeKernel((const void*)tick_kernel, dim3(ctas), dim3(kThreads), args,
                                     tick_smem_bytes(a.n_stages, a.stage_bytes), stream);
}

}  // namespace omni
