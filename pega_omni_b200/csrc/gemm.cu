// The two GEMM paths of the token loop (see gemm.h).
#include "gemm.h"

#include <mutex>

#include <algorithm>
#include <cstdarg>
#include <cstdio>

#include "sm100.cuh"

namespace omni {

__device__ __forceinline__ bf16 finish(float acc, int n, const bf16* bias, int kind) {
  float t = bf16_round(acc);
  if (kind != kEpiNone) {
    t = bf16_round(t + __bfloat162float(bias[n]));
    if (kind == kEpiBiasSilu) t = t / (1.f + __expf(-t));
  }
  return __float2bfloat16(t);
}

// ---------------------------------------------------------------------------
// Vector GEMV: a warp owns an output column, lanes stride the weight row in
// 16-byte pieces, up to R input rows ride along in registers, the R x K input
// slab sits in shared memory. Weight bytes are read once per R rows.

constexpr int kGemvWarps = 8;

template <int R>
__global__ void __launch_bounds__(kGemvWarps * 32) gemv_kernel(const bf16* __restrict__ w, int N, int K,
                                                                const bf16* __restrict__ x, int rows,
                                                                bf16* __restrict__ y, int ldy, const bf16* bias,
                                                                int kind, int cols_per_warp) {
  extern __shared__ __align__(16) unsigned char gemv_smem[];
  bf16* xs = reinterpret_cast<bf16*>(gemv_smem);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = (blockIdx.x * kGemvWarps + warp) * cols_per_warp;
  for (int r0 = 0; r0 < rows; r0 += R) {
    __syncthreads();
    for (int i = threadIdx.x; i < R * K / 8; i += blockDim.x) {
      const int r = i / (K / 8), c = i % (K / 8) * 8;
      *reinterpret_cast<uint4*>(xs + r * K + c) =
          r0 + r < rows ? *reinterpret_cast<const uint4*>(x + (int64_t)(r0 + r) * K + c) : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    for (int j = 0; j < cols_per_warp; ++j) {
      const int n = col0 + j;
      if (n >= N) break;
      const bf16* wr = w + (int64_t)n * K;
      float acc[R];
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r] = 0.f;
#pragma unroll 4
      for (int c = lane * 8; c < K; c += 256) {
        float wv[8];
        ld8(wr + c, wv);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float xv[8];
          ld8(xs + r * K + c, xv);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[r] = fmaf(wv[e], xv[e], acc[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float s = warp_add(acc[r]);
        if (lane == 0 && r0 + r < rows) y[(int64_t)(r0 + r) * ldy + n] = finish(s, n, bias, kind);
      }
    }
  }
}

template <int R>
static cudaError_t gemv_launch_r(const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy, Epilogue epi,
                                 int sm_count, cudaStream_t stream) {
  const size_t smem = (size_t)R * K * sizeof(bf16);  // tc_configure() has raised the limit to 200 KB
  // enough warps to cover the machine a few times over, at most 4 columns per warp
  int cpw = N / (kGemvWarps * sm_count * 4);
  cpw = std::max(1, std::min(cpw, 4));
  const int blocks = (N + kGemvWarps * cpw - 1) / (kGemvWarps * cpw);
  gemv_kernel<R><<<blocks, kGemvWarps * 32, smem, stream>>>(w, N, K, x, rows, y, ldy, epi.bias, epi.kind, cpw);
  return cudaGetLastError();
}

cudaError_t gemv_launch(const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy, Epilogue epi,
                        int sm_count, cudaStream_t stream) {
  if (K % 8 != 0) return cudaErrorInvalidValue;
  // the slab must fit in shared memory: fewer rows per pass for very wide K
  int r = rows >= 8 ? 8 : rows > 2 ? 4 : rows;
  while (r > 1 && (size_t)r * K * 2 > 200 * 1024) r >>= 1;
  switch (r) {
    case 1: return gemv_launch_r<1>(w, N, K, x, rows, y, ldy, epi, sm_count, stream);
    case 2: return gemv_launch_r<2>(w, N, K, x, rows, y, ldy, epi, sm_count, stream);
    case 4: return gemv_launch_r<4>(w, N, K, x, rows, y, ldy, epi, sm_count, stream);
    default: return gemv_launch_r<8>(w, N, K, x, rows, y, ldy, epi, sm_count, stream);
  }
}

// ---------------------------------------------------------------------------
// Tensor-core tiles. One CTA = one 128-row slab of W (the MMA M dimension)
// times one tile of BN input rows (the MMA N dimension) over one K split.
//   warp 0 / lane 0: TMA producer, a ring of kStages {W tile, X tile} buffers
//   warp 1 / lane 0: issues tcgen05.mma (K = 16 per instruction, 4 per 64-wide
//                    K block), commits each stage back to the producer
//   all four warps:  epilogue, each reading its 32 TMEM lanes
// The accumulator D[128, BN] f32 lives in BN TMEM columns.
// With splits > 1 each split stores its f32 tile to scratch; the last CTA to
// arrive at the tile's counter sums the splits in index order (so the result
// does not depend on arrival order) and writes the output.

constexpr int kTileW = 128;  // weight rows per CTA
constexpr int kTileK = 64;   // K elements per stage: one 128-byte swizzle row

template <int BN>
struct TcShape {
  static constexpr int kStageBytes = kTileW * kTileK * 2 + BN * kTileK * 2;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
  // One accumulator: the pipeline is bound by its TMA copies, not by the tensor pipe, so rotating accumulators
  // buys nothing.
  static constexpr int kAccs = 1;
  static constexpr int kTmemCols = BN * kAccs < 32 ? 32 : BN * kAccs;
  static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

// The last CTA of a tile sums the splits' partial tiles ([column][128 lanes] f32 each) in split order and stages the
// finished bf16 tile. This is a chain of L2 round trips on one CTA, so each trip carries as much as the registers
// hold: PER column chunks of 16 at a time, 8 / PER splits of each (PER = 4, 2, 1 for at most 2, 4, 8+ splits).
template <int BN, int PER>
__device__ __forceinline__ void reduce_tile(const float* partial0, size_t split_stride, int splits, int tl, int n, int N,
                                            const bf16* bias, int kind, bf16* stage) {
  constexpr int SB = 8 / PER;
#pragma unroll 1
  for (int c0 = 0; c0 < BN; c0 += 16 * PER) {
    float acc[PER][16];
#pragma unroll
    for (int q = 0; q < PER; ++q)
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[q][j] = 0.f;
    for (int s0 = 0; s0 < splits; s0 += SB) {
      float f[PER][SB][16];
#pragma unroll
      for (int q = 0; q < PER; ++q)
#pragma unroll
        for (int b = 0; b < SB; ++b) {
          const bool live = s0 + b < splits && c0 + q * 16 < BN;
          const float* p = partial0 + (size_t)(s0 + b) * split_stride + (size_t)(c0 + q * 16) * kTileW + tl;
#pragma unroll
          for (int j = 0; j < 16; ++j) f[q][b][j] = live ? __ldcg(p + j * kTileW) : 0.f;
        }
#pragma unroll
      for (int q = 0; q < PER; ++q)
#pragma unroll
        for (int b = 0; b < SB; ++b)  // adding 0 for a missing split leaves the sum unchanged
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[q][j] += f[q][b][j];
    }
#pragma unroll
    for (int q = 0; q < PER; ++q)
      if (c0 + q * 16 < BN) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          stage[(c0 + q * 16 + j) * kTileW + tl] = n < N ? finish(acc[q][j], n, bias, kind) : __float2bfloat16(0.f);
      }
  }
}

template <int BN>
__global__ void __launch_bounds__(128, 1)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                   bf16* __restrict__ y, int ldy, int N, int K, int rows, int splits, int kbs,
                   float* __restrict__ partials, uint32_t* __restrict__ counters, const bf16* bias, int kind,
                   uint32_t* err) {
  using S = TcShape<BN>;
  // kbs k-blocks per ring stage and per TMA copy (rank-3 maps when kbs > 1): a stage is kbs W slices, then kbs X slices
  const int n_stages = S::kStages / kbs;
  const uint32_t stage_bytes = (uint32_t)kbs * S::kStageBytes, x_base = (uint32_t)kbs * kTileW * kTileK * 2;
  using namespace sm100;
  if (*reinterpret_cast<volatile uint32_t*>(err) != 0) return;  // an earlier kernel failed: do not wait on hardware

  extern __shared__ unsigned char tc_smem_raw[];
  const uint32_t raw = smem_addr(tc_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = tc_smem_raw + (base - raw);
  const uint32_t bars = base + S::kStages * S::kStageBytes;
  // barrier words: full[kStages], empty[kStages], acc, then the TMEM base slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (S::kStages + s); };
  const uint32_t acc_bar = bars + 8u * (2 * S::kStages);
  const uint32_t tmem_slot = acc_bar + 8u;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + S::kStages * S::kStageBytes + 8 * (2 * S::kStages) + 8);
  __shared__ int is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y, row_tile = blockIdx.z;
  const int nkb = K / kTileK;
  const int kb_begin = (int)((int64_t)nkb * split / splits), kb_end = (int)((int64_t)nkb * (split + 1) / splits);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    mbar_init_fence();
    prefetch_tensormap(&wmap);
    prefetch_tensormap(&xmap);
  }
  if (warp == 1) tmem_alloc(tmem_slot, S::kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  bool ok = true;
  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb_begin; kb < kb_end; kb += kbs) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, err)) break;
        const uint32_t a_dst = base + stage * stage_bytes, b_dst = a_dst + x_base;
        mbar_expect_tx(full_bar(stage), stage_bytes);
        if (kbs == 1) {
          tma_load_2d(a_dst, &wmap, full_bar(stage), kb * kTileK, tile * kTileW, kEvictFirst);
          tma_load_2d(b_dst, &xmap, full_bar(stage), kb * kTileK, row_tile * BN, kEvictLast);
        } else {
          tma_load_3d(a_dst, &wmap, full_bar(stage), 0, tile * kTileW, kb, kEvictFirst);
          tma_load_3d(b_dst, &xmap, full_bar(stage), 0, row_tile * BN, kb, kEvictLast);
        }
        if (++stage == n_stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16_f32(kTileW, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int kb = kb_begin; kb < kb_end && alive; kb += kbs) {
        alive = mbar_wait(full_bar(stage), phase, err);
        if (!alive) break;
        tc_fence_after_sync();
        const uint32_t a_src = base + stage * stage_bytes, b_src = a_src + x_base;
        for (int j = 0; j < kbs; ++j) {
          const uint64_t adesc = kmajor_sw128_desc(a_src + (uint32_t)j * (kTileW * kTileK * 2));
          const uint64_t bdesc = kmajor_sw128_desc(b_src + (uint32_t)j * (BN * kTileK * 2));
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k)
            mma_bf16(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                     (kb > kb_begin || j > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
        if (++stage == n_stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (alive) mma_commit(acc_bar);
    }
    __syncwarp();
  }

  ok = mbar_wait(acc_bar, 0, err);
  tc_fence_after_sync();
  const int tl = warp * 32 + lane;        // row of the W tile = TMEM lane
  const int n = tile * kTileW + tl;       // this thread's weight row = output column
  const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
  // Once the accumulator is complete every TMA write has landed and every MMA has read its operands, so the
  // pipeline buffers are free: the finished bf16 tile is staged there as [BN][128] and stored row by row.
  bf16* stage = reinterpret_cast<bf16*>(base_ptr);
  const size_t tile_floats = (size_t)BN * kTileW;
  // split-K partials: [row_tile][split][tile][column][128 lanes], so a warp stores 128 contiguous bytes
  float* partial0 = partials + (((size_t)row_tile * splits) * gridDim.x + tile) * tile_floats;
  const size_t split_stride = (size_t)gridDim.x * tile_floats;
  if (ok) {
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 16) {
      float v[16];
      tmem_ld16(lane_addr + c0, v);
#pragma unroll
      for (int a = 1; a < S::kAccs; ++a) {  // fixed order: ((acc0 + acc1) + acc2) + acc3
        float w[16];
        tmem_ld16(lane_addr + a * BN + c0, w);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] += w[j];
      }
      if (splits == 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          stage[(c0 + j) * kTileW + tl] = n < N ? finish(v[j], n, bias, kind) : __float2bfloat16(0.f);
      } else {
        float* mine = partial0 + split * split_stride + (size_t)c0 * kTileW + tl;
#pragma unroll
        for (int j = 0; j < 16; ++j) mine[j * kTileW] = v[j];
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, S::kTmemCols);

  bool write_out = ok && splits == 1;
  if (splits > 1) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t slot = row_tile * gridDim.x + tile;
      const uint32_t prev = atomicAdd(&counters[slot], 1u);
      is_last = prev == (uint32_t)(splits - 1);
      if (is_last) counters[slot] = 0;  // every split has arrived; ready for the next launch
    }
    __syncthreads();
    if (is_last) {
      __threadfence();
      // sum the splits in index order: the result does not depend on which CTA arrived last
      if (splits <= 2)
        reduce_tile<BN, 4>(partial0, split_stride, splits, tl, n, N, bias, kind, stage);
      else if (splits <= 4)
        reduce_tile<BN, 2>(partial0, split_stride, splits, tl, n, N, bias, kind, stage);
      else
        reduce_tile<BN, 1>(partial0, split_stride, splits, tl, n, N, bias, kind, stage);
      write_out = true;
    }
  }
  if (write_out) {  // uniform across the block
    __syncthreads();
    const int m0 = row_tile * BN, n0 = tile * kTileW;
    const bool vec = (ldy % 8 == 0) && (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
    if (vec) {
      for (int idx = threadIdx.x; idx < BN * (kTileW / 8); idx += blockDim.x) {
        const int m = idx / (kTileW / 8), ch = idx % (kTileW / 8);
        if (m0 + m < rows && n0 + ch * 8 < N)
          *reinterpret_cast<uint4*>(y + (int64_t)(m0 + m) * ldy + n0 + ch * 8) =
              *reinterpret_cast<const uint4*>(stage + m * kTileW + ch * 8);
      }
    } else {
      for (int idx = threadIdx.x; idx < BN * kTileW; idx += blockDim.x) {
        const int m = idx / kTileW, c = idx % kTileW;
        if (m0 + m < rows && n0 + c < N) y[(int64_t)(m0 + m) * ldy + n0 + c] = stage[m * kTileW + c];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Tensor-core tiles with the input rows on the MMA M dimension (at most 128 of them) and TN weight rows on N: one CTA
// computes y[:, tile] over the whole K, so there is no split, no partial tile and no reduction. It is the faster
// one for the decode-sized GEMMs of the secondary model shells (at most 128 sessions, K up to 4096), whose small
// matrices the split-K kernel cannot spread without paying a serial reduction per tile.
//   warp 0 / lane 0: TMA producer, a ring of {X tile 128 x 64 x kbs, W tile TN x 64 x kbs} (kbs k-blocks per copy);
//   warp 1 / lane 0: MMA issuer;
//   all four warps: epilogue, a thread owns one output row (its TMEM lane) and writes it 16 columns at a time.

// The tile width TN (weight rows per CTA, a multiple of 16 up to 256) is a launch parameter: the host picks the
// narrowest one whose tile count still fits one wave, because what bounds a CTA here is the number of 128-byte tile
// rows its TMA unit moves per k-block (128 activation rows + TN weight rows), so the weight rows should be spread over
// every SM.
struct RmShape {
  static constexpr int kRingBytes = 192 * 1024;
  static constexpr int kMaxStages = 8;
  static constexpr size_t kSmemBytes = (size_t)kRingBytes + 1024 + 256;
  // bn: rows of the activation box (16, 32, 64 or 128). The MMA reads 128 rows from where the box starts, so with a
  // smaller box it reads on into whatever follows (those TMEM lanes are never read back); 16 KB of the ring stay
  // unused so that the last stage's reads end inside the CTA's shared memory.
  static int box_rows(int rows) { return rows <= 16 ? 16 : rows <= 32 ? 32 : rows <= 64 ? 64 : 128; }
  static int stage_bytes(int tn, int kbs, int bn) { return kbs * (bn * kTileK * 2 + tn * kTileK * 2); }
  static int stages(int tn, int kbs, int bn) {
    return std::min(kMaxStages, (kRingBytes - (bn < 128 ? 16 * 1024 : 0)) / stage_bytes(tn, kbs, bn));
  }
  static uint32_t tmem_cols(int tn) { return tn <= 32 ? 32u : tn <= 64 ? 64u : tn <= 128 ? 128u : 256u; }
};

__global__ void __launch_bounds__(128, 1)
    gemm_rm_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                   bf16* __restrict__ y, int ldy, int N, int K, int rows, int tn, int kbs, int bn, int n_stages,
                   uint32_t tmem_cols,
                   const bf16* bias, int kind, uint32_t* err) {
  using namespace sm100;
  if (*reinterpret_cast<volatile uint32_t*>(err) != 0) return;
  extern __shared__ unsigned char rm_smem_raw[];
  const uint32_t raw = smem_addr(rm_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = rm_smem_raw + (base - raw);
  const uint32_t x_slice = (uint32_t)bn * kTileK * 2, x_bytes = (uint32_t)kbs * x_slice, w_slice = (uint32_t)tn * kTileK * 2;
  const uint32_t stage_bytes = x_bytes + (uint32_t)kbs * w_slice;
  const uint32_t bars = base + RmShape::kRingBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (RmShape::kMaxStages + s); };
  const uint32_t acc_bar = bars + 8u * (2 * RmShape::kMaxStages);
  const uint32_t tmem_slot = acc_bar + 8u;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + RmShape::kRingBytes + 8 * (2 * RmShape::kMaxStages) + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, nkb = K / kTileK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_bar, 1);
    mbar_init_fence();
    prefetch_tensormap(&wmap);
    prefetch_tensormap(&xmap);
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < nkb; kb += kbs) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, err)) break;
        const uint32_t a_dst = base + stage * stage_bytes, b_dst = a_dst + x_bytes;
        mbar_expect_tx(full_bar(stage), stage_bytes);
        tma_load_3d(a_dst, &xmap, full_bar(stage), 0, 0, kb, kEvictLast);
        tma_load_3d(b_dst, &wmap, full_bar(stage), 0, tile * tn, kb, kEvictFirst);
        if (++stage == n_stages) stage = 0, phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16_f32(128, tn);
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int kb = 0; kb < nkb && alive; kb += kbs) {
        alive = mbar_wait(full_bar(stage), phase, err);
        if (!alive) break;
        tc_fence_after_sync();
        const uint32_t a_src = base + stage * stage_bytes, b_src = a_src + x_bytes;
        for (int j = 0; j < kbs; ++j) {
          const uint64_t adesc = kmajor_sw128_desc(a_src + (uint32_t)j * x_slice);
          const uint64_t bdesc = kmajor_sw128_desc(b_src + (uint32_t)j * w_slice);
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k)
            mma_bf16(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                     (kb > 0 || j > 0 || k > 0) ? 1u : 0u);
        }
        mma_commit(empty_bar(stage));
        if (++stage == n_stages) stage = 0, phase ^= 1u;
      }
      if (alive) mma_commit(acc_bar);
    }
    __syncwarp();
  }

  const bool ok = mbar_wait(acc_bar, 0, err);
  tc_fence_after_sync();
  const int m = warp * 32 + lane;  // output row = TMEM lane
  const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
  if (ok && warp * 32 < rows) {
    const int n0 = tile * tn;
    const bool vec = (ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(y) & 15) == 0);
#pragma unroll 2
    for (int c0 = 0; c0 < tn; c0 += 16) {
      float v[16];
      tmem_ld16(lane_addr + c0, v);
      if (m >= rows || n0 + c0 >= N) continue;
      bf16* dst = y + (int64_t)m * ldy + n0 + c0;
      if (vec && n0 + c0 + 16 <= N) {
        float o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j] = __bfloat162float(finish(v[j], n0 + c0 + j, bias, kind));
        st8(dst, o);
        st8(dst + 8, o + 8);
      } else {
        for (int j = 0; j < 16 && n0 + c0 + j < N; ++j) dst[j] = finish(v[j], n0 + c0 + j, bias, kind);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// --- host side ----------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

int tc_init() {
  if (g_encode) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) return -1;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return 0;
}

static int encode_kmajor(CUtensorMap* map, const bf16* base, int rows, int K, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(bf16)};
  const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<bf16*>(base), dims, strides, box,
                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -1;
}

// A bf16 tensor of any rank up to 5 with the 128-byte swizzle (box[0] must be 64 elements); strides in bytes for the
// dimensions above the innermost. For callers that tile something other than a dense [rows, K] matrix.
int tc_encode_bf16(CUtensorMap* map, const bf16* base, int rank, const uint64_t* dims, const uint64_t* strides,
                   const uint32_t* box) {
  if (tc_init() != 0) return -1;
  cuuint64_t d[5], s[4];
  cuuint32_t b[5], elem[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) d[i] = dims[i], b[i] = box[i];
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides[i];
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<bf16*>(base), d, s, b,
                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -1;
}

// The same matrix as a rank-3 map {element in a k-block, row, k-block} whose box holds `kbs` k-blocks of `box_rows` rows.
static int encode_kmajor3(CUtensorMap* map, const bf16* base, int rows, int K, int box_rows, int kbs) {
  const cuuint64_t dims[3] = {(cuuint64_t)kTileK, (cuuint64_t)rows, (cuuint64_t)(K / kTileK)};
  const cuuint64_t strides[2] = {(cuuint64_t)K * sizeof(bf16), (cuuint64_t)kTileK * sizeof(bf16)};
  const cuuint32_t box[3] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows, (cuuint32_t)kbs};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<bf16*>(base), dims, strides, box,
                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -1;
}

bool tc_supports(int N, int K, int rows) {
  return K % kTileK == 0 && K >= kTileK && N >= 1 && rows >= 1;
}

static int pick_bn(int rows) {
  if (rows <= 16) return 16;
  if (rows <= 32) return 32;
  if (rows <= 64) return 64;
  if (rows <= 128) return 128;
  return 256;
}

int tc_plan(TcGemmPlan* plan, const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy, Epilogue epi,
            int sm_count, int force_splits) {
  if (tc_init() != 0) return -1;
  if (!tc_supports(N, K, rows)) return -2;
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return -3;
  TcGemmPlan& p = *plan;
  p.N = N;
  p.K = K;
  p.rows = rows;
  p.BN = pick_bn(rows);
  p.row_tiles = (rows + p.BN - 1) / p.BN;
  p.y = y;
  p.ldy = ldy;
  p.epi = epi;
  const int nkb = K / kTileK, ctas = p.tiles_n() * p.row_tiles;
  int splits = force_splits > 0 ? force_splits : std::max(1, sm_count / ctas);
  // at least four K blocks per split (two when forced): below that the reduction costs more than it spreads
  splits = std::max(1, std::min(splits, force_splits > 0 ? nkb / 2 : nkb / 4));
  // the last CTA's reduction is a serial chain of L2 round trips: at most 8 splits, 4 for wide row tiles
  if (force_splits <= 0) splits = std::min(splits, p.BN >= 128 ? 4 : 8);
  p.splits = splits;
  // k-blocks per TMA copy: a tiled copy occupies the TMA unit for about 0.19 us whatever its size; the ring must still
  // hold two stages, and every split must be a whole number of copies
  p.kbs = 1;
  if (nkb % splits == 0) {
    const int per = nkb / splits, stage = kTileW * kTileK * 2 + p.BN * kTileK * 2;
    const int stages1 = std::min(8, 200 * 1024 / stage);
    double best = 1e30;
    for (int kbs : {1, 2, 4}) {
      if (per % kbs || stages1 / kbs < 2) continue;
      const double cost = (per / kbs) * std::max({0.38, kbs * stage / 110e3, 2.0 / (stages1 / kbs)});
      if (cost < best - 1e-9) best = cost, p.kbs = kbs;
    }
  }
  if (p.kbs == 1) {
    if (encode_kmajor(&p.wmap, w, N, K, kTileW) != 0) return -4;
    if (encode_kmajor(&p.xmap, x, rows, K, p.BN) != 0) return -4;
  } else {
    if (encode_kmajor3(&p.wmap, w, N, K, kTileW, p.kbs) != 0) return -4;
    if (encode_kmajor3(&p.xmap, x, rows, K, p.BN, p.kbs) != 0) return -4;
  }
  return 0;
}

template <int BN>
static cudaError_t tc_launch_bn(const TcGemmPlan& p, const GemmScratch& s, uint32_t* err, cudaStream_t stream) {
  using S = TcShape<BN>;
  const dim3 grid(p.tiles_n(), p.splits, p.row_tiles);
  gemm_tc_kernel<BN><<<grid, 128, S::kSmemBytes, stream>>>(p.wmap, p.xmap, p.y, p.ldy, p.N, p.K, p.rows, p.splits,
                                                           p.kbs, s.partials, s.counters, p.epi.bias, p.epi.kind, err);
  return cudaGetLastError();
}

// Raises the dynamic shared-memory limit of every instantiation up front, so no
// attribute call falls inside a stream capture.
void tc_configure() {
  cudaFuncSetAttribute(gemm_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcShape<16>::kSmemBytes);
  cudaFuncSetAttribute(gemm_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcShape<32>::kSmemBytes);
  cudaFuncSetAttribute(gemm_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcShape<64>::kSmemBytes);
  cudaFuncSetAttribute(gemm_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcShape<128>::kSmemBytes);
  cudaFuncSetAttribute(gemm_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcShape<256>::kSmemBytes);
  cudaFuncSetAttribute(gemm_rm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RmShape::kSmemBytes);
  cudaFuncSetAttribute(gemv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaFuncSetAttribute(gemv_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaFuncSetAttribute(gemv_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  cudaFuncSetAttribute(gemv_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}

cudaError_t tc_launch(const TcGemmPlan& p, const GemmScratch& s, uint32_t* err, cudaStream_t stream) {
  if (p.splits > 1) {
    if (p.partial_floats() > s.partial_floats || p.tiles_n() * p.row_tiles > s.counter_slots)
      return cudaErrorInvalidValue;
  }
  switch (p.BN) {
    case 16: return tc_launch_bn<16>(p, s, err, stream);
    case 32: return tc_launch_bn<32>(p, s, err, stream);
    case 64: return tc_launch_bn<64>(p, s, err, stream);
    case 128: return tc_launch_bn<128>(p, s, err, stream);
    case 256: return tc_launch_bn<256>(p, s, err, stream);
  }
  return cudaErrorInvalidValue;
}

// ---- rows-on-M path ---------------------------------------------------------------

bool rm_supports(int N, int K, int rows) {
  return K % kTileK == 0 && K >= kTileK && K <= 4096 && rows >= 1 && rows <= 128 && N >= 1;
}

int rm_plan(RmGemmPlan* plan, const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy, Epilogue epi,
            int sm_count) {
  if (tc_init() != 0) return -1;
  if (!rm_supports(N, K, rows)) return -2;
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15)) return -3;
  RmGemmPlan& p = *plan;
  p.N = N, p.K = K, p.rows = rows, p.y = y, p.ldy = ldy, p.epi = epi;
  // the narrowest tile (a multiple of 16 weight rows) whose count still fits one wave of CTAs
  const int per_sm = (N + sm_count - 1) / std::max(1, sm_count);
  p.TN = std::min(256, std::max(16, (per_sm + 15) / 16 * 16));
  // k-blocks per stage: a tiled copy occupies the TMA unit for about 0.19 us whatever its size, a stage is two copies
  // (about 110 GB/s per SM at best), and the ring must cover about 2 us of latency
  const int nkb = K / kTileK;
  double best = 1e30;
  p.kbs = 1;
  p.bn = RmShape::box_rows(rows);
  for (int kbs : {1, 2, 4}) {
    if (nkb % kbs) continue;
    const int stages = RmShape::stages(p.TN, kbs, p.bn);
    if (stages < 2) continue;
    const double per_stage = std::max({0.38, RmShape::stage_bytes(p.TN, kbs, p.bn) / 110e3, 2.0 / stages});
    const double cost = per_stage * (nkb / kbs);
    if (cost < best - 1e-9) best = cost, p.kbs = kbs;
  }
  if (encode_kmajor3(&p.wmap, w, N, K, p.TN, p.kbs) != 0) return -4;
  if (encode_kmajor3(&p.xmap, x, rows, K, p.bn, p.kbs) != 0) return -4;
  return 0;
}

cudaError_t rm_launch(const RmGemmPlan& p, uint32_t* err, cudaStream_t stream) {
  if (p.TN < 16 || p.TN > 256 || p.TN % 16) return cudaErrorInvalidValue;
  gemm_rm_kernel<<<(p.N + p.TN - 1) / p.TN, 128, RmShape::kSmemBytes, stream>>>(
      p.wmap, p.xmap, p.y, p.ldy, p.N, p.K, p.rows, p.TN, p.kbs, p.bn, RmShape::stages(p.TN, p.kbs, p.bn),
      RmShape::tmem_cols(p.TN),
      p.epi.bias,
      p.epi.kind, err);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// The split-K tensor-core GEMM for callers that must not allocate.
//
// The split-K path needs scratch in global memory: one f32 tile per split and
// an arrival counter per output tile. Everywhere else in this library that
// scratch comes from cudaMalloc. Here it is a fixed array inside the loaded
// module instead, so the call never asks the driver for memory.

namespace {
constexpr size_t kStaticPartialFloats = (size_t)4 << 20;  // 16 MiB of f32 partial tiles
constexpr int kStaticCounterSlots = 2048;

// Reserved on every GPU that loads this library, from load until the process exits.
static __device__ __align__(256) float g_static_partials[kStaticPartialFloats];
static __device__ __align__(256) uint32_t g_static_counters[kStaticCounterSlots];
static __device__ __align__(256) uint32_t g_static_error[64];

// In host code the three names above are only handles to the device arrays; the
// device addresses a kernel can use are looked up once per device, with that
// device current, and kept here.
constexpr int kStaticDevices = 64;
struct StaticScratch {
  bool ready = false;
  float* partials = nullptr;
  uint32_t* counters = nullptr;
  uint32_t* error = nullptr;
};
StaticScratch g_static[kStaticDevices];
std::mutex g_static_mutex;  // two host threads may make their first call on a device at once

void say(char* buf, size_t len, const char* fmt, ...) {
  if (!buf || len == 0) return;
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, len, fmt, ap);
  va_end(ap);
}
}  // namespace

}  // namespace omni

extern "C" int32_t omni_op_gemm_noalloc(const void* w, int32_t N, int32_t K, const void* x, int32_t rows, void* y,
                                        int32_t ldy, int32_t splits, const void* bias, int32_t epilogue, void* stream,
                                        char* message, size_t message_len) {
  using namespace omni;
  const int32_t kInvalid = -1, kCuda = -2, kDevice = -3, kUnsupported = -5;  // enum omni_status
  if (message && message_len) message[0] = 0;
  if (!w || !x || !y || N < 1 || rows < 1 || K < 64 || K % 64 || ldy < N) {
    say(message, message_len, "bad argument: need w, x, y, N >= 1, rows >= 1, K a multiple of 64, ldy >= N");
    return kInvalid;
  }
  if (epilogue != kEpiNone && !bias) {
    say(message, message_len, "epilogue %d needs a bias", epilogue);
    return kInvalid;
  }
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) {
    say(message, message_len, "cudaGetDevice: %s", cudaGetErrorString(e));
    return kCuda;
  }
  if (device < 0 || device >= kStaticDevices) {
    say(message, message_len, "device index %d is beyond the %d devices this entry point keeps addresses for", device,
        kStaticDevices);
    return kUnsupported;
  }
  if (stream) {  // the scratch addresses belong to the current device: a stream of another device would get the wrong ones
    int stream_device = device;
#if CUDART_VERSION >= 12080
    if (cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &stream_device) != cudaSuccess) {
      cudaGetLastError();
      stream_device = device;
    }
#endif
    if (stream_device != device) {
      say(message, message_len, "the stream belongs to device %d, the current device is %d", stream_device, device);
      return kInvalid;
    }
  }
  StaticScratch& sc = g_static[device];
  std::lock_guard<std::mutex> lock(g_static_mutex);  // (also serialises this entry point's calls from host threads)
  if (!sc.ready) {  // first call on this device: resolve the arrays' device addresses
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess || prop.major != 10) {
      say(message, message_len, "device %d is not sm_100 (%s)", device, cudaGetErrorString(e));
      return e != cudaSuccess ? kCuda : kUnsupported;
    }
    if (tc_init() != 0) {
      say(message, message_len, "cuTensorMapEncodeTiled entry point not found");
      return kCuda;
    }
    tc_configure();
    void *p = nullptr, *c = nullptr, *r = nullptr;
    if ((e = cudaGetSymbolAddress(&p, g_static_partials)) != cudaSuccess ||
        (e = cudaGetSymbolAddress(&c, g_static_counters)) != cudaSuccess ||
        (e = cudaGetSymbolAddress(&r, g_static_error)) != cudaSuccess) {
      say(message, message_len, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return kCuda;
    }
    sc.partials = static_cast<float*>(p);
    sc.counters = static_cast<uint32_t*>(c);
    sc.error = static_cast<uint32_t*>(r);
    sc.ready = true;
  }
  int sm_count = 148;
  if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sm_count = 148;
  Epilogue epi;
  epi.bias = static_cast<const bf16*>(bias);
  epi.kind = epilogue;
  TcGemmPlan plan;
  const int rc = tc_plan(&plan, static_cast<const bf16*>(w), N, K, static_cast<const bf16*>(x), rows,
                         static_cast<bf16*>(y), ldy, epi, sm_count, splits);
  if (rc != 0) {
    say(message, message_len, "tensor-map encode failed (%d): operands must be 16-byte aligned", rc);
    return kInvalid;
  }
  if (plan.partial_floats() > kStaticPartialFloats || plan.tiles_n() * plan.row_tiles > kStaticCounterSlots) {
    say(message, message_len,
        "too large for the built-in scratch: needs %zu partial floats (limit %zu) and %d tile counters (limit %d); "
        "use omni_op_gemm, whose context allocates its scratch",
        plan.partial_floats(), kStaticPartialFloats, plan.tiles_n() * plan.row_tiles, kStaticCounterSlots);
    return kUnsupported;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the arrays keep whatever the previous call left: counters and the error word must start at zero
  if ((e = cudaMemsetAsync(sc.counters, 0, sizeof(uint32_t) * kStaticCounterSlots, s)) != cudaSuccess ||
      (e = cudaMemsetAsync(sc.error, 0, sizeof(uint32_t), s)) != cudaSuccess) {
    say(message, message_len, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    return kCuda;
  }
  GemmScratch scratch;
  scratch.partials = sc.partials;
  scratch.partial_floats = kStaticPartialFloats;
  scratch.counters = sc.counters;
  scratch.counter_slots = kStaticCounterSlots;
  if ((e = tc_launch(plan, scratch, sc.error, s)) != cudaSuccess) {
    say(message, message_len, "launch: %s", cudaGetErrorString(e));
    return kCuda;
  }
  uint32_t word = 0;
  if ((e = cudaMemcpyAsync(&word, sc.error, sizeof(word), cudaMemcpyDeviceToHost, s)) != cudaSuccess ||
      (e = cudaStreamSynchronize(s)) != cudaSuccess) {
    say(message, message_len, "wait: %s", cudaGetErrorString(e));
    return kCuda;
  }
  if (word != 0) {
    say(message, message_len, "device error word 0x%x (1: a bounded barrier wait ran out)", word);
    return kDevice;
  }
  return 0;
}
