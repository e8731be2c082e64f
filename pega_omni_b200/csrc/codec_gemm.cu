// The codec decoder's causal conv as an implicit GEMM on tcgen05 (declared in codec.h).
//
// The reference materialises every conv's dilated im2col matrix [rows, taps * C] and hands it to a library GEMM
// (crates/omni-qwen3-tts/src/codec.rs:60-93, kernels/codec.cu:291-318). Here the im2col matrix never exists: the
// activation is kept once, padded with its history, as [stream][H + T][C], and the K loop walks (tap, channel block);
// for tap j the activation tile of 128 output rows is the same rank-3/4 TMA box shifted down by j * dil rows. The rows
// of a tile are SB streams x TB consecutive frame rows (TB * SB = 128), so a tile never reads across a stream's padding.
//
//   warp 0 / lane 0: TMA producer, a ring of {activation tile 128 x 64 x kbs, weight tile tn x 64 x kbs};
//   warp 1 / lane 0: MMA issuer (M = 128 rows, N = tn output channels, two accumulators in TMEM);
//   twelve warps:    epilogue, three per TMEM lane quadrant, 32 channels of 32 rows per step. The epilogue (SnakeBeta
//                    over every value of a tile, or a read-modify-write of the residual stream) is what a tile costs
//                    once the K loop is fed: with 4 / 8 / 12 epilogue warps the decoder's frame takes 1.49 / 1.42 / 1.39 ms.
//
// Channel counts that are not multiples of 64 (96 in the last decoder block) take the "ragged" loads: the activation
// box past channel C is zero-filled by TMA, so whatever weight columns of the next tap the weight box then covers
// multiply zeros.
#include <algorithm>

#include "codec.h"
#include "gemm.h"
#include "sm100.cuh"

namespace omni {

namespace {

constexpr int kConvK = 64;        // channels per k-block: one 128-byte swizzle row
constexpr int kConvRows = 128;    // output rows per tile
constexpr int kConvRing = 168 * 1024;
constexpr int kConvMaxStages = 8;
constexpr int kConvEpilogueWarps = 12;  // three per TMEM lane quadrant, each taking every third 32-channel step
constexpr int kConvThreads = 64 + 32 * kConvEpilogueWarps;  // warp 0 producer, warp 1 MMA issuer, the rest epilogue
constexpr int kStagePitch = 36;   // floats per row of an epilogue warp's 32 x 32 staging block (16-byte aligned, conflict-free)
constexpr size_t kConvSmem = (size_t)kConvRing + 1024 + 256 + kConvEpilogueWarps * 32 * kStagePitch * sizeof(float);

struct ConvArgs {
  bf16* y;
  const bf16* bias;
  const float* alpha;
  const float* inv_b;
  uint32_t* err;
  int N, C, taps, dil, T, seqs, TB, SB, tn, kbs, cpb, ragged, stages, kind, t_tiles, n_tiles, tiles;
  uint32_t acc_cols;  // TMEM columns per accumulator (a power of two >= tn); two accumulators are allocated
};

// Persistent: a CTA walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... (output-channel tile fastest, so CTAs that run
// together share activation rows in L2). The ring never drains between tiles: the producer runs ahead into the next
// tile's loads while the epilogue warps drain the accumulator of the one before, which is why there are two.
__global__ void __launch_bounds__(kConvThreads, 1)
    conv_gemm_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap,
                     const ConvArgs a) {
  using namespace sm100;
  if (*reinterpret_cast<volatile uint32_t*>(a.err) != 0) return;
  extern __shared__ unsigned char conv_smem_raw[];
  const uint32_t raw = smem_addr(conv_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char* base_ptr = conv_smem_raw + (base - raw);
  const uint32_t x_slice = kConvRows * kConvK * 2, x_bytes = (uint32_t)a.kbs * x_slice;
  const uint32_t w_slice = (uint32_t)a.tn * kConvK * 2, stage_bytes = x_bytes + (uint32_t)a.kbs * w_slice;
  const uint32_t bars = base + kConvRing;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kConvMaxStages + s); };
  auto acc_full = [&](int b) { return bars + 8u * (2 * kConvMaxStages + b); };
  auto acc_empty = [&](int b) { return bars + 8u * (2 * kConvMaxStages + 2 + b); };
  const uint32_t tmem_slot = bars + 8u * (2 * kConvMaxStages + 4);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + kConvRing + 8 * (2 * kConvMaxStages + 4));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int steps = a.taps * a.cpb / a.kbs;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full(b), 1);
      mbar_init(acc_empty(b), kConvEpilogueWarps);  // one arrival per epilogue warp
    }
    mbar_init_fence();
    prefetch_tensormap(&xmap);
    prefetch_tensormap(&wmap);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 2 * a.acc_cols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < a.tiles && alive; tile += gridDim.x) {
        const int n0 = (tile % a.n_tiles) * a.tn, rt = tile / a.n_tiles;
        const int t0 = (rt % a.t_tiles) * a.TB, s0 = (rt / a.t_tiles) * a.SB;
        for (int i = 0; i < steps; ++i) {
          alive = mbar_wait(empty_bar(stage), phase ^ 1u, a.err);
          if (!alive) break;
          const int kb = i * a.kbs, tap = kb / a.cpb, cb = kb % a.cpb;
          const uint32_t a_dst = base + stage * stage_bytes, b_dst = a_dst + x_bytes;
          mbar_expect_tx(full_bar(stage), stage_bytes);
          if (a.ragged) {
            tma_load_3d(a_dst, &xmap, full_bar(stage), cb * kConvK, t0 + tap * a.dil, s0, kEvictNormal);
            tma_load_2d(b_dst, &wmap, full_bar(stage), tap * a.C + cb * kConvK, n0, kEvictLast);
          } else {
            tma_load_4d(a_dst, &xmap, full_bar(stage), 0, t0 + tap * a.dil, s0, cb, kEvictNormal);
            tma_load_3d(b_dst, &wmap, full_bar(stage), 0, n0, tap * a.cpb + cb, kEvictLast);
          }
          if (++stage == a.stages) stage = 0, phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = idesc_bf16_f32(kConvRows, a.tn);
      int stage = 0, use = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < a.tiles && alive; tile += gridDim.x, ++use) {
        const int buf = use & 1;
        // the epilogue of this accumulator's previous tile must have read it out (a fresh barrier passes at once)
        alive = mbar_wait(acc_empty(buf), ((uint32_t)(use >> 1) & 1u) ^ 1u, a.err);
        if (!alive) break;
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + (uint32_t)buf * a.acc_cols;
        for (int i = 0; i < steps; ++i) {
          alive = mbar_wait(full_bar(stage), phase, a.err);
          if (!alive) break;
          tc_fence_after_sync();
          const uint32_t a_src = base + stage * stage_bytes, b_src = a_src + x_bytes;
          for (int j = 0; j < a.kbs; ++j) {
            const uint64_t adesc = kmajor_sw128_desc(a_src + (uint32_t)j * x_slice);
            const uint64_t bdesc = kmajor_sw128_desc(b_src + (uint32_t)j * w_slice);
#pragma unroll
            for (int k = 0; k < kConvK / 16; ++k)
              mma_bf16(acc, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                       (i > 0 || j > 0 || k > 0) ? 1u : 0u);
          }
          mma_commit(empty_bar(stage));
          if (++stage == a.stages) stage = 0, phase ^= 1u;
        }
        if (alive) mma_commit(acc_full(buf));
      }
    }
    __syncwarp();
  } else {
    // Epilogue. A warp reaches the 32 TMEM lanes of quadrant warp % 4, one output row per thread, and takes the tile 32
    // channels at a time. A thread's row is 2 * N bytes away from its neighbour's, so storing from that layout would
    // cost one memory transaction per thread and 16 bytes; instead the 32 x 32 f32 block goes through shared memory
    // and comes back with four lanes per row (8 channels each), so that a warp instruction covers 8 rows x 64 bytes.
    // The old values of an accumulating GEMM, the bias and the SnakeBeta parameters are read in that layout too.
    const int quad = warp & 3, turn = (warp - 2) >> 2;  // this warp takes steps turn, turn + 3, ... of 32 channels
    float* stg = reinterpret_cast<float*>(base_ptr + kConvRing + 256) + (warp - 2) * (32 * kStagePitch);
    const int sub_row = lane >> 2, chunk = lane & 3;
    int use = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < a.tiles && alive; tile += gridDim.x, ++use) {
      const int buf = use & 1;
      const int n0 = (tile % a.n_tiles) * a.tn, rt = tile / a.n_tiles;
      const int t0 = (rt % a.t_tiles) * a.TB, s0 = (rt / a.t_tiles) * a.SB;
      const uint32_t lane_addr = tmem_base + (uint32_t)buf * a.acc_cols + ((uint32_t)(quad * 32) << 16);
      // the four rows this lane stores in every step
      bf16* rows[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = quad * 32 + 8 * i + sub_row, s = s0 + m / a.TB, t = t0 + m % a.TB;
        rows[i] = s < a.seqs ? a.y + ((int64_t)s * a.T + t) * a.N : nullptr;
      }
      alive = mbar_wait(acc_full(buf), (uint32_t)(use >> 1) & 1u, a.err);
      if (!alive) break;
      tc_fence_after_sync();
#pragma unroll 1
      for (int c0 = 32 * turn; c0 < a.tn; c0 += 32 * (kConvEpilogueWarps / 4)) {
        uint32_t r0[16], r1[16];
        const bool second = c0 + 16 < a.tn;  // tn is a multiple of 16: the last step may hold one half only
        tmem_ld16_issue(lane_addr + c0, r0);  // warp-wide: every lane takes part whether or not its row is live
        if (second) {
          tmem_ld16_issue(lane_addr + c0 + 16, r1);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r1[j] = 0u;
        }
        const int nn = n0 + c0 + 8 * chunk;
        const bool cols_live = c0 + 8 * chunk < a.tn && nn + 8 <= a.N;
        uint4 old[4] = {};
        if (a.kind == kConvAccumulate && cols_live) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (rows[i]) old[i] = *reinterpret_cast<const uint4*>(rows[i] + nn);
        }
        tmem_ld_fence(r0, r1);
        uint4* mine = reinterpret_cast<uint4*>(stg + lane * kStagePitch);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          mine[q] = make_uint4(r0[4 * q], r0[4 * q + 1], r0[4 * q + 2], r0[4 * q + 3]);
          mine[4 + q] = make_uint4(r1[4 * q], r1[4 * q + 1], r1[4 * q + 2], r1[4 * q + 3]);
        }
        __syncwarp();
        if (cols_live) {
          float b[8], al[8], ib[8];
          if (a.kind == kConvBiasSnake) {
            ld8v(a.bias + nn, b);
            const float4 a0 = *reinterpret_cast<const float4*>(a.alpha + nn), a1 = *reinterpret_cast<const float4*>(a.alpha + nn + 4);
            const float4 i0 = *reinterpret_cast<const float4*>(a.inv_b + nn), i1 = *reinterpret_cast<const float4*>(a.inv_b + nn + 4);
            al[0] = a0.x, al[1] = a0.y, al[2] = a0.z, al[3] = a0.w, al[4] = a1.x, al[5] = a1.y, al[6] = a1.z, al[7] = a1.w;
            ib[0] = i0.x, ib[1] = i0.y, ib[2] = i0.z, ib[3] = i0.w, ib[4] = i1.x, ib[5] = i1.y, ib[6] = i1.z, ib[7] = i1.w;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (!rows[i]) continue;
            const float4* src = reinterpret_cast<const float4*>(stg + (8 * i + sub_row) * kStagePitch + 8 * chunk);
            const float4 lo = src[0], hi = src[1];
            float o[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            if (a.kind == kConvAccumulate) {
              float prev[8];
              unpack8v(old[i], prev);
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] += prev[j];
            } else if (a.kind == kConvBiasSnake) {
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] = snake_beta(bf16_round(o[j]) + b[j], al[j], ib[j]);
            }
            st8v(rows[i] + nn, o);
          }
        }
        __syncwarp();  // the block is read out before the next step overwrites it
      }
      // this warp's part of the accumulator has been read (a warp without a step of its own arrives all the same)
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(buf));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * a.acc_cols);
}

}  // namespace

void conv_configure() {
  cudaFuncSetAttribute(conv_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kConvSmem);
}

int conv_plan(ConvGemmPlan* plan, const bf16* w, int N, int C, int taps, int dil, const bf16* x, int T, int seqs, bf16* y,
              int kind, const bf16* bias, const float* alpha, const float* inv_b, int sm_count) {
  if (N < 8 || N % 8 || C < 8 || C % 8 || taps < 1 || T < 1 || seqs < 1) return -2;
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15))
    return -3;
  ConvGemmPlan& p = *plan;
  p.N = N, p.C = C, p.taps = taps, p.dil = dil, p.T = T, p.seqs = seqs, p.y = y;
  p.kind = kind, p.bias = bias, p.alpha = alpha, p.inv_b = inv_b;
  p.TB = 1;
  while (p.TB < kConvRows && T % (p.TB * 2) == 0) p.TB *= 2;
  p.SB = kConvRows / p.TB;
  p.row_tiles = (T / p.TB) * ((seqs + p.SB - 1) / p.SB);
  p.cpb = (C + kConvK - 1) / kConvK;
  p.ragged = C % kConvK != 0;
  // output channels per CTA: as wide as the accumulator allows when the rows alone fill the machine, else narrow
  // enough that every SM gets a tile
  const int min_tiles = (N + 255) / 256;
  const int want = std::max(min_tiles, std::min((N + 15) / 16, sm_count / std::max(1, p.row_tiles)));
  p.tn = std::min(256, ((N + want - 1) / want + 15) / 16 * 16);
  p.n_tiles = (N + p.tn - 1) / p.tn;
  // k-blocks per TMA copy: a tiled copy occupies the SM's TMA unit for about 0.19 us whatever its size, so narrow
  // tiles move several channel blocks of a tap at once; the ring keeps at least three stages
  p.kbs = 1;
  if (!p.ragged)
    for (int kbs : {4, 3, 2})
      if (p.cpb % kbs == 0 && kConvRing / (kbs * (kConvRows * kConvK * 2 + p.tn * kConvK * 2)) >= 3) {
        p.kbs = kbs;
        break;
      }
  p.stages = std::min(kConvMaxStages, kConvRing / (p.kbs * (kConvRows * kConvK * 2 + p.tn * kConvK * 2)));
  p.ctas = std::min(p.n_tiles * p.row_tiles, sm_count);
  if (p.stages < 2) return -2;
  const int P = (taps - 1) * dil + T, Ktot = taps * C;
  if (p.ragged) {
    const uint64_t xd[3] = {(uint64_t)C, (uint64_t)P, (uint64_t)seqs};
    const uint64_t xs[2] = {(uint64_t)C * 2, (uint64_t)P * C * 2};
    const uint32_t xb[3] = {kConvK, (uint32_t)p.TB, (uint32_t)p.SB};
    if (tc_encode_bf16(&p.xmap, x, 3, xd, xs, xb) != 0) return -4;
    const uint64_t wd[2] = {(uint64_t)Ktot, (uint64_t)N};
    const uint64_t ws[1] = {(uint64_t)Ktot * 2};
    const uint32_t wb[2] = {kConvK, (uint32_t)p.tn};
    if (tc_encode_bf16(&p.wmap, w, 2, wd, ws, wb) != 0) return -4;
  } else {
    const uint64_t xd[4] = {kConvK, (uint64_t)P, (uint64_t)seqs, (uint64_t)p.cpb};
    const uint64_t xs[3] = {(uint64_t)C * 2, (uint64_t)P * C * 2, kConvK * 2};
    const uint32_t xb[4] = {kConvK, (uint32_t)p.TB, (uint32_t)p.SB, (uint32_t)p.kbs};
    if (tc_encode_bf16(&p.xmap, x, 4, xd, xs, xb) != 0) return -4;
    const uint64_t wd[3] = {kConvK, (uint64_t)N, (uint64_t)(Ktot / kConvK)};
    const uint64_t ws[2] = {(uint64_t)Ktot * 2, kConvK * 2};
    const uint32_t wb[3] = {kConvK, (uint32_t)p.tn, (uint32_t)p.kbs};
    if (tc_encode_bf16(&p.wmap, w, 3, wd, ws, wb) != 0) return -4;
  }
  return 0;
}

cudaError_t conv_launch(const ConvGemmPlan& p, uint32_t* err, cudaStream_t stream) {
  ConvArgs a;
  a.y = p.y, a.bias = p.bias, a.alpha = p.alpha, a.inv_b = p.inv_b, a.err = err;
  a.N = p.N, a.C = p.C, a.taps = p.taps, a.dil = p.dil, a.T = p.T, a.seqs = p.seqs, a.TB = p.TB, a.SB = p.SB;
  a.tn = p.tn, a.kbs = p.kbs, a.cpb = p.cpb, a.ragged = p.ragged, a.stages = p.stages, a.kind = p.kind;
  a.t_tiles = p.T / p.TB, a.n_tiles = p.n_tiles, a.tiles = p.n_tiles * p.row_tiles;
  a.acc_cols = p.tn <= 32 ? 32u : p.tn <= 64 ? 64u : p.tn <= 128 ? 128u : 256u;
  conv_gemm_kernel<<<p.ctas, kConvThreads, kConvSmem, stream>>>(p.xmap, p.wmap, a);
  return cudaGetLastError();
}

}  // namespace omni
