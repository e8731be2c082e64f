// Decode attention of one (row, kv head) by a team of W warps (four for long paged sequences, one for the code
// predictor's single-page frames) over the paged KV
//   kv[page][kv_head][K | V][16 tokens][D]   (bf16)
// shared by the stand-alone attention kernel and the persistent tick kernel.
// Value semantics of `attend` (crates/omni-qwen3/kernels/qwen3.cu:123-207): f32 scores and
// accumulation, __expf, per-warp online softmax states merged at the end, bf16 output.
#pragma once
#include "sm100.cuh"
#include "util.cuh"

namespace omni {

constexpr int kAttnWarps = 4;

// A warp's staging slots for K|V blocks: a (page, kv head) block is 2 * 16 * D contiguous bf16 of this GPU's own
// memory, so one untiled bulk copy brings it into shared memory while the warp works on the block before it. With
// S slots a warp has S blocks in flight or in use. `slots`: S * kv_block_bytes<D>() bytes, 128-byte aligned; `bars`:
// S mbarriers initialised with count 1 by the owner (one lane arms and issues). `par` holds the slots' wait parities
// and lives as long as the barriers do.
template <int D>
__host__ __device__ constexpr uint32_t kv_block_bytes() { return 2u * 16u * D * 2u; }

template <int S>
struct PageStage {
  static constexpr int kSlots = S;
  unsigned char* slots;  // this warp's S slots
  uint64_t* bars;        // this warp's S barriers
  uint32_t par;
  uint32_t* err;
};
struct NoStage {
  static constexpr int kSlots = 0;
};

// Element offset of (page, head, K or V, token-in-page) in a layer's KV buffer.
template <int D>
__device__ __forceinline__ int64_t kv_offset(int64_t page, int hk, int head, int which, int tok) {
  return (((page * hk + head) * 2 + which) * 16 + tok) * D;
}

template <int D, int G, int W = kAttnWarps>
struct AttnShared {
  float qs[G][D];  // the G query heads sharing this kv head, f32, filled by the caller
  float ms[W][G], ls[W][G];
  float os[W][G][D];
};
template <int D, int G>
struct AttnShared<D, G, 1> {  // a one-warp team has nothing to merge
  float qs[G][D];
};

struct WarpSync {  // team barrier of a one-warp team
  __device__ __forceinline__ void sync() const { __syncwarp(); }
};

// One (page, kv head) K|V block in a warp's registers. Every load instruction covers contiguous memory: a K block is
// 16 rows of D bf16 back to back, so instruction c takes bytes [512c, 512c + 512) with 16 bytes per lane (a key row
// is spread over LPT = D/8 lanes); of a value row every lane takes its D/32 output dims.
template <int D>
struct KvBlock {
  static constexpr int PV = D / 32;           // output dims per lane
  static constexpr int LPT = D / 8;           // lanes per key row
  static constexpr int TPI = 32 / LPT;        // key rows per load instruction
  static constexpr int NI = 16 / TPI;         // load instructions per K block
  uint4 k[NI];  // loaded as 16-byte words: one request per lane and instruction
  uint2 v[16];
  // `block`: the K rows, then the V rows (global or shared memory)
  __device__ __forceinline__ void load(const bf16* block, int lane) {
    const bf16* vrows = block + 16 * D;
#pragma unroll
    for (int c = 0; c < NI; ++c) k[c] = *reinterpret_cast<const uint4*>(block + (c * 32 + lane) * 8);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if constexpr (PV == 4)
        v[j] = *reinterpret_cast<const uint2*>(vrows + j * D + lane * 4);
      else
        v[j] = make_uint2(*reinterpret_cast<const uint32_t*>(vrows + j * D + lane * 2), 0u);
    }
  }
};

// One online-softmax step of G query heads (`qs`, f32 in shared memory) over the first `ntok` keys of a block:
// q.k with the key rows spread over lanes and finished by shuffles (lane & 15 then owns a key), the running maximum
// and sum, then p.v with every lane on its own output dims. Whole warp.
template <int D, int G>
__device__ __forceinline__ void page_update(const KvBlock<D>& blk, const float (*qs)[D], int ntok, float scale, int lane,
                                            float (&m)[G], float (&l)[G], float (&acc)[G][D / 32]) {
  constexpr int PV = KvBlock<D>::PV, LPT = KvBlock<D>::LPT, TPI = KvBlock<D>::TPI, NI = KvBlock<D>::NI;
  const int key = lane & 15;
  const int sub = lane % LPT;  // which 8 dims of the head this lane multiplies
  float q8[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) q8[g][e] = qs[g][sub * 8 + e];
  float sc[G];
#pragma unroll
  for (int g = 0; g < G; ++g) sc[g] = 0.f;
#pragma unroll
  for (int c = 0; c < NI; ++c) {
    float kf[8];
    unpack8v(blk.k[c], kf);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float part = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) part = fmaf(q8[g][e], kf[e], part);
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
#pragma unroll
      for (int gi = 0; gi < TPI; ++gi) {  // token c*TPI + gi was summed by lane group gi
        const float v = __shfl_sync(0xffffffffu, part, gi * LPT);
        if (key == c * TPI + gi) sc[g] = v;
      }
    }
  }
  float p[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float s = key < ntok ? sc[g] * scale : -INFINITY;
    const float m2 = fmaxf(m[g], warp_fmax(s));
    const float corr = __expf(m[g] - m2);
    p[g] = __expf(s - m2);
    float ps = p[g];  // sum over the 16 keys (both half-warps hold the same values)
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
    l[g] = l[g] * corr + ps;
#pragma unroll
    for (int d = 0; d < PV; ++d) acc[g][d] *= corr;
    m[g] = m2;
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float vf[PV];
    if constexpr (PV == 4) {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&blk.v[j].x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&blk.v[j].y));
      vf[0] = a.x, vf[1] = a.y, vf[2] = b.x, vf[3] = b.y;
    } else {
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&blk.v[j].x));
      vf[0] = a.x, vf[1] = a.y;
    }
    const bool live = j < ntok;  // tokens past the sequence end contribute nothing
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float pj = __shfl_sync(0xffffffffu, p[g], j);
#pragma unroll
      for (int d = 0; d < PV; ++d) acc[g][d] = live ? fmaf(pj, vf[d], acc[g][d]) : acc[g][d];
    }
  }
}

// tid: 0 .. 32*W-1 within the team.
// `pages`: the sequence's page list, or nullptr when the sequence owns page `seq_page` alone (the code
// predictor's per-frame KV). `len` keys. `out`: G heads of D, contiguous.
// Warps take pages round-robin (block load and page step above). Ends with a team barrier (sh may be reused).
// `stage` (optional): the warp's staging slots; the blocks then come through bulk copies, S of them ahead, and the
// arithmetic reads the same bytes from shared memory in the same order (results are bit-identical).
template <int D, int G, int W = kAttnWarps, typename TeamSync, typename Stage = NoStage>
__device__ __forceinline__ void attend_pages(AttnShared<D, G, W>& sh, const bf16* __restrict__ kv,
                                             const int32_t* __restrict__ pages, int seq_page, int len, int hk, int kh,
                                             float scale, bf16* __restrict__ out, int tid, const TeamSync& team,
                                             Stage* stage = nullptr) {
  constexpr int PV = D / 32;   // output dims per lane
  constexpr int S = Stage::kSlots;
  const int lane = tid & 31, warp = tid >> 5;
  float m[G], l[G], acc[G][PV];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < PV; ++d) acc[g][d] = 0.f;
  }
  const int npages = (len + 15) >> 4;
  auto issue = [&](int s, int pi) {  // one lane: block `pi` of the sequence into slot s
    if constexpr (S > 0) {
      const int64_t page = pages ? pages[pi] : seq_page;
      const uint32_t bar = sm100::smem_addr(stage->bars + s);
      sm100::mbar_expect_tx(bar, kv_block_bytes<D>());
      sm100::bulk_load(sm100::smem_addr(stage->slots + s * kv_block_bytes<D>()), kv + kv_offset<D>(page, hk, kh, 0, 0),
                       kv_block_bytes<D>(), bar);
    }
  };
  if constexpr (S > 0) {
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < S; ++s)
        if (warp + s * W < npages) issue(s, warp + s * W);
    }
  }
  int turn = 0;
  for (int pi = warp; pi < npages; pi += W, ++turn) {
    const int ntok = min(16, len - pi * 16);
    KvBlock<D> blk;
    if constexpr (S > 0) {
      const int s = turn % S;
      sm100::mbar_wait(sm100::smem_addr(stage->bars + s), stage->par >> s & 1u, stage->err);
      stage->par ^= 1u << s;
      blk.load(reinterpret_cast<const bf16*>(stage->slots + s * kv_block_bytes<D>()), lane);
      __syncwarp();  // the block is in registers: its slot takes the block S turns ahead
      if (lane == 0 && pi + S * W < npages) issue(s, pi + S * W);
    } else {
      const int64_t page = pages ? pages[pi] : seq_page;
      blk.load(kv + kv_offset<D>(page, hk, kh, 0, 0), lane);
    }
    page_update<D, G>(blk, sh.qs, ntok, scale, lane, m, l, acc);
  }
  if constexpr (W == 1) {
    // the merge below would multiply by exp(0) = 1: the same quotient, straight from the registers
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int d = 0; d < PV; ++d) out[(int64_t)g * D + lane * PV + d] = __float2bfloat16(acc[g][d] / l[g]);
    team.sync();
    return;
  } else {
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      sh.ms[warp][g] = m[g];
      sh.ls[warp][g] = l[g];
    }
#pragma unroll
    for (int d = 0; d < PV; ++d) sh.os[warp][g][lane * PV + d] = acc[g][d];
  }
  team.sync();
  for (int i = tid; i < G * D; i += W * 32) {
    const int g = i / D, d = i % D;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < W; ++w) top = fmaxf(top, sh.ms[w][g]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const float e = __expf(sh.ms[w][g] - top);
      num += sh.os[w][g][d] * e;
      den += sh.ls[w][g] * e;
    }
    out[(int64_t)g * D + d] = __float2bfloat16(num / den);
  }
  team.sync();
  }
}

}  // namespace omni
