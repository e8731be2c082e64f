// The code predictor's fifteen sub-steps of a decode tick as ONE launch of thread-block clusters
// (`Talker::tail` after the first draw: crates/omni-qwen3-tts/src/talker.rs:300-356; op order of a pass:
// crates/omni-qwen3/src/stack.rs:152-241).
//
// Why clusters. A predictor pass is ~40 dependent steps over a few megabytes of weights each; split over all 148 SMs
// every step pays a grid-wide hand-over (store -> barrier -> load through L2, 2-3 us), which is most of its time.
// Sessions are independent, so here they are dealt to clusters of C CTAs (C = the predictor's query heads, 16 at the
// headline shape) that never talk to one another: a cluster runs all sub-steps for its (at most 16) sessions, every
// matrix split C ways by output rows with the whole K per CTA, so a step's hand-over is a cluster barrier (an
// mbarrier in each CTA's shared memory, arrived on by one thread of every peer) around a few KB in L2. Every cluster
// streams every weight byte (from L2 after the first cluster pulled it from HBM).
//
// What was measured on B200 (64 sessions, 7 resident clusters of 16): the launch takes 6.1 ms against 3.9 ms for the
// same sub-steps inside the persistent tick kernel, so the tick kernel stays the default and this one is an option.
// A CTA consumes its weight stream at 48 GB/s (a 128 x 1024 box in 5.3 us), not the 114 GB/s its TMA unit can
// deliver: 64 tcgen05.mma (M = 128, N = 16) take 5.3 us whether they accumulate into one TMEM accumulator or
// alternate between two, and with the MMAs left out the same loop streams the box in 2.0 us. (mma.sync m16n8k16
// from the same stages: 7.6 us.) Eight-fold re-reading of the weights needs the full ingest rate; a hand-over
// through a cluster barrier (1.5-2 us with the L2 round trip of the exchanged rows) is not cheap enough to pay for it.
//
// Per CTA: one weight producer thread (TMA into a ring of 40 KB stages, free-running over the whole launch, with an
// L2 prefetch of its boxes about 1 MB ahead), one activation producer thread (TMA of activation k-blocks that another
// CTA wrote, gated by the cluster barrier), eight consumer warps: thread 0 issues tcgen05.mma with the weight rows
// on M (128 or 64) and the cluster's 16 session rows on N, accumulator in TMEM; all eight read it back and run the
// epilogues, norms, attention and draws. Work is a flat list of entries (one weight box of 64 or 128 rows each)
// compiled once per bucket by the host, as the tick kernel's phase list is.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "tick.h"
#include "util.cuh"

namespace omni {

constexpr int kPredRows = 16;  // activation rows (sessions) a cluster holds: two n8 MMA tiles

enum PredEpilogue : int32_t {
  kPeBiasNorm = 0,  // mtp projection: + bias, residual start, (barrier) RMSNorm into the resident activation tile
  kPeQ = 1,         // a query head: head RMSNorm + RoPE into shared memory
  kPeKv = 2,        // even rank: the key head (norm + RoPE), odd rank: the value head; KV write, (barrier) attention, (barrier)
  kPeAddNorm = 3,   // o / down projection: residual add, (barrier) RMSNorm into the resident activation tile
  kPeSwiglu = 4,    // a box of gate|up rows: SiLU(gate) * up; barrier after the CTA's last box
  kPeHead = 5,      // a box of vocabulary rows: logits; after the last box (barrier) draw + next input (barrier)
};

// One box of weight rows x the whole K, for every CTA of every cluster.
struct alignas(16) PredEntry {
  int32_t epi;
  int32_t wmap;        // tensor map of the weight matrix: {64 elements, rows, k-blocks}, box {64, rows, kbs}
  int32_t wrow;        // first weight row of rank 0's box; rank r reads wrow + r * cta_stride (kPeKv: see wrow2)
  int32_t wrow2;       // kPeKv: first row of the value heads (wrow: of the key heads); head index = rank / 2
  int32_t cta_stride;  // weight rows between the boxes of consecutive ranks
  int32_t rows;        // box rows: 64 or 128
  int32_t nkb, kbs;    // K / 64 and k-blocks per ring stage
  int32_t xmap;        // >= 0: the activation operand comes through TMA from this map (rows = sessions); -1: resident tile
  int32_t xz0;         // first k-block inside the map (the talker's hidden / code embedding halves of p_in)
  int32_t need_bars;   // cluster barriers that must have completed before the activation operand may be loaded
  int32_t last;        // 1: the CTA's last box of this matrix (the barrier / draw follows)
  int32_t pos;         // position of the sub-step's row in the per-frame sequence (0 .. 15)
  int32_t group;       // codebook the head draws (kPeHead)
  int32_t col0;        // output column of rank 0's first row (kPeHead: vocabulary index; kPeSwiglu: unused)
  int32_t next_dim;    // kPeHead: elements of the next input row (0: no next sub-step)
  float eps, theta;
  int32_t pad_[2];
  const void* w;        // the weight matrix (row-major, K contiguous: a box of whole rows is one contiguous range)
  const void *p0, *p1;  // BiasNorm: bias, gain; Q/Kv: norm gain, -; AddNorm: -, gain; Head: next-input table, -
  void *q0, *q1;        // Kv: KV layer, attention out; Swiglu: act; Head: logits out (row stride = vocab), next-input rows
};

struct PredConfig {
  int32_t C;           // CTAs per cluster = query heads
  int32_t hidden;      // predictor hidden (64 * C)
  int32_t q_heads, kv_heads, inter, granule, vocab;
  int32_t next_stride;  // elements between the next-input rows of consecutive sessions
  float temperature, top_p;
  int32_t top_k, philox;
};

struct PredProgram {
  std::vector<PredEntry> entries;
  std::vector<CUtensorMap> maps;
  PredConfig cfg{};
  int rows = 0;          // sessions (bucket)
  int per_cluster = 0;   // sessions per cluster
  int clusters = 0;
  int stage_bytes = 0, stages = 0;
  PredEntry* d_entries = nullptr;
  CUtensorMap* d_maps = nullptr;
};

// Appends the {64, rows, K/64} map of a K-major bf16 matrix with a box of {64, box_rows, kbs}; row_stride in elements.
int pred_add_map(PredProgram* prog, const bf16* base, int64_t rows, int K, int64_t row_stride, int box_rows, int kbs);
// Clusters of C CTAs that can be resident at once (0: the device cannot run this kernel with that cluster size).
int pred_configure(int C);
int pred_upload(PredProgram* prog);
void pred_free(PredProgram* prog);
// One launch: prog.clusters clusters of C CTAs. `vbuf`: rows x hidden floats of exchange space. `trace` (optional,
// three u64 per entry): the global timer when rank 0 of cluster 0 started the entry, left its main loop, finished it.
cudaError_t pred_launch(const PredProgram& prog, const TickIo& io, float* vbuf, uint32_t* err, cudaStream_t stream,
                        unsigned long long* trace = nullptr);

}  // namespace omni
