// y[rows, N] = bf16( x[rows, K] . w[N, K]^T ) with f32 accumulation: the one
// GEMM shape the token loop uses (all operands bf16 row-major, weights [N, K]).
// Two device paths, chosen by the caller from the row count:
//   - gemv:  CUDA-core vector kernel, HBM-bound while the row count is small;
//   - tc:    tcgen05 tensor-core tiles with the weights on the MMA M dimension
//            (128 weight rows per tile) and the rows (sessions) on N, TMA-fed,
//            split along K so enough CTAs stream weights to fill the machine.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "util.cuh"

namespace omni {

// What happens to the f32 accumulator a after its rounding to bf16:
//   kEpiNone:     y = bf16(a)
//   kEpiBias:     y = bf16(bf16(a) + bias[n])
//   kEpiBiasSilu: t = bf16(bf16(a) + bias[n]); y = bf16(t / (1 + exp(-t)))
enum EpilogueKind : int { kEpiNone = 0, kEpiBias = 1, kEpiBiasSilu = 2 };

struct Epilogue {
  const bf16* bias = nullptr;
  int kind = kEpiNone;
};

// Scratch for split-K: per-split f32 partial tiles and one arrival counter per
// output tile (zero between launches; the last CTA of a tile resets its counter).
struct GemmScratch {
  float* partials = nullptr;
  size_t partial_floats = 0;
  uint32_t* counters = nullptr;
  int counter_slots = 0;
};

struct TcGemmPlan {
  CUtensorMap wmap, xmap;
  int N = 0, K = 0, rows = 0;
  int BN = 0;        // rows (sessions) per tile: 16..256, multiple of 16
  int row_tiles = 1; // ceil(rows / BN)
  int splits = 1;
  int kbs = 1;       // k-blocks per ring stage and per TMA copy
  bf16* y = nullptr;
  int ldy = 0;
  Epilogue epi;
  size_t partial_floats() const { return splits > 1 ? (size_t)splits * row_tiles * tiles_n() * 128 * BN : 0; }
  int tiles_n() const { return (N + 127) / 128; }  // partial_floats() matches the kernel's [row_tile][split][tile][BN][128]
};

// Raises the shared-memory limits of the GEMM kernels; call once per process before any launch.
void tc_configure();
// Resolves the driver entry point used to encode tensor maps. 0 on success.
int tc_init();
// Encodes a bf16 tensor map of rank <= 5 with the 128-byte swizzle; strides (bytes) for dimensions 1..rank-1. 0 on success.
int tc_encode_bf16(CUtensorMap* map, const bf16* base, int rank, const uint64_t* dims, const uint64_t* strides,
                   const uint32_t* box);
// Whether a GEMM of this shape can run on the tensor-core path.
bool tc_supports(int N, int K, int rows);
// Encodes the tensor maps and picks the tiling. x is [rows, K] dense, w is [N, K] dense.
int tc_plan(TcGemmPlan* plan, const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy, Epilogue epi,
            int sm_count, int force_splits = 0);
cudaError_t tc_launch(const TcGemmPlan& plan, const GemmScratch& scratch, uint32_t* err, cudaStream_t stream);

// The tensor-core path with the input rows on the MMA M dimension (rows <= 128, K <= 4096): one CTA per tile of TN
// weight rows over the whole K, no split and no reduction. For decode-sized GEMMs with small weight matrices.
struct RmGemmPlan {
  CUtensorMap wmap, xmap;
  int N = 0, K = 0, rows = 0, TN = 64, kbs = 1, bn = 128;  // TN weight rows per CTA, kbs k-blocks per TMA copy, bn rows per activation box
  bf16* y = nullptr;
  int ldy = 0;
  Epilogue epi;
};
bool rm_supports(int N, int K, int rows);
int rm_plan(RmGemmPlan* plan, const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy, Epilogue epi,
            int sm_count);
cudaError_t rm_launch(const RmGemmPlan& plan, uint32_t* err, cudaStream_t stream);

cudaError_t gemv_launch(const bf16* w, int N, int K, const bf16* x, int rows, bf16* y, int ldy, Epilogue epi,
                        int sm_count, cudaStream_t stream);

}  // namespace omni
