// The persistent tick kernel: one cooperative launch runs a whole graph program (the talker pass, the
// codec head, and the fifteen code-predictor sub-steps with their heads and draws) as a list of phases
// separated by grid-wide barriers. The host compiles the list once per (program, batch bucket), the way
// the reference compiles its manifest call list (crates/omni-qwen3-tts/src/model.rs:335-342); the kernel
// interprets it. Weight tiles keep streaming across phase boundaries: the weight producer of every CTA
// runs ahead of the barriers (weights do not depend on activations), only the activation tiles wait.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "util.cuh"

namespace omni {

enum PhaseType : int32_t {
  kPhGemm = 0,        // W tiles x activation rows -> f32 partial tiles (or SwiGLU activations)
  kPhEmbedNorm = 1,   // talker input: frame embedding from the slot, residual start, RMSNorm
  kPhReduceNorm = 2,  // predictor input: reduce partials (+ bias), residual start, RMSNorm
  kPhAddNorm = 3,     // reduce partials, residual add, RMSNorm (strided keep on the last layer)
  kPhRopeAttn = 4,    // reduce qkv partials, q/k norm + RoPE, KV write, attention
  kPhSample = 5,      // reduce logits partials, draw, next predictor input
  kPhReduceSilu = 6,  // reduce gate|up partials -> SwiGLU activations (when the gate|up GEMM is split along K)
};

enum GemmMode : int32_t { kGemmPartials = 0, kGemmSwiglu = 1 };
enum NextInput : int32_t { kNextNone = 0, kNextHiddenAndCode = 1, kNextCode = 2, kNextProjected = 3 };

// One phase. Field use by type:
//  Gemm:       N, K, bn, rows, tiles, splits, wmap, xmap, mode; dst0 = act (SwiGLU), i0 = inter, i1 = k-blocks per
//              ring stage (one TMA copy each for the activations and the weights)
//  EmbedNorm:  rows, dim = N; src0 pad, src1 codec_emb, src2 p_emb, src3 gain; dst0 res, dst1 x; i0 vocab, i1 p_vocab,
//              i2 groups; f0 eps
//  ReduceNorm: rows, dim = N, tiles, splits, bn; src0 bias (or null), src3 gain; dst0 res, dst1 x; f0 eps
//  AddNorm:    rows, dim = N, tiles, splits, bn; src3 gain; dst0 res, dst1 out; i0 every, i1 which; f0 eps
//  RopeAttn:   rows, tiles, splits, bn; i0 hq, i1 hk, i2 head_dim, i3 per, i4 base, i5 paged, i6 kv_pages;
//              src0 q_norm, src1 k_norm; dst0 kv layer, dst1 attn out; f0 eps, f1 theta
//  RopeAttn (one-page sequences only): src2 != nullptr: the rows' q | k | v are rows of the table at src2 (bf16, i8
//              elements per row), row = the code of group i7 drawn for the sequence; no partial tiles are read
//  ReduceSilu: rows, tiles, splits, bn; dst0 act; i0 inter
//  Sample:     rows, tiles, splits, bn, N = vocab; dst0 logits out, i0 ldl (row stride of logits out, elements);
//              sampling constants in f0..f3 / i1..i7; next-input in i8, src0 table, src1 hidden, dst1 p_in, i9 dim;
//              i8 = kNextProjected: src0 is the table of code embeddings ALREADY sent through the predictor's input
//              projection (one row of i9 elements per code), so the drawn code's row is the next pass's residual
//              start: dst1 residual rows, dst2 normed rows, src3 the first layer's norm gain, f3 its eps
struct alignas(16) Phase {
  int32_t type, rows, bn, N, K, tiles, splits, wmap, xmap, mode, cta_offset, tile_n;  // tile_n: weight rows per GEMM tile (64, 128 or 256; 96 with the SwiGLU epilogue)
  int32_t i0, i1, i2, i3, i4, i5, i6, i7, i8, i9, i10, i11;
  float f0, f1, f2, f3;
  const void *src0, *src1, *src2, *src3;
  void *dst0, *dst1, *dst2;
};

// Pointers every phase may need (the staged inputs of the call and the per-sequence state).
struct TickIo {
  const int32_t* lines;
  const int32_t* frames;  // frame index of each row (`pos` input)
  const float* uniforms;
  const int32_t* force;
  const int32_t* d_pos;
  const int32_t* d_slot;
  const int32_t* indptr;
  const int32_t* pages;
  void* state;
  int64_t stride;
  int32_t* codes;
  int32_t seen_words;
};

struct TickProgram {
  std::vector<Phase> phases;
  std::vector<CUtensorMap> maps;
  int max_bn = 16;
  size_t partial_floats = 0;
  // device copies
  Phase* d_phases = nullptr;
  CUtensorMap* d_maps = nullptr;
};

// Appends a K-major bf16 tensor map ([rows, K] with a box of box_rows rows x kbs k-blocks of 64) and returns its index.
int tick_add_map(TickProgram* prog, const bf16* base, int rows, int K, int box_rows, int kbs);
// Bytes of shared memory the kernel's tile ring takes (what a GEMM phase's stages must fit).
int tick_ring_size();
// Largest SwiGLU/partials GEMM the kernel can run; false when a shape needs the per-op path.
bool tick_supports(int hidden, int head_dim, int q_heads, int kv_heads, int rows_max);
// Copies the phase list and the maps to the device. 0 on success.
int tick_upload(TickProgram* prog);
void tick_free(TickProgram* prog);
// Raises the kernel's shared-memory limit and reports how many CTAs can be co-resident (0 on failure).
int tick_configure(int device);
// One cooperative launch of the whole program. `barrier` is one device u32, zero before the first launch;
// `*barrier_base` (host, starts at 0) tracks the arrivals earlier launches left in it. Set *barrier_base = ~0u after a
// launch that raised the error word (its CTAs may not all have arrived): the next launch then restarts the counter.
// `trace` (optional, four u64 per (phase, CTA), phase-major): the global timer when the CTA's first activation tile
// of the phase arrived, when its first accumulator was complete (both GEMM phases only), when its own share of
// the phase was done, and when it saw the phase's grid barrier complete.
cudaError_t tick_launch(const TickProgram& prog, const TickIo& io, float* partials, uint32_t* barrier,
                        uint32_t* barrier_base, uint32_t* err, int ctas, cudaStream_t stream,
                        unsigned long long* trace = nullptr);

}  // namespace omni
