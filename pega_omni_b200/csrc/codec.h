// The streaming codec decoder's device code: the causal-conv GEMM (codec_gemm.cu) and the glue kernels around it
// (codec_kernels.cu). Activations are bf16 [rows, C] with row (s, t) = frame row t of stream s at s * T + t; a conv with
// history reads a padded copy [s][H + T][C] whose first H rows per stream are the rows before the frame.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "util.cuh"

namespace omni {

// What the conv GEMM does with its f32 accumulator a:
//   kConvStore:      y = bf16(a)
//   kConvAccumulate: y = bf16(y + a)                      (one rounding of the f32 sum)
//   kConvBiasSnake:  t = bf16(a) + bias[n]; y = bf16(t + inv_b[n] * sin^2(alpha[n] * t))
enum ConvEpilogue : int { kConvStore = 0, kConvAccumulate = 1, kConvBiasSnake = 2 };

// y[s * T + t, n] = sum over taps j and channels c of x[s][t + j * dil][c] * w[n][j * C + c]: a causal conv of `taps`
// taps as an implicit GEMM. x is the padded activation [seqs][P][C], P = (taps - 1) * dil + T (taps = 1: the dense
// activation itself); w is [N, taps * C], tap-major. A CTA computes 128 output rows (SB streams x TB rows, TB the
// largest power of two dividing T, at most 128) by tn output channels over all taps and channels: for every tap, TMA
// boxes of the padded activation shifted by j * dil rows land as K-major tiles next to the matching weight columns.
struct ConvGemmPlan {
  CUtensorMap xmap, wmap;
  int N = 0, C = 0, taps = 1, dil = 1, T = 1, seqs = 1;
  int TB = 1, SB = 128, tn = 16, kbs = 1, cpb = 1, ragged = 0, stages = 2;
  int n_tiles = 1, row_tiles = 1, ctas = 1;
  bf16* y = nullptr;
  int kind = kConvStore;
  const bf16* bias = nullptr;
  const float *alpha = nullptr, *inv_b = nullptr;
};

void conv_configure();
int conv_plan(ConvGemmPlan* plan, const bf16* w, int N, int C, int taps, int dil, const bf16* x, int T, int seqs, bf16* y,
              int kind, const bf16* bias, const float* alpha, const float* inv_b, int sm_count);
cudaError_t conv_launch(const ConvGemmPlan& plan, uint32_t* err, cudaStream_t stream);

// SnakeBeta with the sine taken by the hardware approximation after a two-step reduction to [-pi, pi]
// (crates/omni-qwen3-tts/kernels/codec.cu:34-42 does the same, so the two agree bit for bit on one GPU).
__device__ __forceinline__ float snake_beta(float x, float alpha, float inv_b) {
  const float y = alpha * x;
  const float k = rintf(y * 0.159154943091895336f);
  const float s = __sinf(fmaf(-k, -1.74845553e-7f, fmaf(-k, 6.28318548202514648f, y)));
  return x + inv_b * s * s;
}

struct CodecStateRef {
  char* base;            // state of every slot
  const int32_t* lines;  // slot of each stream of the call
  const int32_t* pos;    // frames each stream has decoded before this call
  int64_t stride;        // bytes per slot
};

// ---- glue kernels (codec_kernels.cu); every launcher returns cudaGetLastError() ----------------------------------
cudaError_t launch_codec_rvq(const int32_t* codes, const bf16* books, bf16* out, int n, int half, int book_rows,
                             cudaStream_t stream);
// res += add (add_stride 0: one row for all); res stored bf16; out = bf16(v * (rsqrt(mean v^2 + eps) * w))
cudaError_t launch_codec_add_norm(const bf16* add, int64_t add_stride, bf16* res, const bf16* w, bf16* out, int rows,
                                  int dim, float eps, cudaStream_t stream);
cudaError_t launch_codec_window_attend(const bf16* qkv, CodecStateRef st, int64_t ring_offset, bf16* out, int n, int heads,
                                       float theta, cudaStream_t stream);
cudaError_t launch_codec_silu_mul(const bf16* gate_up, bf16* out, int rows, int inter, cudaStream_t stream);
cudaError_t launch_codec_bias_gelu(bf16* x, const bf16* bias, int64_t rows, int cols, cudaStream_t stream);
cudaError_t launch_codec_bias_snake(const bf16* x, const bf16* bias, const float* alpha, const float* inv_b, bf16* out,
                                    int64_t rows, int cols, cudaStream_t stream);
// padded[s][r] = r < H ? history row r : act(x[s * T + r - H] + bias); the last H rows become the next history
cudaError_t launch_codec_stage(const bf16* x, const bf16* bias, const float* alpha, const float* inv_b, CodecStateRef st,
                               int64_t hist_offset, bf16* padded, int n, int T, int C, int H, cudaStream_t stream);
// col[s * T + t][j * C + c] = padded[s][t + j * dil][c]
cudaError_t launch_codec_gather_taps(const bf16* padded, bf16* col, int n, int T, int C, int taps, int dil,
                                     cudaStream_t stream);
// transposed conv with kernel 2r, stride r: out[s][l * r + j] = bias + z[s][l][j] + z[s][l - 1][j + r]
cudaError_t launch_codec_overlap_add(const bf16* z, const bf16* bias, CodecStateRef st, int64_t prev_offset, bf16* out,
                                     int n, int L, int r, int C, cudaStream_t stream);
// x = bf16(z + zb[row % r]) kept in xin; depthwise 7-tap causal conv; LayerNorm into out
cudaError_t launch_codec_dwconv_ln(const bf16* z, const bf16* zb, const bf16* w, const bf16* b, const bf16* ln_w,
                                   const bf16* ln_b, CodecStateRef st, int64_t hist_offset, bf16* xin, bf16* out, int n,
                                   int T, int r, int C, float eps, cudaStream_t stream);
// last SnakeBeta, the C -> 1 conv of 7 taps, the clamp; wav f32 [n][T]
cudaError_t launch_codec_out_conv(const bf16* x, const bf16* bias, const float* alpha, const float* inv_b, const bf16* w,
                                  const bf16* wb, CodecStateRef st, int64_t hist_offset, float* wav, int n, int T, int C,
                                  cudaStream_t stream);

}  // namespace omni
