// Per-head RMSNorm + half-rotation rotary embedding of one q/k head held by a warp (crates/omni-qwen3/kernels/
// qwen3.cu:66-107), shared by the tick kernel and the cluster predictor kernel.
#pragma once
#include "util.cuh"

namespace omni {

// Rotation angles of this lane's E element pairs at `pos`: inv_freq = theta^(-2i/D) (qwen3.cu:94-98). The same for
// every head of a row, so computed once per row.
template <int D>
__device__ __forceinline__ void rope_angles(int lane, int pos, float theta, float (&cs)[D / 64], float (&sn)[D / 64]) {
#pragma unroll
  for (int e = 0; e < D / 64; ++e) {
    const int i = lane * (D / 64) + e;
    const float inv_freq = 1.f / powf(theta, (float)(2 * i) / D);
    sincosf((float)pos * inv_freq, &sn[e], &cs[e]);
  }
}

// q/k of one head: RMSNorm over the head, the normalised value rounded to bf16 before the gain, half-rotation
// rotary embedding (qwen3.cu:66-107). lo/hi: this lane's E elements of each half; wl/wh: the gains of those elements.
template <int D>
__device__ __forceinline__ void rope_head(float (&lo)[D / 64], float (&hi)[D / 64], const float (&wl)[D / 64],
                                          const float (&wh)[D / 64], const float (&cs)[D / 64],
                                          const float (&sn)[D / 64], float eps) {
  constexpr int E = D / 64;
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < E; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
  const float rn = rsqrtf(warp_add(ss) / D + eps);
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const float a = bf16_round(lo[e] * rn) * wl[e];
    const float b = bf16_round(hi[e] * rn) * wh[e];
    lo[e] = bf16_round(a * cs[e] - b * sn[e]);
    hi[e] = bf16_round(b * cs[e] + a * sn[e]);
  }
}

}  // namespace omni
