// Glue kernels of the streaming codec decoder (declared in codec.h). The arithmetic and every rounding point follow
// the reference's kernels (crates/omni-qwen3-tts/kernels/codec.cu:66-513), whose results these must reproduce; the
// decomposition into kernels does not: there is no im2col (the conv GEMM reads the padded activation directly, so the
// staging kernel writes each transformed row once instead of once per tap), the second SnakeBeta of a residual unit
// lives in the conv GEMM's epilogue, and the waveform leaves the last kernel as f32.
//
// Per-stream state (one slot per stream, zeroed when the stream opens; offsets are fixed at create):
//   conv history .... [2][H][C] bf16: frame p reads half p & 1 and writes the next frame's rows into the other half, so
//                     a launch never overwrites rows another of its threads still reads;
//   overlap rows .... [rate][C] bf16: taps rate.. of the last GEMM row of a transposed conv;
//   attention ring .. K[72][heads * 64] then V, frame p at p % 72.
#include <algorithm>

#include "codec.h"

namespace omni {

namespace {

constexpr int kHeadDim = 64, kWindow = 72, kTaps = 7;

__device__ __forceinline__ bf16* slot_ptr(const CodecStateRef& st, int s, int64_t offset) {
  return reinterpret_cast<bf16*>(st.base + (int64_t)st.lines[s] * st.stride + offset);
}

__device__ __forceinline__ void ldf8(const float* p, float* v) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}

// One stream per block: [codebook 0 | sum of codebooks 1..15], the sum in f32 in codebook order.
__global__ void codec_rvq_kernel(const int32_t* __restrict__ codes, const bf16* __restrict__ books, bf16* __restrict__ out,
                                 int half, int book_rows) {
  const int s = blockIdx.x;
  for (int c = threadIdx.x * 8; c < half; c += blockDim.x * 8) {
    const int32_t* code = codes + s * 16;
    const int64_t first = code[0] < book_rows ? code[0] : 0;  // a code past the book (end of speech) reads as 0
    *reinterpret_cast<uint4*>(out + (int64_t)s * 2 * half + c) = *reinterpret_cast<const uint4*>(books + first * half + c);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int g = 1; g < 16; ++g) {
      float v[8];
      ld8v(books + ((int64_t)g * book_rows + code[g]) * half + c, v);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += v[k];
    }
    st8v(out + (int64_t)s * 2 * half + half + c, acc);
  }
}

// A warp per row, dim a multiple of 256 up to 1024.
__global__ void codec_add_norm_kernel(const bf16* add, int64_t add_stride, bf16* __restrict__ res,
                                      const bf16* __restrict__ w, bf16* out, int rows, int dim, float eps) {  // out may be add
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const bf16* a = add + r * add_stride;
  bf16* rr = res + (int64_t)r * dim;
  float v[4][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = (k * 32 + lane) * 8;
    if (c < dim) {
      float x[8];
      ld8v(a + c, x);
      ld8v(rr + c, v[k]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[k][e] += x[e];
        ss += v[k][e] * v[k][e];
      }
      st8v(rr + c, v[k]);
    }
  }
  const float rs = rsqrtf(warp_add(ss) / dim + eps);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int c = (k * 32 + lane) * 8;
    if (c < dim) {
      float g[8];
      ld8v(w + c, g);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[k][e] *= rs * g[e];
      st8v(out + (int64_t)r * dim + c, v[k]);
    }
  }
}

// A warp per (stream, head): rotary embedding of q and k (a lane holds dims lane and lane + 32, the pair one rotation
// mixes), k and v into the ring, then q against the last min(p + 1, 72) frames: a lane scores whole frames (its q copy
// comes from shared memory), the softmax runs across lanes, and for the weighted sum of V a lane owns two dims.
__global__ void __launch_bounds__(128)
    codec_window_attend_kernel(const bf16* __restrict__ qkv, CodecStateRef st, int64_t ring_offset, bf16* __restrict__ out,
                               int heads, float theta) {
  __shared__ float sq[4][kHeadDim];
  __shared__ float sp[4][kWindow + 8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.x, head = blockIdx.y * 4 + warp;
  if (head >= heads) return;
  const int width = heads * kHeadDim;
  const bf16* row = qkv + (int64_t)s * 3 * width + head * kHeadDim;
  bf16* ring = slot_ptr(st, s, ring_offset);
  const int p = st.pos[s];
  const int n = min(p + 1, kWindow), first = p - n + 1;
  const int64_t v_ofs = (int64_t)kWindow * width;
  const float inv_freq = 1.f / powf(theta, (float)(2 * lane) / kHeadDim);
  float sn, cs;
  sincosf((float)p * inv_freq, &sn, &cs);
  const float q_lo = __bfloat162float(row[lane]), q_hi = __bfloat162float(row[lane + 32]);
  const float k_lo = __bfloat162float(row[width + lane]), k_hi = __bfloat162float(row[width + lane + 32]);
  const bf16 ka = __float2bfloat16(k_lo * cs - k_hi * sn), kb = __float2bfloat16(k_hi * cs + k_lo * sn);
  sq[warp][lane] = bf16_round(q_lo * cs - q_hi * sn);
  sq[warp][lane + 32] = bf16_round(q_hi * cs + q_lo * sn);
  bf16* at = ring + (int64_t)(p % kWindow) * width + head * kHeadDim;
  at[lane] = ka;
  at[lane + 32] = kb;
  reinterpret_cast<uint32_t*>(at + v_ofs)[lane] = reinterpret_cast<const uint32_t*>(row + 2 * width)[lane];
  __syncwarp();  // the ring rows of this (stream, head) are written and read by this warp alone
  float mx = -INFINITY;
  for (int j = lane; j < n; j += 32) {
    const uint4* kr = reinterpret_cast<const uint4*>(ring + (int64_t)((first + j) % kWindow) * width + head * kHeadDim);
    float dot = 0.f;
#pragma unroll
    for (int q8 = 0; q8 < 8; ++q8) {
      float kv[8];
      unpack8v(kr[q8], kv);
#pragma unroll
      for (int e = 0; e < 8; ++e) dot += sq[warp][q8 * 8 + e] * kv[e];
    }
    dot *= 0.125f;  // 1 / sqrt(64)
    sp[warp][j] = dot;
    mx = fmaxf(mx, dot);
  }
  mx = warp_fmax(mx);
  float l = 0.f;
  for (int j = lane; j < n; j += 32) {
    const float e = __expf(sp[warp][j] - mx);
    sp[warp][j] = e;
    l += e;
  }
  l = warp_add(l);
  __syncwarp();
  float o0 = 0.f, o1 = 0.f;
  for (int j = 0; j < n; ++j) {
    const __nv_bfloat162 v2 = reinterpret_cast<const __nv_bfloat162*>(
        ring + v_ofs + (int64_t)((first + j) % kWindow) * width + head * kHeadDim)[lane];
    const float pj = sp[warp][j];
    o0 += pj * __low2float(v2);
    o1 += pj * __high2float(v2);
  }
  reinterpret_cast<__nv_bfloat162*>(out + (int64_t)s * width + head * kHeadDim)[lane] =
      __floats2bfloat162_rn(o0 / l, o1 / l);
}

__global__ void codec_silu_mul_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int inter, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int per = inter / 8;
  const int64_t r = i / per, c = i % per * 8;
  float g[8], u[8];
  ld8v(gate_up + r * 2 * inter + c, g);
  ld8v(gate_up + r * 2 * inter + inter + c, u);
#pragma unroll
  for (int k = 0; k < 8; ++k) g[k] = bf16_round(g[k] / (1.f + __expf(-g[k]))) * u[k];
  st8v(out + i * 8, g);
}

__global__ void codec_bias_gelu_kernel(bf16* __restrict__ x, const bf16* __restrict__ bias, int cols, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v[8], b[8];
  ld8v(x + i * 8, v);
  ld8v(bias + i % (cols / 8) * 8, b);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float y = bf16_round(v[k] + b[k]);
    v[k] = 0.5f * y * (1.f + erff(y * 0.70710678118654752f));
  }
  st8v(x + i * 8, v);
}

__device__ __forceinline__ void bias_snake8(float* v, const bf16* bias, const float* alpha, const float* inv_b, int c) {
  float b[8], al[8], ib[8];
  ld8v(bias + c, b);
  ldf8(alpha + c, al);
  ldf8(inv_b + c, ib);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = snake_beta(v[k] + b[k], al[k], ib[k]);
}

__global__ void codec_bias_snake_kernel(const bf16* __restrict__ x, const bf16* __restrict__ bias,
                                        const float* __restrict__ alpha, const float* __restrict__ inv_b,
                                        bf16* __restrict__ out, int cols, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float v[8];
  ld8v(x + i * 8, v);
  bias_snake8(v, bias, alpha, inv_b, (int)(i % (cols / 8)) * 8);
  st8v(out + i * 8, v);
}

// One thread per eight channels of a padded row: rows below H come from the history, the rest are the transformed
// frame; whatever lands in the last H rows is also the next frame's history.
__global__ void codec_stage_kernel(const bf16* __restrict__ x, const bf16* __restrict__ bias, const float* __restrict__ alpha,
                                   const float* __restrict__ inv_b, CodecStateRef st, int64_t hist_offset,
                                   bf16* __restrict__ padded, int T, int C, int H, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int per = C / 8, P = H + T;
  const int c = (int)(i % per) * 8;
  const int64_t g = i / per;
  const int s = (int)(g / P), r = (int)(g % P);
  const int p = st.pos[s];
  bf16* hist = slot_ptr(st, s, hist_offset);
  const int64_t half = (int64_t)H * C;
  uint4 u;
  if (r < H) {
    u = *reinterpret_cast<const uint4*>(hist + (p & 1) * half + (int64_t)r * C + c);
  } else {
    float v[8];
    ld8v(x + ((int64_t)s * T + r - H) * C + c, v);
    if (alpha != nullptr) {
      bias_snake8(v, bias, alpha, inv_b, c);
    } else {
      float b[8];
      ld8v(bias + c, b);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] += b[k];
    }
    u = pack8v(v);
  }
  *reinterpret_cast<uint4*>(padded + ((int64_t)s * P + r) * C + c) = u;
  if (r >= T) *reinterpret_cast<uint4*>(hist + ((p + 1) & 1) * half + (int64_t)(r - T) * C + c) = u;
}

__global__ void codec_gather_taps_kernel(const bf16* __restrict__ padded, bf16* __restrict__ col, int T, int C, int taps,
                                         int dil, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int per = C / 8, P = (taps - 1) * dil + T;
  const int c = (int)(i % per) * 8;
  int64_t g = i / per;
  const int j = (int)(g % taps);
  g /= taps;
  const int t = (int)(g % T), s = (int)(g / T);
  *reinterpret_cast<uint4*>(col + (((int64_t)s * T + t) * taps + j) * C + c) =
      *reinterpret_cast<const uint4*>(padded + ((int64_t)s * P + t + j * dil) * C + c);
}

__global__ void codec_overlap_add_kernel(const bf16* __restrict__ z, const bf16* __restrict__ bias, CodecStateRef st,
                                         int64_t prev_offset, bf16* __restrict__ out, int L, int r, int C, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int per = C / 8;
  const int c = (int)(i % per) * 8;
  const int64_t g = i / per;
  const int s = (int)(g / (L * r)), t = (int)(g % (L * r));
  const int l = t / r, j = t % r;
  const int64_t w = (int64_t)2 * r * C;
  const bf16* zs = z + (int64_t)s * L * w;
  float v[8], y[8];
  ld8v(bias + c, v);
  ld8v(zs + l * w + (int64_t)j * C + c, y);
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] += y[k];
  if (l > 0) {
    ld8v(zs + (l - 1) * w + (int64_t)(j + r) * C + c, y);
  } else {  // the row before the frame's first: kept from the last call; this thread alone touches the entry
    bf16* prev = slot_ptr(st, s, prev_offset) + (int64_t)j * C + c;
    ld8v(prev, y);
    *reinterpret_cast<uint4*>(prev) = *reinterpret_cast<const uint4*>(zs + (L - 1) * w + (int64_t)(j + r) * C + c);
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] += y[k];
  st8v(out + i * 8, v);
}

// One block per row, eight channels per thread; the block is a whole number of warps, threads past the last channel
// only take part in the two block-wide sums.
__global__ void codec_dwconv_ln_kernel(const bf16* __restrict__ z, const bf16* __restrict__ zb, const bf16* __restrict__ w,
                                       const bf16* __restrict__ b, const bf16* __restrict__ ln_w,
                                       const bf16* __restrict__ ln_b, CodecStateRef st, int64_t hist_offset,
                                       bf16* __restrict__ xin, bf16* __restrict__ out, int T, int r, int C, float eps) {
  constexpr int H = kTaps - 1;
  __shared__ float scratch[32];
  const int64_t g = blockIdx.x;
  const int s = (int)(g / T), t = (int)(g % T), c = threadIdx.x * 8;
  const bool on = c < C;
  const int p = st.pos[s];
  bf16* hist = slot_ptr(st, s, hist_offset);
  const bf16* old = hist + (p & 1) * (int64_t)H * C;
  bf16* next = hist + ((p + 1) & 1) * (int64_t)H * C;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, cur[8];
  if (on) {
    ld8v(b + c, acc);
#pragma unroll
    for (int j = 0; j < kTaps; ++j) {
      const int src = t - (H - j);
      float v[8], wt[8];
      if (src >= 0) {
        float bias[8];
        ld8v(z + ((int64_t)s * T + src) * C + c, v);
        ld8v(zb + (int64_t)(src % r) * C + c, bias);
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = bf16_round(v[k] + bias[k]);
      } else {
        ld8v(old + (int64_t)(H + src) * C + c, v);
      }
      ld8v(w + (int64_t)j * C + c, wt);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        acc[k] += wt[k] * v[k];
        cur[k] = v[k];
      }
    }
    st8v(xin + g * C + c, cur);
    if (t + H - T >= 0) st8v(next + (int64_t)(t + H - T) * C + c, cur);
    // with fewer rows per frame than the history holds, the old history's tail moves up
    for (int m = t; m < H - T; m += T)
      *reinterpret_cast<uint4*>(next + (int64_t)m * C + c) = *reinterpret_cast<const uint4*>(old + (int64_t)(m + T) * C + c);
  }
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    acc[k] = bf16_round(acc[k]);
    sum += acc[k];
  }
  const float mean = block_add(sum, scratch) / C;
  float sq = 0.f;
  if (on) {
#pragma unroll
    for (int k = 0; k < 8; ++k) sq += (acc[k] - mean) * (acc[k] - mean);
  }
  const float rstd = rsqrtf(block_add(sq, scratch) / C + eps);
  if (on) {
    float lw[8], lb[8];
    ld8v(ln_w + c, lw);
    ld8v(ln_b + c, lb);
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = (acc[k] - mean) * rstd * lw[k] + lb[k];
    st8v(out + g * C + c, acc);
  }
}

constexpr int kOutTile = 64;  // output samples per block

// A block of 256 per (64 samples, stream): the 70 rows the tile needs are transformed once into shared memory (f32
// values of their bf16 roundings). A thread then sums four consecutive samples over a sixteenth of the channels: per
// channel it reads ten rows and seven weights for 28 multiply-adds, and sixteen lanes reduce. Rows are C + 4 floats
// apart, so the two row groups a warp reads (four rows apart) fall into opposite halves of the banks.
__global__ void __launch_bounds__(256)
    codec_out_conv_kernel(const bf16* __restrict__ x, const bf16* __restrict__ bias, const float* __restrict__ alpha,
                          const float* __restrict__ inv_b, const bf16* __restrict__ w, const bf16* __restrict__ wb,
                          CodecStateRef st, int64_t hist_offset, float* __restrict__ wav, int T, int C) {
  constexpr int H = kTaps - 1, kPer = 4;  // samples per thread
  extern __shared__ __align__(16) float out_smem[];
  const int ld = C + 4, per = C / 8;
  float* sx = out_smem;                        // [64 + 6][C + 4]
  float* sw = out_smem + (kOutTile + H) * ld;  // [7][C]
  const int s = blockIdx.y, t0 = blockIdx.x * kOutTile, tid = threadIdx.x;
  const int p = st.pos[s];
  bf16* hist = slot_ptr(st, s, hist_offset);
  const bf16* old = hist + (p & 1) * (int64_t)H * C;
  bf16* next = hist + ((p + 1) & 1) * (int64_t)H * C;
  for (int i = tid; i < kTaps * C; i += blockDim.x) sw[i] = __bfloat162float(w[i]);
  for (int i = tid; i < (kOutTile + H) * per; i += blockDim.x) {
    const int row = i / per, c = i % per * 8, src = t0 - H + row;
    float v[8];
    if (src < 0) {
      ld8v(old + (int64_t)(H + src) * C + c, v);
    } else {
      ld8v(x + ((int64_t)s * T + src) * C + c, v);
      bias_snake8(v, bias, alpha, inv_b, c);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] = bf16_round(v[k]);
      // the frame's last six rows are the next history; rows below the tile's own (row < H) belong to the tile before
      if (src >= T - H && row >= H) st8v(next + (int64_t)(src - (T - H)) * C + c, v);
    }
    float4* dst = reinterpret_cast<float4*>(sx + row * ld + c);
    dst[0] = make_float4(v[0], v[1], v[2], v[3]);
    dst[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
  __syncthreads();
  const int q = tid & 15, rg = tid >> 4;  // channels q, q + 16, ...; samples rg * 4 .. rg * 4 + 3
  float acc[kPer] = {0.f, 0.f, 0.f, 0.f};
  for (int c = q; c < C; c += 16) {
    float v[kPer + H], wt[kTaps];
#pragma unroll
    for (int i = 0; i < kPer + H; ++i) v[i] = sx[(rg * kPer + i) * ld + c];
#pragma unroll
    for (int j = 0; j < kTaps; ++j) wt[j] = sw[j * C + c];
#pragma unroll
    for (int j = 0; j < kTaps; ++j)
#pragma unroll
      for (int o = 0; o < kPer; ++o) acc[o] += v[o + j] * wt[j];
  }
#pragma unroll
  for (int o = 0; o < kPer; ++o)
#pragma unroll
    for (int m = 1; m < 16; m <<= 1) acc[o] += __shfl_xor_sync(0xffffffffu, acc[o], m);
  if (q < kPer)
    wav[(int64_t)s * T + t0 + rg * kPer + q] = fminf(1.f, fmaxf(-1.f, bf16_round(acc[q] + __bfloat162float(wb[0]))));
}

inline unsigned blocks_for(int64_t total, int threads) { return (unsigned)((total + threads - 1) / threads); }

}  // namespace

cudaError_t launch_codec_rvq(const int32_t* codes, const bf16* books, bf16* out, int n, int half, int book_rows,
                             cudaStream_t stream) {
  codec_rvq_kernel<<<n, std::min(256, std::max(32, half / 8)), 0, stream>>>(codes, books, out, half, book_rows);
  return cudaGetLastError();
}

cudaError_t launch_codec_add_norm(const bf16* add, int64_t add_stride, bf16* res, const bf16* w, bf16* out, int rows,
                                  int dim, float eps, cudaStream_t stream) {
  codec_add_norm_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(add, add_stride, res, w, out, rows, dim, eps);
  return cudaGetLastError();
}

cudaError_t launch_codec_window_attend(const bf16* qkv, CodecStateRef st, int64_t ring_offset, bf16* out, int n, int heads,
                                       float theta, cudaStream_t stream) {
  codec_window_attend_kernel<<<dim3(n, (heads + 3) / 4), 128, 0, stream>>>(qkv, st, ring_offset, out, heads, theta);
  return cudaGetLastError();
}

cudaError_t launch_codec_silu_mul(const bf16* gate_up, bf16* out, int rows, int inter, cudaStream_t stream) {
  const int64_t total = (int64_t)rows * inter / 8;
  codec_silu_mul_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(gate_up, out, inter, total);
  return cudaGetLastError();
}

cudaError_t launch_codec_bias_gelu(bf16* x, const bf16* bias, int64_t rows, int cols, cudaStream_t stream) {
  const int64_t total = rows * cols / 8;
  codec_bias_gelu_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(x, bias, cols, total);
  return cudaGetLastError();
}

cudaError_t launch_codec_bias_snake(const bf16* x, const bf16* bias, const float* alpha, const float* inv_b, bf16* out,
                                    int64_t rows, int cols, cudaStream_t stream) {
  const int64_t total = rows * cols / 8;
  codec_bias_snake_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(x, bias, alpha, inv_b, out, cols, total);
  return cudaGetLastError();
}

cudaError_t launch_codec_stage(const bf16* x, const bf16* bias, const float* alpha, const float* inv_b, CodecStateRef st,
                               int64_t hist_offset, bf16* padded, int n, int T, int C, int H, cudaStream_t stream) {
  const int64_t total = (int64_t)n * (H + T) * (C / 8);
  codec_stage_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(x, bias, alpha, inv_b, st, hist_offset, padded, T, C, H,
                                                                 total);
  return cudaGetLastError();
}

cudaError_t launch_codec_gather_taps(const bf16* padded, bf16* col, int n, int T, int C, int taps, int dil,
                                     cudaStream_t stream) {
  const int64_t total = (int64_t)n * T * taps * (C / 8);
  codec_gather_taps_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(padded, col, T, C, taps, dil, total);
  return cudaGetLastError();
}

cudaError_t launch_codec_overlap_add(const bf16* z, const bf16* bias, CodecStateRef st, int64_t prev_offset, bf16* out,
                                     int n, int L, int r, int C, cudaStream_t stream) {
  const int64_t total = (int64_t)n * L * r * (C / 8);
  codec_overlap_add_kernel<<<blocks_for(total, 256), 256, 0, stream>>>(z, bias, st, prev_offset, out, L, r, C, total);
  return cudaGetLastError();
}

cudaError_t launch_codec_dwconv_ln(const bf16* z, const bf16* zb, const bf16* w, const bf16* b, const bf16* ln_w,
                                   const bf16* ln_b, CodecStateRef st, int64_t hist_offset, bf16* xin, bf16* out, int n,
                                   int T, int r, int C, float eps, cudaStream_t stream) {
  codec_dwconv_ln_kernel<<<(unsigned)((int64_t)n * T), (C / 8 + 31) / 32 * 32, 0, stream>>>(z, zb, w, b, ln_w, ln_b, st, hist_offset, xin,
                                                                          out, T, r, C, eps);
  return cudaGetLastError();
}

cudaError_t launch_codec_out_conv(const bf16* x, const bf16* bias, const float* alpha, const float* inv_b, const bf16* w,
                                  const bf16* wb, CodecStateRef st, int64_t hist_offset, float* wav, int n, int T, int C,
                                  cudaStream_t stream) {
  const size_t smem = ((size_t)(kOutTile + kTaps - 1) * (C + 4) + (size_t)kTaps * C) * sizeof(float);
  codec_out_conv_kernel<<<dim3(T / kOutTile, n), 256, smem, stream>>>(x, bias, alpha, inv_b, w, wb, st, hist_offset, wav,
                                                                      T, C);
  return cudaGetLastError();
}

}  // namespace omni
