// Memory-bound kernels: LayerNorm (fwd/bwd), SwiGLU (fwd/bwd), shared-mask dropout + residual add
// (fwd/bwd) and the flat AdamW + EMA step. Each makes one pass over its operands.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "common.cuh"

namespace df3 {
// Status word of the element-wise kernels (they take no status argument): written only by the bounds checks of the
// debug build, read by elementwise_status().
__device__ int ew_status = 0;
}  // namespace df3

namespace df3 {

constexpr int kLnMaxPerLane = 32;  // one warp per row, up to 32 * 32 = 1024 channels; kernels are
                                   // instantiated for 4 / 8 / 16 / 32 values per lane

// ---------------------------------------------------------------------------------------------
// LayerNorm forward: y = (x - mean) * rstd * w + b with fp32 statistics. One warp per row.
template <typename T, int K>
__global__ void __launch_bounds__(256) layer_norm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w,
                                                             const float* __restrict__ b, T* __restrict__ y,
                                                             float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                             int64_t rows, int C, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * C;
  float v[K];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + 32 * k;
    v[k] = (c < C) ? to_float<T>(xr[c]) : 0.f;
    s += v[k];
  }
  const float mean = warp_sum(s) / C;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + 32 * k;
    const float d = (c < C) ? v[k] - mean : 0.f;
    q += d * d;
  }
  const float rstd = rsqrtf(warp_sum(q) / C + eps);
  T* yr = y + row * C;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + 32 * k;
    if (c < C) {
      float o = (v[k] - mean) * rstd;
      if (w) o *= w[c];
      if (b) o += b[c];
      yr[c] = from_float<T>(o);
    }
  }
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
}

// LayerNorm forward for bf16 rows whose length is a multiple of 128: a lane owns groups of 4 consecutive channels
// (8-byte loads and stores, a warp covers 256 contiguous bytes per step). Same math as the generic kernel.
template <int G, int R>  // G groups of 4 channels per lane (C = 128 * G); R rows per warp in flight
__global__ void __launch_bounds__(256) layer_norm_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                                 const float* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                                 float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                 int64_t rows, float eps) {
  constexpr int C = 128 * G;
  const int lane = threadIdx.x & 31;
  float wv[4 * G], bv[4 * G];  // gain and bias stay in registers for every row this warp visits
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = 4 * (lane + 32 * g) + k;
      wv[4 * g + k] = w ? w[c] : 1.f;
      bv[4 * g + k] = b ? b[c] : 0.f;
    }
  const int64_t warp_stride = (int64_t)gridDim.x * (blockDim.x >> 5) * R;
  for (int64_t row0 = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * R; row0 < rows; row0 += warp_stride) {
  uint2 raw[R][G];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int64_t row = row0 + r < rows ? row0 + r : rows - 1;  // tail rows re-read the last row; their stores are skipped
    const uint2* xr = reinterpret_cast<const uint2*>(x + row * C);
#pragma unroll
    for (int g = 0; g < G; ++g)
      raw[r][g] = in_bounds(row * C + 4 * (lane + 32 * g) + 3, rows * C, &ew_status) ? xr[lane + 32 * g] : make_uint2(0u, 0u);
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float v[4 * G];
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw[r][g].x);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw[r][g].y);
      v[4 * g + 0] = __low2float(lo); v[4 * g + 1] = __high2float(lo);
      v[4 * g + 2] = __low2float(hi); v[4 * g + 3] = __high2float(hi);
      s += (v[4 * g + 0] + v[4 * g + 1]) + (v[4 * g + 2] + v[4 * g + 3]);
    }
    const float mean = warp_sum(s) / C;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < 4 * G; ++k) {
      const float d = v[k] - mean;
      q += d * d;
    }
    const float rstd = rsqrtf(warp_sum(q) / C + eps);
    if (row0 + r >= rows) continue;
    uint2* yr = reinterpret_cast<uint2*>(y + (row0 + r) * C);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) o[k] = (v[4 * g + k] - mean) * rstd * wv[4 * g + k] + bv[4 * g + k];
      __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
      uint2 out;
      out.x = *reinterpret_cast<uint32_t*>(&lo);
      out.y = *reinterpret_cast<uint32_t*>(&hi);
      yr[lane + 32 * g] = out;
    }
    if (lane == 0) {
      mean_out[row0 + r] = mean;
      rstd_out[row0 + r] = rstd;
    }
  }
  }
}

// LayerNorm backward. dx per row; dw / db are accumulated per block into partial[blockIdx.x][2][C]
// (summed on the host side in a fixed order, so the result is deterministic).
template <typename T, int K>
__global__ void __launch_bounds__(256) layer_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                             const float* __restrict__ w,
                                                             const float* __restrict__ mean_in,
                                                             const float* __restrict__ rstd_in, T* __restrict__ dx,
                                                             float* __restrict__ partial, int64_t rows, int C) {
  extern __shared__ float smem[];  // [warps][2][C]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float aw[K], ab[K];
#pragma unroll
  for (int k = 0; k < K; ++k) aw[k] = ab[k] = 0.f;
  for (int64_t row = (int64_t)blockIdx.x * nwarp + warp; row < rows; row += (int64_t)gridDim.x * nwarp) {
    const T* xr = x + row * C;
    const T* gr = dy + row * C;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[K], g[K];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + 32 * k;
      if (c < C) {
        const float go = to_float<T>(gr[c]);
        xh[k] = (to_float<T>(xr[c]) - mean) * rstd;
        g[k] = w ? go * w[c] : go;
        aw[k] += go * xh[k];
        ab[k] += go;
        s1 += g[k];
        s2 += g[k] * xh[k];
      } else {
        xh[k] = g[k] = 0.f;
      }
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
    T* dr = dx + row * C;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + 32 * k;
      if (c < C) dr[c] = from_float<T>(rstd * (g[k] - s1 - xh[k] * s2));
    }
  }
  if (partial == nullptr) return;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = lane + 32 * k;
    if (c < C) {
      smem[(warp * 2 + 0) * C + c] = aw[k];
      smem[(warp * 2 + 1) * C + c] = ab[k];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) {
    float s = 0.f;
    for (int wi = 0; wi < nwarp; ++wi) s += smem[wi * 2 * C + i];
    partial[(int64_t)blockIdx.x * 2 * C + i] = s;
  }
}

// LayerNorm backward for bf16 rows of 128 * G channels: 8-byte loads, R rows per warp in flight; same math and the
// same per-block (dw, db) partials as the generic kernel.
template <int G, int R>
__global__ void __launch_bounds__(256) layer_norm_bwd_vec_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                 const float* __restrict__ w, const float* __restrict__ mean_in,
                                                                 const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                                                 float* __restrict__ partial, int64_t rows) {
  constexpr int C = 128 * G;
  extern __shared__ float smem[];  // [warps][2][C]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float aw[4 * G], ab[4 * G], wv[4 * G];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      aw[4 * g + k] = ab[4 * g + k] = 0.f;
      wv[4 * g + k] = w ? w[4 * (lane + 32 * g) + k] : 1.f;
    }
  for (int64_t row0 = ((int64_t)blockIdx.x * nwarp + warp) * R; row0 < rows; row0 += (int64_t)gridDim.x * nwarp * R) {
    uint2 rx[R][G], rg[R][G];
    float mean[R], rstd[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int64_t row = row0 + r < rows ? row0 + r : rows - 1;
      const uint2* xr = reinterpret_cast<const uint2*>(x + row * C);
      const uint2* gr = reinterpret_cast<const uint2*>(dy + row * C);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        rx[r][g] = xr[lane + 32 * g];
        rg[r][g] = gr[lane + 32 * g];
      }
      mean[r] = mean_in[row];
      rstd[r] = rstd_in[row];
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= rows) continue;
      float xh[4 * G], gg[4 * G];
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const __nv_bfloat162 x0 = *reinterpret_cast<const __nv_bfloat162*>(&rx[r][g].x), x1 = *reinterpret_cast<const __nv_bfloat162*>(&rx[r][g].y);
        const __nv_bfloat162 g0 = *reinterpret_cast<const __nv_bfloat162*>(&rg[r][g].x), g1 = *reinterpret_cast<const __nv_bfloat162*>(&rg[r][g].y);
        const float xs[4] = {__low2float(x0), __high2float(x0), __low2float(x1), __high2float(x1)};
        const float gs[4] = {__low2float(g0), __high2float(g0), __low2float(g1), __high2float(g1)};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int i = 4 * g + k;
          xh[i] = (xs[k] - mean[r]) * rstd[r];
          gg[i] = gs[k] * wv[i];
          aw[i] += gs[k] * xh[i];
          ab[i] += gs[k];
          s1 += gg[i];
          s2 += gg[i] * xh[i];
        }
      }
      s1 = warp_sum(s1) / C;
      s2 = warp_sum(s2) / C;
      uint2* dr = reinterpret_cast<uint2*>(dx + (row0 + r) * C);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = rstd[r] * (gg[4 * g + k] - s1 - xh[4 * g + k] * s2);
        __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
        uint2 out;
        out.x = *reinterpret_cast<uint32_t*>(&lo);
        out.y = *reinterpret_cast<uint32_t*>(&hi);
        dr[lane + 32 * g] = out;
      }
    }
  }
  if (partial == nullptr) return;
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = 4 * (lane + 32 * g) + k;
      smem[(warp * 2 + 0) * C + c] = aw[4 * g + k];
      smem[(warp * 2 + 1) * C + c] = ab[4 * g + k];
    }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) {
    float s = 0.f;
    for (int wi = 0; wi < nwarp; ++wi) s += smem[wi * 2 * C + i];
    partial[(int64_t)blockIdx.x * 2 * C + i] = s;
  }
}

// LayerNorm over the channel axis of a channel-major tensor, fused with the transpose to channel-last:
//   x [C, M] (one plane per channel)  ->  y [M, C] = LN_c(x[:, m]) * w + b,   C = 32 * KC.
// A block owns 64 consecutive positions: planes are read in 128-byte rows into a [C][65] fp32 tile (the odd pitch makes
// the column reads conflict-free), then each warp normalises positions with lanes over channels and writes channel-last.
constexpr int kPlaneTile = 64;

template <int KC>
__global__ void __launch_bounds__(256) plane_layer_norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                                   const float* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                                   float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                   int64_t M, float eps) {
  constexpr int C = 32 * KC;
  extern __shared__ float tile[];  // [C][65]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t m0 = (int64_t)blockIdx.x * kPlaneTile;
  for (int c = warp; c < C; c += 8) {
    const __nv_bfloat16* src = x + (int64_t)c * M + m0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int pidx = lane + 32 * h;
      tile[c * 65 + pidx] = (m0 + pidx < M) ? __bfloat162float(src[pidx]) : 0.f;
    }
  }
  __syncthreads();
  for (int pidx = warp; pidx < kPlaneTile; pidx += 8) {
    if (m0 + pidx >= M) break;
    float v[KC];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      v[k] = tile[(lane + 32 * k) * 65 + pidx];
      s += v[k];
    }
    const float mean = warp_sum(s) / C;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < KC; ++k) q += (v[k] - mean) * (v[k] - mean);
    const float rstd = rsqrtf(warp_sum(q) / C + eps);
    __nv_bfloat16* yr = y + (m0 + pidx) * C;
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int c = lane + 32 * k;
      float o = (v[k] - mean) * rstd;
      if (w) o *= w[c];
      if (b) o += b[c];
      yr[c] = __float2bfloat16_rn(o);
    }
    if (lane == 0) {
      mean_out[m0 + pidx] = mean;
      rstd_out[m0 + pidx] = rstd;
    }
  }
}

// LayerNorm forward for 128-channel bf16 rows (the pair tensor) with eight lanes per row: a warp normalises four rows at
// once, every lane holds 16 channels (two 16-byte loads), and the two reductions take three shuffle steps over a group
// of eight lanes instead of five over the warp, i.e. 1.5 shuffles per row instead of 10 (the shuffle unit, one warp
// instruction per clock per SM, is what bounded the warp-per-row form below copy bandwidth). Two row groups per
// iteration keep 2 KiB of loads in flight per warp.
__global__ void __launch_bounds__(256) layer_norm_fwd_lane8_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                                   const float* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                                   float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                   int64_t rows, float eps) {
  constexpr int C = 128, kGroups = 2;
  const int lane = threadIdx.x & 31, sub = lane & 7, row_in_warp = lane >> 3;
  float wv[16], bv[16];
#pragma unroll
  for (int v = 0; v < 2; ++v)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int c = (sub + 8 * v) * 8 + e;
      wv[8 * v + e] = w ? w[c] : 1.f;
      bv[8 * v + e] = b ? b[c] : 0.f;
    }
  const int64_t warp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t warp_stride = (int64_t)gridDim.x * (blockDim.x >> 5) * 4 * kGroups;
  for (int64_t row0 = warp_id * 4 * kGroups; row0 < rows; row0 += warp_stride) {
    uint4 raw[kGroups][2];
#pragma unroll
    for (int gidx = 0; gidx < kGroups; ++gidx) {
      const int64_t want = row0 + gidx * 4 + row_in_warp;
      const int64_t row = want < rows ? want : rows - 1;  // tail lanes re-read the last row; their stores are skipped
      const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
      raw[gidx][0] = xr[sub];
      raw[gidx][1] = xr[sub + 8];
    }
#pragma unroll
    for (int gidx = 0; gidx < kGroups; ++gidx) {
      const int64_t row = row0 + gidx * 4 + row_in_warp;
      float v[16];
      float s = 0.f;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t ww[4] = {raw[gidx][h].x, raw[gidx][h].y, raw[gidx][h].z, raw[gidx][h].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(&ww[e]);
          v[8 * h + 2 * e] = __low2float(pr);
          v[8 * h + 2 * e + 1] = __high2float(pr);
          s += v[8 * h + 2 * e] + v[8 * h + 2 * e + 1];
        }
      }
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      const float mean = s * (1.f / C);
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < 16; ++k) q += (v[k] - mean) * (v[k] - mean);
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
      const float rstd = rsqrtf(q * (1.f / C) + eps);
      if (row < rows) {
        uint4* yr = reinterpret_cast<uint4*>(y + row * C);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t out[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int k = 8 * h + 2 * e;
            const __nv_bfloat162 pr = __floats2bfloat162_rn((v[k] - mean) * rstd * wv[k] + bv[k], (v[k + 1] - mean) * rstd * wv[k + 1] + bv[k + 1]);
            out[e] = *reinterpret_cast<const uint32_t*>(&pr);
          }
          yr[sub + 8 * h] = make_uint4(out[0], out[1], out[2], out[3]);
        }
        if (sub == 0) {
          mean_out[row] = mean;
          rstd_out[row] = rstd;
        }
      }
    }
  }
}

// The same with 16-byte accesses on both sides, for M % 8 == 0. A block owns 128 consecutive positions: every thread
// fetches eight positions of a plane per load (a half-warp covers 256 contiguous bytes of the plane) into a bf16 tile
// [C][130] (pitch 65 words: the column reads of the second phase hit 32 different banks), each warp then normalises
// positions with lanes over channels into a dense [128][C] bf16 tile, which is exactly the block's contiguous piece of
// the channel-last output and leaves with 16-byte stores.
constexpr int kPlaneTileV = 128;
constexpr int kPlanePitchV = 130;

template <int KC>
__global__ void __launch_bounds__(256) plane_layer_norm_fwd_vec_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                                                       const float* __restrict__ b, __nv_bfloat16* __restrict__ y,
                                                                       float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                       int64_t M, float eps) {
  constexpr int C = 32 * KC;
  extern __shared__ __align__(16) unsigned char plane_smem[];
  __nv_bfloat16* tin = reinterpret_cast<__nv_bfloat16*>(plane_smem);                       // [C][130]
  __nv_bfloat16* tout = tin + C * kPlanePitchV + 8;                                          // [128][C], 16-byte aligned
  float* stats = reinterpret_cast<float*>(tout + kPlaneTileV * C);                           // [4][128]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t m0 = (int64_t)blockIdx.x * kPlaneTileV;
  const int chunk = threadIdx.x & 15;           // eight positions
  const int64_t p0 = m0 + chunk * 8;
  for (int c = threadIdx.x >> 4; c < C; c += 16) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (p0 < M && in_bounds((int64_t)c * M + p0 + 7, (int64_t)C * M, &ew_status))   // M % 8 == 0: the chunk is inside or outside
      v = *reinterpret_cast<const uint4*>(x + (int64_t)c * M + p0);
    uint32_t* dst = reinterpret_cast<uint32_t*>(tin + c * kPlanePitchV + chunk * 8);
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
  }
  float wv[KC], bv[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    wv[k] = w ? w[lane + 32 * k] : 1.f;
    bv[k] = b ? b[lane + 32 * k] : 0.f;
  }
  __syncthreads();
  // statistics: one thread per (position, half of the channels), consecutive lanes on consecutive positions; sums are
  // taken about the position's first channel so that the single pass does not cancel; the two halves meet in shared memory
  {
    const int pidx = threadIdx.x & 127, half = threadIdx.x >> 7;
    const float shift = __bfloat162float(tin[pidx]);
    float s1 = 0.f, s2 = 0.f;
#pragma unroll 8
    for (int c = half * (C / 2); c < (half + 1) * (C / 2); ++c) {
      const float d = __bfloat162float(tin[c * kPlanePitchV + pidx]) - shift;
      s1 += d;
      s2 += d * d;
    }
    stats[(half * 2 + 0) * kPlaneTileV + pidx] = s1;
    stats[(half * 2 + 1) * kPlaneTileV + pidx] = s2;
  }
  __syncthreads();
  if (threadIdx.x < kPlaneTileV) {
    const int pidx = threadIdx.x;
    const float s1 = stats[pidx] + stats[2 * kPlaneTileV + pidx];
    const float s2 = stats[kPlaneTileV + pidx] + stats[3 * kPlaneTileV + pidx];
    const float dm = s1 / C;
    const float mean = __bfloat162float(tin[pidx]) + dm;
    const float rstd = rsqrtf(fmaxf(s2 / C - dm * dm, 0.f) + eps);
    stats[pidx] = mean;
    stats[kPlaneTileV + pidx] = rstd;
    if (m0 + pidx < M) {
      mean_out[m0 + pidx] = mean;
      rstd_out[m0 + pidx] = rstd;
    }
  }
  __syncthreads();
  for (int pidx = warp; pidx < kPlaneTileV; pidx += 8) {
    if (m0 + pidx >= M) break;
    const float mean = stats[pidx], rstd = stats[kPlaneTileV + pidx];
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const float v = __bfloat162float(tin[(lane + 32 * k) * kPlanePitchV + pidx]);
      tout[pidx * C + lane + 32 * k] = __float2bfloat16_rn((v - mean) * rstd * wv[k] + bv[k]);
    }
  }
  __syncthreads();
  const int64_t valid = (M - m0 < kPlaneTileV ? M - m0 : kPlaneTileV) * C / 8;   // 16-byte pieces of this block's output
  uint4* dst = reinterpret_cast<uint4*>(y + m0 * C);
  const uint4* src = reinterpret_cast<const uint4*>(tout);
  for (int64_t i = threadIdx.x; i < valid; i += 256)
    if (in_bounds(m0 * C / 8 + i, M * C / 8, &ew_status)) dst[i] = src[i];
}

// Backward of the above: dy [M, C] channel-last, x planes [C, M] -> dx planes [C, M]; (dw, db) partials per block.
template <int KC>
__global__ void __launch_bounds__(256) plane_layer_norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                                                   const float* __restrict__ w, const float* __restrict__ mean_in,
                                                                   const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                                                                   float* __restrict__ partial, int64_t M) {
  constexpr int C = 32 * KC;
  extern __shared__ float tile[];  // [C][65], then [8 warps][2][C] for the parameter gradients
  float* red = tile + C * 65;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t m0 = (int64_t)blockIdx.x * kPlaneTile;
  for (int c = warp; c < C; c += 8) {
    const __nv_bfloat16* src = x + (int64_t)c * M + m0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int pidx = lane + 32 * h;
      tile[c * 65 + pidx] = (m0 + pidx < M) ? __bfloat162float(src[pidx]) : 0.f;
    }
  }
  __syncthreads();
  float aw[KC], ab[KC], wv[KC];
#pragma unroll
  for (int k = 0; k < KC; ++k) {
    aw[k] = ab[k] = 0.f;
    wv[k] = w ? w[lane + 32 * k] : 1.f;
  }
  for (int pidx = warp; pidx < kPlaneTile; pidx += 8) {
    if (m0 + pidx >= M) break;
    const float mean = mean_in[m0 + pidx], rstd = rstd_in[m0 + pidx];
    const __nv_bfloat16* gr = dy + (m0 + pidx) * C;
    float xh[KC], g[KC];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const float go = __bfloat162float(gr[lane + 32 * k]);
      xh[k] = (tile[(lane + 32 * k) * 65 + pidx] - mean) * rstd;
      g[k] = go * wv[k];
      aw[k] += go * xh[k];
      ab[k] += go;
      s1 += g[k];
      s2 += g[k] * xh[k];
    }
    s1 = warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
#pragma unroll
    for (int k = 0; k < KC; ++k) tile[(lane + 32 * k) * 65 + pidx] = rstd * (g[k] - s1 - xh[k] * s2);  // own column only
  }
  if (partial != nullptr) {
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      red[(warp * 2 + 0) * C + lane + 32 * k] = aw[k];
      red[(warp * 2 + 1) * C + lane + 32 * k] = ab[k];
    }
  }
  __syncthreads();
  for (int c = warp; c < C; c += 8) {
    __nv_bfloat16* dst = dx + (int64_t)c * M + m0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int pidx = lane + 32 * h;
      if (m0 + pidx < M) dst[pidx] = __float2bfloat16_rn(tile[c * 65 + pidx]);
    }
  }
  if (partial != nullptr)
    for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) {
      float s = 0.f;
      for (int wi = 0; wi < 8; ++wi) s += red[wi * 2 * C + i];
      partial[(int64_t)blockIdx.x * 2 * C + i] = s;
    }
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int D) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D) return;
  const int64_t r = i / D;
  const int c = (int)(i - r * D);
  const float a = to_float<T>(x[r * 2 * D + c]), b = to_float<T>(x[r * 2 * D + D + c]);
  y[i] = from_float<T>(a * sigmoidf_(a) * b);
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx, int64_t rows,
                                  int D) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D) return;
  const int64_t r = i / D;
  const int c = (int)(i - r * D);
  const float a = to_float<T>(x[r * 2 * D + c]), b = to_float<T>(x[r * 2 * D + D + c]), g = to_float<T>(dy[i]);
  const float s = sigmoidf_(a);
  dx[r * 2 * D + c] = from_float<T>(g * b * s * (1.f + a * (1.f - s)));
  dx[r * 2 * D + D + c] = from_float<T>(g * a * s);
}

// bf16 rows with D a multiple of 8: a thread owns 8 consecutive channels (16-byte loads and stores).
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    f[2 * k] = __low2float(h[k]);
    f[2 * k + 1] = __high2float(h[k]);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  return u;
}

__global__ void __launch_bounds__(256) swiglu_fwd_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int64_t rows, int D8) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D8) return;
  const int64_t r = i / D8;
  const int c = (int)(i - r * D8);
  float a[8], b[8], o[8];
  unpack8(x[r * 2 * D8 + c], a);
  unpack8(x[r * 2 * D8 + D8 + c], b);
#pragma unroll
  for (int k = 0; k < 8; ++k) o[k] = a[k] * sigmoidf_(a[k]) * b[k];
  y[i] = pack8(o);
}

__global__ void __launch_bounds__(256) swiglu_bwd_vec_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ x,
                                                              uint4* __restrict__ dx, int64_t rows, int D8) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D8) return;
  const int64_t r = i / D8;
  const int c = (int)(i - r * D8);
  float a[8], b[8], g[8], da[8], db[8];
  unpack8(x[r * 2 * D8 + c], a);
  unpack8(x[r * 2 * D8 + D8 + c], b);
  unpack8(dy[i], g);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float s = sigmoidf_(a[k]);
    da[k] = g[k] * b[k] * s * (1.f + a[k] * (1.f - s));
    db[k] = g[k] * a[k] * s;
  }
  dx[r * 2 * D8 + c] = pack8(da);
  dx[r * 2 * D8 + D8 + c] = pack8(db);
}

// ---------------------------------------------------------------------------------------------
// Dropout whose Bernoulli draw is shared along one axis of x viewed as [outer, A, B, C]:
// share_rows: mask index (outer, b, c)  (shared along A);  else: (outer, a, c)  (shared along B).
// The mask is never stored: it is regenerated from (seed, mask index) in forward and backward.
__device__ __forceinline__ float drop_scale(const Philox& rng, int64_t mask_idx, float p, float inv_keep) {
  const uint4 r = rng((uint64_t)(mask_idx >> 2), 0);
  const uint32_t bits = ((mask_idx & 3) == 0) ? r.x : ((mask_idx & 3) == 1) ? r.y : ((mask_idx & 3) == 2) ? r.z : r.w;
  return uniform01(bits) >= p ? inv_keep : 0.f;
}

template <typename T, bool kAdd>
__global__ void dropout_shared_kernel(const T* __restrict__ res, const T* __restrict__ x, T* __restrict__ out,
                                      int64_t total, int64_t A, int64_t B, int64_t C, bool share_rows, float p,
                                      uint64_t seed, const long long* __restrict__ seed_dev) {
  if (seed_dev) seed += (uint64_t)*seed_dev;  // base seed kept on the device: a captured launch draws a new mask per replay
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int64_t c = i % C, ab = i / C, b = ab % B, oa = ab / B, a = oa % A, o = oa / A;
  const int64_t mi = share_rows ? (o * B + b) * C + c : (o * A + a) * C + c;
  const Philox rng(seed);
  const float m = drop_scale(rng, mi, p, 1.f / (1.f - p));
  const float v = to_float<T>(x[i]) * m;
  out[i] = from_float<T>(kAdd ? to_float<T>(res[i]) + v : v);
}

// Vector form for C % 8 == 0: a thread owns 8 consecutive channels of one mask position, draws their
// mask once (two Philox calls, the same values as the scalar kernel) and walks kSpan positions of the
// axis the mask is shared along, 16 bytes (bf16) or 32 bytes (fp32) per step.
template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  uint4 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ __forceinline__ float get(int i) const { return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(&raw)[i]); }
  __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<__nv_bfloat16*>(&raw)[i] = __float2bfloat16_rn(v); }
};
template <> struct Vec8<float> {
  float4 lo, hi;
  __device__ __forceinline__ void load(const float* p) { lo = reinterpret_cast<const float4*>(p)[0]; hi = reinterpret_cast<const float4*>(p)[1]; }
  __device__ __forceinline__ void store(float* p) const { reinterpret_cast<float4*>(p)[0] = lo; reinterpret_cast<float4*>(p)[1] = hi; }
  __device__ __forceinline__ float get(int i) const { return i < 4 ? (&lo.x)[i] : (&hi.x)[i - 4]; }
  __device__ __forceinline__ void set(int i, float v) { if (i < 4) (&lo.x)[i] = v; else (&hi.x)[i - 4] = v; }
};

template <typename T, bool kAdd, int kSpan>
__global__ void __launch_bounds__(256) dropout_shared_vec_kernel(const T* __restrict__ res, const T* __restrict__ x,
                                                                 T* __restrict__ out, int64_t O, int64_t A, int64_t B,
                                                                 int64_t C, bool share_rows, float p, uint64_t seed,
                                                                 const long long* __restrict__ seed_dev) {
  if (seed_dev) seed += (uint64_t)*seed_dev;
  const int64_t c8n = C / 8;
  const int64_t shared_len = share_rows ? A : B;   // axis the mask is shared along
  const int64_t other_len = share_rows ? B : A;    // axis that indexes the mask together with (o, c)
  const int64_t spans = (shared_len + kSpan - 1) / kSpan;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= O * spans * other_len * c8n) return;
  const int64_t c8 = t % c8n;
  int64_t rest = t / c8n;
  const int64_t other = rest % other_len; rest /= other_len;
  const int64_t span = rest % spans;
  const int64_t o = rest / spans;
  const int64_t mi = (o * other_len + other) * C + c8 * 8;  // mask index of channel c8 * 8; a multiple of 4
  const Philox rng(seed);
  const uint4 r0 = rng((uint64_t)(mi >> 2), 0), r1 = rng((uint64_t)(mi >> 2) + 1, 0);
  const uint32_t bits[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
  const float inv_keep = 1.f / (1.f - p);
  float m[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) m[i] = uniform01(bits[i]) >= p ? inv_keep : 0.f;
  const int64_t s_end = min(shared_len, (span + 1) * (int64_t)kSpan);
  for (int64_t sidx = span * kSpan; sidx < s_end; ++sidx) {
    const int64_t a = share_rows ? sidx : other, b = share_rows ? other : sidx;
    const int64_t off = ((o * A + a) * B + b) * C + c8 * 8;
    Vec8<T> vx, vr;
    vx.load(x + off);
    if (kAdd) vr.load(res + off);
#pragma unroll
    for (int i = 0; i < 8; ++i) vx.set(i, kAdd ? vr.get(i) + vx.get(i) * m[i] : vx.get(i) * m[i]);
    vx.store(out + off);
  }
}

// ---------------------------------------------------------------------------------------------
// Flat AdamW + EMA: g = grad * scale; decoupled decay; moments; bias-corrected update; shadow lerp.
__global__ void __launch_bounds__(256) adamw_ema_kernel(float4* __restrict__ p, const float4* __restrict__ g,
                                                        float4* __restrict__ m, float4* __restrict__ v,
                                                        float4* __restrict__ ema, const float4* __restrict__ decay,
                                                        uint2* __restrict__ p16,  // bf16 mirror of p, 4 values per item, or null
                                                        const float* __restrict__ scale_ptr, int64_t n4, float lr,
                                                        float b1, float b2, float eps, float bc1, float bc2_sqrt,
                                                        float ema_w) {
  const float scale = *scale_ptr;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 pp = p[i], gg = g[i], mm = m[i], vv = v[i], dd = decay[i];
    float* P = &pp.x; float* G = &gg.x; float* M = &mm.x; float* V = &vv.x; float* D = &dd.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = G[k] * scale;
      float pk = P[k] * (1.f - lr * D[k]);
      M[k] = M[k] + (gk - M[k]) * (1.f - b1);
      V[k] = V[k] * b2 + gk * gk * (1.f - b2);
      pk -= (lr / bc1) * M[k] / (sqrtf(V[k]) / bc2_sqrt + eps);
      P[k] = pk;
    }
    p[i] = pp; m[i] = mm; v[i] = vv;
    if (p16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 w;
      w.x = *reinterpret_cast<uint32_t*>(&lo);
      w.y = *reinterpret_cast<uint32_t*>(&hi);
      p16[i] = w;
    }
    if (ema) {
      float4 ee = ema[i];
      ee.x += (pp.x - ee.x) * ema_w; ee.y += (pp.y - ee.y) * ema_w;
      ee.z += (pp.z - ee.z) * ema_w; ee.w += (pp.w - ee.w) * ema_w;
      ema[i] = ee;
    }
  }
}

}  // namespace df3

namespace df3 {
// Backward of out = sigmoid(g) * p * m with (g, p) stored as gp[row] = [g(0..D) | p(0..D)]:
// dgp[row] = [dy m p sg (1 - sg) | dy m sg].
__global__ void gated_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gp,
                                 const float* __restrict__ mask, __nv_bfloat16* __restrict__ dgp, int64_t rows, int D) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D) return;
  const int64_t r = i / D;
  const int c = (int)(i - r * D);
  const float g = __bfloat162float(gp[r * 2 * D + c]), pv = __bfloat162float(gp[r * 2 * D + D + c]);
  const float sg = sigmoidf_(g);
  const float d = __bfloat162float(dy[i]) * (mask ? mask[r] : 1.f);
  dgp[r * 2 * D + c] = __float2bfloat16_rn(d * pv * sg * (1.f - sg));
  dgp[r * 2 * D + D + c] = __float2bfloat16_rn(d * sg);
}
// Same as gated_bwd_kernel for D a multiple of 8: a thread owns 8 consecutive channels (16-byte accesses).
__global__ void __launch_bounds__(256) gated_bwd_vec_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ gp,
                                                             const float* __restrict__ mask, uint4* __restrict__ dgp, int64_t rows,
                                                             int D8) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D8) return;
  const int64_t r = i / D8;
  const int c = (int)(i - r * D8);
  float g[8], pv[8], d[8], dg[8], dp[8];
  unpack8(gp[r * 2 * D8 + c], g);
  unpack8(gp[r * 2 * D8 + D8 + c], pv);
  unpack8(dy[i], d);
  const float m = mask ? mask[r] : 1.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float sg = sigmoidf_(g[k]);
    dg[k] = d[k] * m * pv[k] * sg * (1.f - sg);
    dp[k] = d[k] * m * sg;
  }
  dgp[r * 2 * D8 + c] = pack8(dg);
  dgp[r * 2 * D8 + D8 + c] = pack8(dp);
}

// Backward of out = sigmoid(g) * other, elementwise: dg = dy other sg (1 - sg), d_other = dy sg. n8 = elements / 8.
__global__ void __launch_bounds__(256) sigmoid_gate_bwd_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ g,
                                                                const uint4* __restrict__ other, uint4* __restrict__ dg,
                                                                uint4* __restrict__ d_other, int64_t n8) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float d[8], gv[8], o[8], a[8], b[8];
  unpack8(dy[i], d);
  unpack8(g[i], gv);
  unpack8(other[i], o);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float sg = sigmoidf_(gv[k]);
    a[k] = d[k] * o[k] * sg * (1.f - sg);
    b[k] = d[k] * sg;
  }
  dg[i] = pack8(a);
  d_other[i] = pack8(b);
}
}  // namespace df3

// ================================================================================================
// host side
using torch::Tensor;

static inline cudaStream_t stream() { return at::cuda::getCurrentCUDAStream(); }

std::tuple<Tensor, Tensor, Tensor> df3_layer_norm_fwd(const Tensor& x, const c10::optional<Tensor>& w,
                                                      const c10::optional<Tensor>& b, double eps) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "layer_norm: x must be a contiguous CUDA tensor");
  const int C = x.size(-1);
  TORCH_CHECK(C <= 32 * df3::kLnMaxPerLane, "layer_norm: at most 1024 channels");
  const int64_t rows = x.numel() / C;
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty_like(x);
  auto opts = x.options().dtype(torch::kFloat32);
  auto mean = torch::empty({rows}, opts), rstd = torch::empty({rows}, opts);
  if (rows == 0) return {y, mean, rstd};
  const float* wp = w.has_value() ? w->data_ptr<float>() : nullptr;
  const float* bp = b.has_value() ? b->data_ptr<float>() : nullptr;
  const int warps = 8;
  const unsigned grid = (unsigned)((rows + warps - 1) / warps);
  const bool bf16 = x.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(bf16 || x.scalar_type() == torch::kFloat32, "layer_norm: bf16 or fp32");
#define DF3_LN_FWD(K)                                                                                              \
  do {                                                                                                             \
    if (bf16)                                                                                                      \
      df3::layer_norm_fwd_kernel<__nv_bfloat16, K><<<grid, warps * 32, 0, stream()>>>(                             \
          (const __nv_bfloat16*)x.data_ptr(), wp, bp, (__nv_bfloat16*)y.data_ptr(), mean.data_ptr<float>(),        \
          rstd.data_ptr<float>(), rows, C, (float)eps);                                                            \
    else                                                                                                           \
      df3::layer_norm_fwd_kernel<float, K><<<grid, warps * 32, 0, stream()>>>(                                     \
          x.data_ptr<float>(), wp, bp, y.data_ptr<float>(), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows,  \
          C, (float)eps);                                                                                          \
  } while (0)
  const bool vec_ok = bf16 && C % 128 == 0 && C <= 768 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 8 == 0;
#define DF3_LN_VEC(G)                                                                                              \
  df3::layer_norm_fwd_vec_kernel<G, (G <= 2 ? 4 : 2)><<<(unsigned)std::min<int64_t>((rows + warps * (G <= 2 ? 4 : 2) - 1) / (warps * (G <= 2 ? 4 : 2)), 148 * 16), \
                                                       warps * 32, 0, stream()>>>(                                   \
      (const __nv_bfloat16*)x.data_ptr(), wp, bp, (__nv_bfloat16*)y.data_ptr(), mean.data_ptr<float>(),            \
      rstd.data_ptr<float>(), rows, (float)eps)
  if (vec_ok && C == 128 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(y.data_ptr()) % 16 == 0)
    df3::layer_norm_fwd_lane8_kernel<<<(unsigned)std::min<int64_t>((rows + 63) / 64, 148 * 16), 256, 0, stream()>>>(
        (const __nv_bfloat16*)x.data_ptr(), wp, bp, (__nv_bfloat16*)y.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows,
        (float)eps);
  else if (vec_ok && C == 128) DF3_LN_VEC(1);
  else if (vec_ok && C == 256) DF3_LN_VEC(2);
  else if (vec_ok && C == 384) DF3_LN_VEC(3);
  else if (vec_ok && C == 512) DF3_LN_VEC(4);
  else if (vec_ok && C == 768) DF3_LN_VEC(6);
  else if (C <= 128) DF3_LN_FWD(4); else if (C <= 256) DF3_LN_FWD(8); else if (C <= 512) DF3_LN_FWD(16); else DF3_LN_FWD(32);
#undef DF3_LN_VEC
#undef DF3_LN_FWD
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, mean, rstd};
}

// returns (dx, partial [blocks, 2, C]); partial is empty when want_wb is false
std::tuple<Tensor, Tensor> df3_layer_norm_bwd(const Tensor& dy, const Tensor& x, const c10::optional<Tensor>& w,
                                              const Tensor& mean, const Tensor& rstd, bool want_wb) {
  const int C = x.size(-1);
  const int64_t rows = x.numel() / C;
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty_like(x);
  const int warps = 8;
  const int blocks = (int)std::min<int64_t>((rows + warps - 1) / warps, 148 * 4);
  auto partial = want_wb ? torch::empty({blocks, 2, C}, x.options().dtype(torch::kFloat32)) : torch::empty({0}, x.options().dtype(torch::kFloat32));
  if (rows == 0) return {dx, partial};
  const float* wp = w.has_value() ? w->data_ptr<float>() : nullptr;
  float* pp = want_wb ? partial.data_ptr<float>() : nullptr;
  const size_t smem = want_wb ? (size_t)warps * 2 * C * sizeof(float) : 0;
  const bool bf16 = x.scalar_type() == torch::kBFloat16;
#define DF3_LN_BWD(K)                                                                                              \
  do {                                                                                                             \
    if (bf16) {                                                                                                    \
      auto k = df3::layer_norm_bwd_kernel<__nv_bfloat16, K>;                                                       \
      if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      k<<<blocks, warps * 32, smem, stream()>>>((const __nv_bfloat16*)dy.data_ptr(),                               \
                                                (const __nv_bfloat16*)x.data_ptr(), wp, mean.data_ptr<float>(),    \
                                                rstd.data_ptr<float>(), (__nv_bfloat16*)dx.data_ptr(), pp, rows, C); \
    } else {                                                                                                       \
      auto k = df3::layer_norm_bwd_kernel<float, K>;                                                               \
      if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      k<<<blocks, warps * 32, smem, stream()>>>(dy.data_ptr<float>(), x.data_ptr<float>(), wp,                     \
                                                mean.data_ptr<float>(), rstd.data_ptr<float>(),                    \
                                                dx.data_ptr<float>(), pp, rows, C);                                \
    }                                                                                                              \
  } while (0)
  const bool vec_ok = bf16 && (C == 128 || C == 256 || C == 384) && reinterpret_cast<uintptr_t>(x.data_ptr()) % 8 == 0 &&
                      reinterpret_cast<uintptr_t>(dy.data_ptr()) % 8 == 0 && dy.scalar_type() == torch::kBFloat16;
#define DF3_LN_BWD_VEC(G)                                                                                          \
  df3::layer_norm_bwd_vec_kernel<G, 2><<<blocks, warps * 32, smem, stream()>>>(                                    \
      (const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)x.data_ptr(), wp, mean.data_ptr<float>(),         \
      rstd.data_ptr<float>(), (__nv_bfloat16*)dx.data_ptr(), pp, rows)
  if (vec_ok && C == 128) DF3_LN_BWD_VEC(1);
  else if (vec_ok && C == 256) DF3_LN_BWD_VEC(2);
  else if (vec_ok && C == 384) DF3_LN_BWD_VEC(3);
  else if (C <= 128) DF3_LN_BWD(4); else if (C <= 256) DF3_LN_BWD(8); else if (C <= 512) DF3_LN_BWD(16); else DF3_LN_BWD(32);
#undef DF3_LN_BWD_VEC
#undef DF3_LN_BWD
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, partial};
}

// x [C, M] bf16 planes -> (y [M, C], mean [M], rstd [M])
std::tuple<Tensor, Tensor, Tensor> df3_plane_layer_norm_fwd(const Tensor& x, const c10::optional<Tensor>& w,
                                                            const c10::optional<Tensor>& b, double eps) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2 && x.scalar_type() == torch::kBFloat16, "plane_layer_norm: contiguous bf16 [C, M]");
  const int C = x.size(0);
  const int64_t M = x.size(1);
  TORCH_CHECK(C == 32 || C == 64 || C == 128 || C == 256, "plane_layer_norm: 32, 64, 128 or 256 channels");
  c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty({M, C}, x.options());
  auto opts = x.options().dtype(torch::kFloat32);
  auto mean = torch::empty({M}, opts), rstd = torch::empty({M}, opts);
  if (M == 0) return {y, mean, rstd};
  const float* wp = w.has_value() ? w->data_ptr<float>() : nullptr;
  const float* bp = b.has_value() ? b->data_ptr<float>() : nullptr;
  if (M % 8 == 0 && (C == 64 || C == 128) && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0) {
    const unsigned vgrid = (unsigned)((M + df3::kPlaneTileV - 1) / df3::kPlaneTileV);
    const size_t vsmem = ((size_t)C * df3::kPlanePitchV + 8 + (size_t)df3::kPlaneTileV * C) * 2 + 4 * df3::kPlaneTileV * sizeof(float);
#define DF3_PLNV(KC)                                                                                               \
  do {                                                                                                             \
    auto k = df3::plane_layer_norm_fwd_vec_kernel<KC>;                                                             \
    static bool attr = false;                                                                                      \
    if (!attr) {                                                                                                   \
      C10_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)vsmem));            \
      attr = true;                                                                                                 \
    }                                                                                                              \
    k<<<vgrid, 256, vsmem, stream()>>>((const __nv_bfloat16*)x.data_ptr(), wp, bp, (__nv_bfloat16*)y.data_ptr(),   \
                                       mean.data_ptr<float>(), rstd.data_ptr<float>(), M, (float)eps);             \
  } while (0)
    if (C == 64) DF3_PLNV(2); else DF3_PLNV(4);
#undef DF3_PLNV
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return {y, mean, rstd};
  }
  const unsigned grid = (unsigned)((M + df3::kPlaneTile - 1) / df3::kPlaneTile);
  const size_t smem = (size_t)C * 65 * sizeof(float);
#define DF3_PLN(KC)                                                                                                \
  do {                                                                                                             \
    auto k = df3::plane_layer_norm_fwd_kernel<KC>;                                                                 \
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
    k<<<grid, 256, smem, stream()>>>((const __nv_bfloat16*)x.data_ptr(), wp, bp, (__nv_bfloat16*)y.data_ptr(),     \
                                     mean.data_ptr<float>(), rstd.data_ptr<float>(), M, (float)eps);               \
  } while (0)
  if (C == 32) DF3_PLN(1); else if (C == 64) DF3_PLN(2); else if (C == 128) DF3_PLN(4); else DF3_PLN(8);
#undef DF3_PLN
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, mean, rstd};
}

// dy [M, C], x planes [C, M] -> (dx planes [C, M], partial [blocks, 2, C])
std::tuple<Tensor, Tensor> df3_plane_layer_norm_bwd(const Tensor& dy, const Tensor& x, const c10::optional<Tensor>& w,
                                                    const Tensor& mean, const Tensor& rstd, bool want_wb) {
  TORCH_CHECK(dy.is_contiguous() && dy.scalar_type() == torch::kBFloat16 && x.is_contiguous(), "plane_layer_norm_bwd: contiguous bf16");
  const int C = x.size(0);
  const int64_t M = x.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = torch::empty_like(x);
  const int blocks = (int)((M + df3::kPlaneTile - 1) / df3::kPlaneTile);
  auto partial = torch::empty({want_wb ? blocks : 0, 2, C}, x.options().dtype(torch::kFloat32));
  if (M == 0) return {dx, partial};
  const float* wp = w.has_value() ? w->data_ptr<float>() : nullptr;
  float* pp = want_wb ? partial.data_ptr<float>() : nullptr;
  const size_t smem = ((size_t)C * 65 + 8 * 2 * C) * sizeof(float);
#define DF3_PLNB(KC)                                                                                               \
  do {                                                                                                             \
    auto k = df3::plane_layer_norm_bwd_kernel<KC>;                                                                 \
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
    k<<<blocks, 256, smem, stream()>>>((const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)x.data_ptr(), wp, \
                                       mean.data_ptr<float>(), rstd.data_ptr<float>(), (__nv_bfloat16*)dx.data_ptr(), pp, M); \
  } while (0)
  if (C == 32) DF3_PLNB(1); else if (C == 64) DF3_PLNB(2); else if (C == 128) DF3_PLNB(4); else DF3_PLNB(8);
#undef DF3_PLNB
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, partial};
}

Tensor df3_gated_bwd(const Tensor& dy, const Tensor& gp, const c10::optional<Tensor>& mask) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && gp.is_contiguous() && dy.scalar_type() == torch::kBFloat16 &&
              gp.scalar_type() == torch::kBFloat16 && gp.size(-1) == 2 * dy.size(-1), "gated_bwd: dy [rows, D], gp [rows, 2 D], bf16");
  c10::cuda::CUDAGuard guard(dy.device());
  const int D = dy.size(-1);
  const int64_t rows = dy.numel() / D;
  auto dgp = torch::empty_like(gp);
  if (rows == 0) return dgp;
  const float* mp = nullptr;
  Tensor m;
  if (mask.has_value() && mask->defined()) {
    m = mask->to(torch::kFloat32).contiguous();
    TORCH_CHECK(m.numel() == rows, "gated_bwd: mask length");
    mp = m.data_ptr<float>();
  }
  const unsigned grid = (unsigned)((rows * D + 255) / 256);
  if (D % 8 == 0 && reinterpret_cast<uintptr_t>(dy.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(gp.data_ptr()) % 16 == 0)
    df3::gated_bwd_vec_kernel<<<(unsigned)((rows * (D / 8) + 255) / 256), 256, 0, stream()>>>(
        (const uint4*)dy.data_ptr(), (const uint4*)gp.data_ptr(), mp, (uint4*)dgp.data_ptr(), rows, D / 8);
  else
  df3::gated_bwd_kernel<<<grid, 256, 0, stream()>>>((const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)gp.data_ptr(), mp,
                                                   (__nv_bfloat16*)dgp.data_ptr(), rows, D);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dgp;
}

// (dg, d_other) of out = sigmoid(g) * other for contiguous bf16 tensors of one shape whose size is a multiple of 8
std::tuple<Tensor, Tensor> df3_sigmoid_gate_bwd(const Tensor& dy, const Tensor& g, const Tensor& other) {
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && g.is_contiguous() && other.is_contiguous(), "sigmoid_gate_bwd: contiguous CUDA tensors");
  TORCH_CHECK(dy.scalar_type() == torch::kBFloat16 && g.scalar_type() == torch::kBFloat16 && other.scalar_type() == torch::kBFloat16,
              "sigmoid_gate_bwd: bf16 tensors");
  TORCH_CHECK(dy.numel() == g.numel() && dy.numel() == other.numel() && dy.numel() % 8 == 0, "sigmoid_gate_bwd: equal sizes, multiple of 8");
  c10::cuda::CUDAGuard guard(dy.device());
  auto dg = torch::empty_like(g), d_other = torch::empty_like(other);
  const int64_t n8 = dy.numel() / 8;
  if (n8 == 0) return {dg, d_other};
  const Tensor* all[5] = {&dy, &g, &other, &dg, &d_other};
  for (const Tensor* t : all)
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0, "sigmoid_gate_bwd: 16-byte aligned tensors");
  df3::sigmoid_gate_bwd_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream()>>>(
      (const uint4*)dy.data_ptr(), (const uint4*)g.data_ptr(), (const uint4*)other.data_ptr(), (uint4*)dg.data_ptr(),
      (uint4*)d_other.data_ptr(), n8);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dg, d_other};
}

// The element-wise kernels' status word: 0, or df3::kBadShape after a bounds check of the debug build failed.
int64_t df3_elementwise_status() {
  int code = 0;
  C10_CUDA_CHECK(cudaMemcpyFromSymbol(&code, df3::ew_status, sizeof(int)));
  if (code != 0) {
    const int zero = 0;
    C10_CUDA_CHECK(cudaMemcpyToSymbol(df3::ew_status, &zero, sizeof(int)));
  }
  return code;
}

Tensor df3_swiglu_fwd(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.size(-1) % 2 == 0, "swiglu: contiguous CUDA tensor, even width");
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1) / 2;
  const int64_t rows = x.numel() / (2 * D);
  auto shape = x.sizes().vec();
  shape.back() = D;
  auto y = torch::empty(shape, x.options());
  const int64_t n = rows * D;
  if (n == 0) return y;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (x.scalar_type() == torch::kBFloat16 && D % 8 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0)
    df3::swiglu_fwd_vec_kernel<<<(unsigned)((rows * (D / 8) + 255) / 256), 256, 0, stream()>>>(
        (const uint4*)x.data_ptr(), (uint4*)y.data_ptr(), rows, D / 8);
  else if (x.scalar_type() == torch::kBFloat16)
    df3::swiglu_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream()>>>((const __nv_bfloat16*)x.data_ptr(), (__nv_bfloat16*)y.data_ptr(), rows, D);
  else
    df3::swiglu_fwd_kernel<float><<<grid, 256, 0, stream()>>>(x.data_ptr<float>(), y.data_ptr<float>(), rows, D);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

Tensor df3_swiglu_bwd(const Tensor& dy, const Tensor& x) {
  c10::cuda::CUDAGuard guard(x.device());
  const int D = x.size(-1) / 2;
  const int64_t rows = x.numel() / (2 * D);
  auto dx = torch::empty_like(x);
  const int64_t n = rows * D;
  if (n == 0) return dx;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (x.scalar_type() == torch::kBFloat16 && D % 8 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(dy.data_ptr()) % 16 == 0)
    df3::swiglu_bwd_vec_kernel<<<(unsigned)((rows * (D / 8) + 255) / 256), 256, 0, stream()>>>(
        (const uint4*)dy.data_ptr(), (const uint4*)x.data_ptr(), (uint4*)dx.data_ptr(), rows, D / 8);
  else if (x.scalar_type() == torch::kBFloat16)
    df3::swiglu_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream()>>>((const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)x.data_ptr(), (__nv_bfloat16*)dx.data_ptr(), rows, D);
  else
    df3::swiglu_bwd_kernel<float><<<grid, 256, 0, stream()>>>(dy.data_ptr<float>(), x.data_ptr<float>(), dx.data_ptr<float>(), rows, D);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dx;
}

// x viewed as [outer, A, B, C]; res may be undefined (then out = dropout(x), used by backward)
Tensor df3_dropout_shared(const c10::optional<Tensor>& res, const Tensor& x, int64_t A, int64_t B, int64_t C,
                          bool share_rows, double p, int64_t seed, const c10::optional<Tensor>& seed_dev) {
  const long long* sd = nullptr;
  if (seed_dev.has_value() && seed_dev->defined()) {
    TORCH_CHECK(seed_dev->is_cuda() && seed_dev->scalar_type() == torch::kInt64 && seed_dev->numel() >= 1, "dropout_shared: seed_dev is an int64 CUDA tensor");
    sd = reinterpret_cast<const long long*>(seed_dev->data_ptr());
  }
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "dropout_shared: contiguous CUDA tensor");
  c10::cuda::CUDAGuard guard(x.device());
  auto out = torch::empty_like(x);
  const int64_t n = x.numel();
  if (n == 0) return out;
  const unsigned grid = (unsigned)((n + 255) / 256);
  const bool add = res.has_value();
  if (add) TORCH_CHECK(res->is_contiguous() && res->sizes() == x.sizes() && res->scalar_type() == x.scalar_type(), "dropout_shared: residual mismatch");
  constexpr int kSpan = 8;
  const bool vec = C % 8 == 0 && reinterpret_cast<uintptr_t>(x.data_ptr()) % 32 == 0 &&
                   reinterpret_cast<uintptr_t>(out.data_ptr()) % 32 == 0 &&
                   (!add || reinterpret_cast<uintptr_t>(res->data_ptr()) % 32 == 0);
  const int64_t O = n / (A * B * C);
  const int64_t vthreads = O * (((share_rows ? A : B) + kSpan - 1) / kSpan) * (share_rows ? B : A) * (C / 8);
  const unsigned vgrid = (unsigned)((vthreads + 255) / 256);
#define DF3_LAUNCH(T, ADD)                                                                                         \
  do {                                                                                                             \
    if (vec)                                                                                                       \
      df3::dropout_shared_vec_kernel<T, ADD, kSpan><<<vgrid, 256, 0, stream()>>>(                                  \
          ADD ? (const T*)res->data_ptr() : nullptr, (const T*)x.data_ptr(), (T*)out.data_ptr(), O, A, B, C,       \
          share_rows, (float)p, (uint64_t)seed, sd);                                                               \
    else                                                                                                           \
      df3::dropout_shared_kernel<T, ADD><<<grid, 256, 0, stream()>>>(ADD ? (const T*)res->data_ptr() : nullptr,    \
                                                                     (const T*)x.data_ptr(), (T*)out.data_ptr(), n, \
                                                                     A, B, C, share_rows, (float)p, (uint64_t)seed, sd); \
  } while (0)
  if (x.scalar_type() == torch::kBFloat16) {
    if (add) DF3_LAUNCH(__nv_bfloat16, true); else DF3_LAUNCH(__nv_bfloat16, false);
  } else {
    TORCH_CHECK(x.scalar_type() == torch::kFloat32, "dropout_shared: bf16 or fp32");
    if (add) DF3_LAUNCH(float, true); else DF3_LAUNCH(float, false);
  }
#undef DF3_LAUNCH
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

void df3_adamw_ema(Tensor p, const Tensor& g, Tensor m, Tensor v, const c10::optional<Tensor>& ema,
                   const Tensor& decay, const Tensor& scale, double lr, double b1, double b2, double eps, double bc1,
                   double bc2, double ema_w, const c10::optional<Tensor>& p16) {
  TORCH_CHECK(p.is_cuda() && p.scalar_type() == torch::kFloat32 && p.numel() % 4 == 0, "adamw_ema: flat fp32, numel % 4 == 0");
  c10::cuda::CUDAGuard guard(p.device());
  const int64_t n4 = p.numel() / 4;
  if (n4 == 0) return;
  const int blocks = (int)std::min<int64_t>((n4 + 255) / 256, 148 * 8);
  df3::adamw_ema_kernel<<<blocks, 256, 0, stream()>>>(
      (float4*)p.data_ptr<float>(), (const float4*)g.data_ptr<float>(), (float4*)m.data_ptr<float>(),
      (float4*)v.data_ptr<float>(), ema.has_value() ? (float4*)ema->data_ptr<float>() : nullptr,
      (const float4*)decay.data_ptr<float>(),
      (p16.has_value() && p16->defined()) ? (uint2*)p16->data_ptr() : nullptr, scale.data_ptr<float>(), n4, (float)lr, (float)b1, (float)b2, (float)eps,
      (float)bc1, (float)std::sqrt(bc2), (float)ema_w);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}
