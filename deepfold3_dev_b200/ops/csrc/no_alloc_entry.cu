// LayerNorm backward behind a plain C symbol that allocates nothing; see no_alloc_entry.h for the
// contract (static scratch, its limit, set-up before capture, no overlapping calls).
#include "no_alloc_entry.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int kMaxC = DF3_NO_ALLOC_MAX_CHANNELS;
constexpr int kMaxBlocks = DF3_NO_ALLOC_MAX_BLOCKS;
constexpr int kWarps = 4;
constexpr int kMaxDevices = 64;

// per-block partial sums of (dw, db): [block][2][channels], rewritten by every call
static __device__ __align__(256) float g_scratch[kMaxBlocks * 2 * kMaxC];

thread_local char t_error[256] = "";
std::mutex g_mutex;
float* g_scratch_ptr[kMaxDevices] = {};

int fail(int code, const char* what) {
  snprintf(t_error, sizeof(t_error), "%s", what);
  return code;
}

int fail_cuda(cudaError_t e, const char* where) {
  snprintf(t_error, sizeof(t_error), "%s: %s", where, cudaGetErrorString(e));
  return (int)e;
}

// One warp per row, K values per lane; dx written per row, (dw, db) partials per block into scratch.
template <typename T, int K>
__global__ void __launch_bounds__(kWarps * 32) ln_bwd_scratch_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                   const float* __restrict__ w,
                                                                   const float* __restrict__ mean_in,
                                                                   const float* __restrict__ rstd_in, T* __restrict__ dx,
                                                                   float* __restrict__ scratch, long long rows, int C) {
  extern __shared__ float smem[];  // [warps][2][C]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float aw[K], ab[K];
#pragma unroll
  for (int k = 0; k < K; ++k) aw[k] = ab[k] = 0.f;
  for (long long row = (long long)blockIdx.x * kWarps + warp; row < rows; row += (long long)gridDim.x * kWarps) {
    const T* xr = x + row * C;
    const T* gr = dy + row * C;
    const float mean = mean_in[row], rstd = rstd_in[row];
    float xh[K], g[K];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + 32 * k;
      xh[k] = g[k] = 0.f;
      if (c < C) {
        const float go = df3::to_float<T>(gr[c]);
        xh[k] = (df3::to_float<T>(xr[c]) - mean) * rstd;
        g[k] = w ? go * w[c] : go;
        aw[k] += go * xh[k];
        ab[k] += go;
        s1 += g[k];
        s2 += g[k] * xh[k];
      }
    }
    s1 = df3::warp_sum(s1) / C;
    s2 = df3::warp_sum(s2) / C;
    T* dr = dx + row * C;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int c = lane + 32 * k;
      if (c < C) dr[c] = df3::from_float<T>(rstd * (g[k] - s1 - xh[k] * s2));
    }
  }
  if (scratch == nullptr) return;
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
    for (int wi = 0; wi < kWarps; ++wi) s += smem[wi * 2 * C + i];
    scratch[(long long)blockIdx.x * 2 * C + i] = s;
  }
}

// dw[c] = sum_b scratch[b][0][c], db[c] = sum_b scratch[b][1][c], in block order (deterministic).
__global__ void ln_bwd_reduce_kernel(const float* __restrict__ scratch, float* __restrict__ dw, float* __restrict__ db,
                                     int blocks, int C) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * C) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += scratch[(long long)b * 2 * C + i];
  if (i < C) dw[i] = s; else db[i - C] = s;
}

template <typename T>
cudaError_t launch(const void* dy, const void* x, const float* w, const float* mean, const float* rstd, void* dx,
                   float* scratch, long long rows, int C, int blocks, cudaStream_t s) {
  const size_t smem = scratch ? (size_t)kWarps * 2 * C * sizeof(float) : 0;  // at most 32 KiB
#define DF3_GO(K)                                                                                                     \
  ln_bwd_scratch_kernel<T, K><<<blocks, kWarps * 32, smem, s>>>((const T*)dy, (const T*)x, w, mean, rstd, (T*)dx,     \
                                                                 scratch, rows, C)
  if (C <= 128) DF3_GO(4); else if (C <= 256) DF3_GO(8); else if (C <= 512) DF3_GO(16); else DF3_GO(32);
#undef DF3_GO
  return cudaGetLastError();
}

}  // namespace

extern "C" int df3_layer_norm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* mean,
                                          const float* rstd, void* dx, float* dw, float* db, long long rows, int channels,
                                          int is_bf16, void* stream) {
  t_error[0] = '\0';
  if (channels < 1 || channels > kMaxC) {
    snprintf(t_error, sizeof(t_error), "channels=%d is outside [1, %d], the size the static scratch array was built for",
             channels, kMaxC);
    return kNoAllocBadSize;
  }
  if (rows < 0) return fail(kNoAllocBadSize, "rows is negative");
  if (!dy || !x || !mean || !rstd || !dx) return fail(kNoAllocBadPointer, "dy, x, mean, rstd and dx are required");
  if ((dw == nullptr) != (db == nullptr)) return fail(kNoAllocBadPointer, "dw and db must be both given or both null");
  if (rows == 0) return kNoAllocOk;

  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (device < 0 || device >= kMaxDevices) return fail(kNoAllocBadDevice, "device ordinal beyond the scratch address table");
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[device] == nullptr) {  // first call on this device: look the array up once
      float* ptr = nullptr;
      e = cudaGetSymbolAddress((void**)&ptr, g_scratch);
      if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(scratch)");
      g_scratch_ptr[device] = ptr;
    }
    scratch = g_scratch_ptr[device];
  }
  cudaStream_t s = (cudaStream_t)stream;
  long long want = (rows + kWarps - 1) / kWarps;
  const int blocks = (int)(want < kMaxBlocks ? want : kMaxBlocks);
  float* part = dw ? scratch : nullptr;
  e = is_bf16 ? launch<__nv_bfloat16>(dy, x, w, mean, rstd, dx, part, rows, channels, blocks, s)
              : launch<float>(dy, x, w, mean, rstd, dx, part, rows, channels, blocks, s);
  if (e != cudaSuccess) return fail_cuda(e, "layer-norm backward launch");
  if (dw) {
    ln_bwd_reduce_kernel<<<(2 * channels + 255) / 256, 256, 0, s>>>(scratch, dw, db, blocks, channels);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, "partial-sum reduction launch");
  }
  return kNoAllocOk;
}

extern "C" const char* df3_no_alloc_last_error(void) { return t_error; }
