// Shared device helpers for the sm_100a kernels: type conversion, warp/block reductions,
// Philox counter RNG, and the status word every bounded wait reports through.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace df3 {

// Error codes written to a kernel's status word. A kernel never traps or spins forever:
// a wait that runs out of iterations records where it gave up and the kernel returns.
enum Status : int {
  kOk = 0,
  kTimeoutTmaFull = 1,    // consumer waited for a TMA-filled stage
  kTimeoutStageEmpty = 2, // producer waited for a free stage
  kTimeoutMmaDone = 3,    // epilogue waited for the accumulator
  kTimeoutPeerFlag = 4,   // waited for another GPU's flag
  kBadShape = 5,
};

// Debug build (-DDF3_BOUNDS_CHECK, `python -m deepfold3_dev_b200.ops.build --checked`): global accesses whose index a
// kernel computes go through this test. An index outside [0, limit) records kBadShape in the status word and the
// access is skipped; nothing traps. In the normal build the test is the constant true and costs nothing.
#ifdef DF3_BOUNDS_CHECK
__device__ __forceinline__ bool in_bounds(long long idx, long long limit, int* status) {
  if (idx >= 0 && idx < limit) return true;
  if (status != nullptr) atomicCAS(status, (int)kOk, (int)kBadShape);
  return false;
}
#else
__device__ __forceinline__ bool in_bounds(long long, long long, int*) { return true; }
#endif

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; `smem` holds 32 floats. Result valid in every thread.
__device__ __forceinline__ float block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  const int nwarp = (blockDim.x + 31) >> 5;
  float r = (threadIdx.x < nwarp) ? smem[threadIdx.x] : 0.f;
  if (warp == 0) {
    r = warp_sum(r);
    if (lane == 0) smem[0] = r;
  }
  __syncthreads();
  return smem[0];
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// sigmoid(x) = 0.5 tanh(x / 2) + 0.5 with the hardware tanh: one special-function op instead of two (exp and
// reciprocal); absolute error about 5e-4 of the result's unit range, below the bf16 rounding of the values it gates.
__device__ __forceinline__ float sigmoid_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}

// Philox-4x32-10: counter-based generator, the same family torch uses for CUDA dropout.
struct Philox {
  uint32_t key0, key1;
  __device__ __forceinline__ Philox(uint64_t seed) : key0((uint32_t)seed), key1((uint32_t)(seed >> 32)) {}
  __device__ __forceinline__ static void mulhilo(uint32_t a, uint32_t b, uint32_t& hi, uint32_t& lo) {
    const uint64_t p = (uint64_t)a * b;
    hi = (uint32_t)(p >> 32);
    lo = (uint32_t)p;
  }
  __device__ __forceinline__ uint4 operator()(uint64_t counter, uint64_t subseq) const {
    uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = (uint32_t)subseq, c3 = (uint32_t)(subseq >> 32);
    uint32_t k0 = key0, k1 = key1;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      uint32_t h0, l0, h1, l1;
      mulhilo(0xD2511F53u, c0, h0, l0);
      mulhilo(0xCD9E8D57u, c2, h1, l1);
      const uint32_t n0 = h1 ^ c1 ^ k0, n1 = l1, n2 = h0 ^ c3 ^ k1, n3 = l0;
      c0 = n0; c1 = n1; c2 = n2; c3 = n3;
      k0 += 0x9E3779B9u;
      k1 += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
  }
};

__device__ __forceinline__ float uniform01(uint32_t bits) { return (bits >> 8) * (1.0f / 16777216.0f); }

}  // namespace df3
