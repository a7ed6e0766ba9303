// Adaptive LayerNorm and gated residual of the diffusion transformer's training path, one pass each way.
//
//   ada_ln:          y = sigmoid(s) * LN(x) + t        LN without affine, statistics in fp32; s, t, y bf16; x fp32 or bf16
//   gated_residual:  y = a + sigmoid(z) * u            a, y fp32 or bf16; z, u bf16
//
// The PyTorch statement of a block issues a LayerNorm, a sigmoid, a multiply, an add and (because the residual stream is
// fp32 under autocast) one cast per consuming projection; these kernels read each operand once and write the bf16 tensor
// the projections consume. One warp per row, a lane owns pairs of consecutive channels (4- or 8-byte accesses). The
// backward kernels return the gradients of all operands in one pass (the gradient of t, respectively a, is the incoming
// gradient itself).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "common.cuh"

using torch::Tensor;

namespace df3 {
namespace {

constexpr int kMaxPairs = 16;  // pairs of channels per lane: rows of up to 2 * 32 * 16 = 1024 channels

template <typename T>
__device__ __forceinline__ float2 load2(const T* p);
template <>
__device__ __forceinline__ float2 load2<float>(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
template <>
__device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T>
__device__ __forceinline__ void store2(T* p, float a, float b);
template <>
__device__ __forceinline__ void store2<float>(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}
template <>
__device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// 2 ulp of fp32 from the fast divide: far below the bf16 rounding of every consumer, and a third of the instructions
__device__ __forceinline__ float sigmoid_exact(float v) { return __fdividef(1.f, 1.f + __expf(-v)); }

template <typename TX, int K>
__global__ void __launch_bounds__(128) ada_ln_fwd_kernel(const TX* __restrict__ x, const __nv_bfloat16* __restrict__ s,
                                                         const __nv_bfloat16* __restrict__ t, __nv_bfloat16* __restrict__ y,
                                                         float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                         int64_t rows, int C, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t base = row * C;
  // every load of the row is issued before the first reduction: the conditioning pairs wait in registers as raw bf16x2,
  // so a row pays the memory latency once instead of once per phase
  float2 v[K];
  __nv_bfloat162 sr[K], tr[K];
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = 2 * (lane + 32 * k);
    const bool in = c < C;
    v[k] = in ? load2<TX>(x + base + c) : make_float2(0.f, 0.f);
    sr[k] = in ? *reinterpret_cast<const __nv_bfloat162*>(s + base + c) : __nv_bfloat162();
    tr[k] = in ? *reinterpret_cast<const __nv_bfloat162*>(t + base + c) : __nv_bfloat162();
  }
#pragma unroll
  for (int k = 0; k < K; ++k) sum += v[k].x + v[k].y;
  const float mean = warp_sum(sum) / C;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = 2 * (lane + 32 * k);
    if (c < C) {
      const float dx = v[k].x - mean, dy = v[k].y - mean;
      q += dx * dx + dy * dy;
    }
  }
  const float rstd = rsqrtf(warp_sum(q) / C + eps);
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = 2 * (lane + 32 * k);
    if (c < C) {
      const float2 sv = __bfloat1622float2(sr[k]), tv = __bfloat1622float2(tr[k]);
      store2<__nv_bfloat16>(y + base + c, sigmoid_exact(sv.x) * (v[k].x - mean) * rstd + tv.x,
                            sigmoid_exact(sv.y) * (v[k].y - mean) * rstd + tv.y);
    }
  }
  if (lane == 0) {
    mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) with g = dy * sigmoid(s);  ds = dy * xhat * sig * (1 - sig)
template <typename TX, int K>
__global__ void __launch_bounds__(128) ada_ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const TX* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ s, const float* __restrict__ mean_in,
                                                         const float* __restrict__ rstd_in, TX* __restrict__ dx,
                                                         __nv_bfloat16* __restrict__ ds, int64_t rows, int C) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int64_t base = row * C;
  const float mean = mean_in[row], rstd = rstd_in[row];
  // all three operands of the row are requested before anything is computed or stored (one latency per row)
  float2 xh[K], g[K];
  __nv_bfloat162 gr[K], sr[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = 2 * (lane + 32 * k);
    const bool in = c < C;
    xh[k] = in ? load2<TX>(x + base + c) : make_float2(0.f, 0.f);  // a constant: the loads must not wait for the statistics
    gr[k] = in ? *reinterpret_cast<const __nv_bfloat162*>(dy + base + c) : __nv_bfloat162();
    sr[k] = in ? *reinterpret_cast<const __nv_bfloat162*>(s + base + c) : __nv_bfloat162();
  }
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = 2 * (lane + 32 * k);
    if (c < C) {
      const float2 gv = __bfloat1622float2(gr[k]), sv = __bfloat1622float2(sr[k]);
      xh[k] = make_float2((xh[k].x - mean) * rstd, (xh[k].y - mean) * rstd);
      const float ga = sigmoid_exact(sv.x), gb = sigmoid_exact(sv.y);
      store2<__nv_bfloat16>(ds + base + c, gv.x * xh[k].x * ga * (1.f - ga), gv.y * xh[k].y * gb * (1.f - gb));
      g[k] = make_float2(gv.x * ga, gv.y * gb);
      s1 += g[k].x + g[k].y;
      s2 += g[k].x * xh[k].x + g[k].y * xh[k].y;
    } else {
      xh[k] = g[k] = make_float2(0.f, 0.f);
    }
  }
  s1 = warp_sum(s1) / C;
  s2 = warp_sum(s2) / C;
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const int c = 2 * (lane + 32 * k);
    if (c < C) store2<TX>(dx + base + c, rstd * (g[k].x - s1 - xh[k].x * s2), rstd * (g[k].y - s1 - xh[k].y * s2));
  }
}

template <typename TA>
__global__ void __launch_bounds__(256) gated_residual_fwd_kernel(const TA* __restrict__ a, const __nv_bfloat16* __restrict__ z,
                                                                 const __nv_bfloat16* __restrict__ u, TA* __restrict__ y,
                                                                 int64_t pairs) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
    const float2 av = load2<TA>(a + 2 * i), zv = load2<__nv_bfloat16>(z + 2 * i), uv = load2<__nv_bfloat16>(u + 2 * i);
    store2<TA>(y + 2 * i, av.x + sigmoid_exact(zv.x) * uv.x, av.y + sigmoid_exact(zv.y) * uv.y);
  }
}

template <typename TG>
__global__ void __launch_bounds__(256) gated_residual_bwd_kernel(const TG* __restrict__ dy, const __nv_bfloat16* __restrict__ z,
                                                                 const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ dz,
                                                                 __nv_bfloat16* __restrict__ du, int64_t pairs) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs; i += (int64_t)gridDim.x * blockDim.x) {
    const float2 gv = load2<TG>(dy + 2 * i), zv = load2<__nv_bfloat16>(z + 2 * i), uv = load2<__nv_bfloat16>(u + 2 * i);
    const float ga = sigmoid_exact(zv.x), gb = sigmoid_exact(zv.y);
    store2<__nv_bfloat16>(dz + 2 * i, gv.x * uv.x * ga * (1.f - ga), gv.y * uv.y * gb * (1.f - gb));
    store2<__nv_bfloat16>(du + 2 * i, gv.x * ga, gv.y * gb);
  }
}

void check_rows(const Tensor& x, const Tensor& s, const char* what) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && s.is_contiguous() && s.sizes() == x.sizes(), what, ": contiguous CUDA tensors of one shape");
  TORCH_CHECK(x.scalar_type() == torch::kFloat32 || x.scalar_type() == torch::kBFloat16, what, ": x must be fp32 or bf16");
  TORCH_CHECK(s.scalar_type() == torch::kBFloat16, what, ": the conditioning tensors must be bf16");
  const int64_t C = x.size(-1);
  TORCH_CHECK(C % 2 == 0 && C >= 2 && C <= 2 * 32 * kMaxPairs, what, ": even channel count up to ", 2 * 32 * kMaxPairs);
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 8 == 0 && reinterpret_cast<uintptr_t>(s.data_ptr()) % 4 == 0, what, ": misaligned");
}

std::tuple<Tensor, Tensor, Tensor> ada_ln_fwd(const Tensor& x, const Tensor& s, const Tensor& t, double eps) {
  check_rows(x, s, "ada_ln_fwd");
  TORCH_CHECK(t.is_contiguous() && t.sizes() == x.sizes() && t.scalar_type() == torch::kBFloat16, "ada_ln_fwd: t like s");
  c10::cuda::CUDAGuard guard(x.device());
  const int C = (int)x.size(-1);
  const int64_t rows = x.numel() / C;
  Tensor y = torch::empty_like(s);
  Tensor mean = torch::empty({rows}, x.options().dtype(torch::kFloat32)), rstd = torch::empty_like(mean);
  if (rows == 0) return {y, mean, rstd};
  const unsigned grid = (unsigned)((rows + 3) / 4);  // four warps, one row each: small blocks keep more rows resident at ~95 registers
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  const int pairs = (C / 2 + 31) / 32;
#define DF3_ADA_FWD(TX, K_)                                                                                                  \
  ada_ln_fwd_kernel<TX, K_><<<grid, 128, 0, st>>>((const TX*)x.data_ptr(), (const __nv_bfloat16*)s.data_ptr(),              \
                                                  (const __nv_bfloat16*)t.data_ptr(), (__nv_bfloat16*)y.data_ptr(),         \
                                                  mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, C, (float)eps)
  if (x.scalar_type() == torch::kFloat32) {
    if (pairs <= 4) DF3_ADA_FWD(float, 4); else if (pairs <= 8) DF3_ADA_FWD(float, 8); else if (pairs <= 12) DF3_ADA_FWD(float, 12); else DF3_ADA_FWD(float, 16);
  } else {
    if (pairs <= 4) DF3_ADA_FWD(__nv_bfloat16, 4); else if (pairs <= 8) DF3_ADA_FWD(__nv_bfloat16, 8); else if (pairs <= 12) DF3_ADA_FWD(__nv_bfloat16, 12); else DF3_ADA_FWD(__nv_bfloat16, 16);
  }
#undef DF3_ADA_FWD
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, mean, rstd};
}

std::tuple<Tensor, Tensor> ada_ln_bwd(const Tensor& dy, const Tensor& x, const Tensor& s, const Tensor& mean, const Tensor& rstd) {
  check_rows(x, s, "ada_ln_bwd");
  TORCH_CHECK(dy.is_contiguous() && dy.sizes() == x.sizes() && dy.scalar_type() == torch::kBFloat16, "ada_ln_bwd: dy bf16 like x");
  c10::cuda::CUDAGuard guard(x.device());
  const int C = (int)x.size(-1);
  const int64_t rows = x.numel() / C;
  TORCH_CHECK(mean.numel() == rows && rstd.numel() == rows && mean.scalar_type() == torch::kFloat32, "ada_ln_bwd: statistics per row");
  Tensor dx = torch::empty_like(x), ds = torch::empty_like(s);
  if (rows == 0) return {dx, ds};
  const unsigned grid = (unsigned)((rows + 3) / 4);  // four warps, one row each: small blocks keep more rows resident at ~95 registers
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  const int pairs = (C / 2 + 31) / 32;
#define DF3_ADA_BWD(TX, K_)                                                                                                  \
  ada_ln_bwd_kernel<TX, K_><<<grid, 128, 0, st>>>((const __nv_bfloat16*)dy.data_ptr(), (const TX*)x.data_ptr(),             \
                                                  (const __nv_bfloat16*)s.data_ptr(), mean.data_ptr<float>(),               \
                                                  rstd.data_ptr<float>(), (TX*)dx.data_ptr(), (__nv_bfloat16*)ds.data_ptr(), rows, C)
  if (x.scalar_type() == torch::kFloat32) {
    if (pairs <= 4) DF3_ADA_BWD(float, 4); else if (pairs <= 8) DF3_ADA_BWD(float, 8); else if (pairs <= 12) DF3_ADA_BWD(float, 12); else DF3_ADA_BWD(float, 16);
  } else {
    if (pairs <= 4) DF3_ADA_BWD(__nv_bfloat16, 4); else if (pairs <= 8) DF3_ADA_BWD(__nv_bfloat16, 8); else if (pairs <= 12) DF3_ADA_BWD(__nv_bfloat16, 12); else DF3_ADA_BWD(__nv_bfloat16, 16);
  }
#undef DF3_ADA_BWD
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, ds};
}

void check_flat(const Tensor& a, const Tensor& z, const Tensor& u, const char* what) {
  TORCH_CHECK(a.is_cuda() && a.is_contiguous() && z.is_contiguous() && u.is_contiguous() && z.sizes() == a.sizes() && u.sizes() == a.sizes(),
              what, ": contiguous CUDA tensors of one shape");
  TORCH_CHECK(a.scalar_type() == torch::kFloat32 || a.scalar_type() == torch::kBFloat16, what, ": first operand fp32 or bf16");
  TORCH_CHECK(z.scalar_type() == torch::kBFloat16 && u.scalar_type() == torch::kBFloat16, what, ": gate and update bf16");
  TORCH_CHECK(a.numel() % 2 == 0 && reinterpret_cast<uintptr_t>(a.data_ptr()) % 8 == 0 && reinterpret_cast<uintptr_t>(z.data_ptr()) % 4 == 0 &&
              reinterpret_cast<uintptr_t>(u.data_ptr()) % 4 == 0, what, ": even size, aligned");
}

unsigned flat_grid(int64_t pairs) { return (unsigned)std::min<int64_t>((pairs + 255) / 256, 148 * 16); }

Tensor gated_residual_fwd(const Tensor& a, const Tensor& z, const Tensor& u) {
  check_flat(a, z, u, "gated_residual_fwd");
  c10::cuda::CUDAGuard guard(a.device());
  Tensor y = torch::empty_like(a);
  const int64_t pairs = a.numel() / 2;
  if (pairs == 0) return y;
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  if (a.scalar_type() == torch::kFloat32)
    gated_residual_fwd_kernel<float><<<flat_grid(pairs), 256, 0, st>>>(a.data_ptr<float>(), (const __nv_bfloat16*)z.data_ptr(),
                                                                      (const __nv_bfloat16*)u.data_ptr(), y.data_ptr<float>(), pairs);
  else
    gated_residual_fwd_kernel<__nv_bfloat16><<<flat_grid(pairs), 256, 0, st>>>((const __nv_bfloat16*)a.data_ptr(), (const __nv_bfloat16*)z.data_ptr(),
                                                                              (const __nv_bfloat16*)u.data_ptr(), (__nv_bfloat16*)y.data_ptr(), pairs);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

std::tuple<Tensor, Tensor> gated_residual_bwd(const Tensor& dy, const Tensor& z, const Tensor& u) {
  check_flat(dy, z, u, "gated_residual_bwd");
  c10::cuda::CUDAGuard guard(dy.device());
  Tensor dz = torch::empty_like(z), du = torch::empty_like(u);
  const int64_t pairs = dy.numel() / 2;
  if (pairs == 0) return {dz, du};
  cudaStream_t st = at::cuda::getCurrentCUDAStream();
  if (dy.scalar_type() == torch::kFloat32)
    gated_residual_bwd_kernel<float><<<flat_grid(pairs), 256, 0, st>>>(dy.data_ptr<float>(), (const __nv_bfloat16*)z.data_ptr(),
                                                                      (const __nv_bfloat16*)u.data_ptr(), (__nv_bfloat16*)dz.data_ptr(),
                                                                      (__nv_bfloat16*)du.data_ptr(), pairs);
  else
    gated_residual_bwd_kernel<__nv_bfloat16><<<flat_grid(pairs), 256, 0, st>>>((const __nv_bfloat16*)dy.data_ptr(), (const __nv_bfloat16*)z.data_ptr(),
                                                                              (const __nv_bfloat16*)u.data_ptr(), (__nv_bfloat16*)dz.data_ptr(),
                                                                              (__nv_bfloat16*)du.data_ptr(), pairs);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dz, du};
}

}  // namespace
}  // namespace df3

void df3_register_ada_norm(torch::Library& m) {
  m.def("ada_ln_fwd(Tensor x, Tensor s, Tensor t, float eps) -> (Tensor, Tensor, Tensor)", &df3::ada_ln_fwd);
  m.def("ada_ln_bwd(Tensor dy, Tensor x, Tensor s, Tensor mean, Tensor rstd) -> (Tensor, Tensor)", &df3::ada_ln_bwd);
  m.def("gated_residual_fwd(Tensor a, Tensor z, Tensor u) -> Tensor", &df3::gated_residual_fwd);
  m.def("gated_residual_bwd(Tensor dy, Tensor z, Tensor u) -> (Tensor, Tensor)", &df3::gated_residual_bwd);
}
