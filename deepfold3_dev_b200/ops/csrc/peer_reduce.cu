// Gradient all-reduce over NVLink peer memory, fused with the per-rank clip scaling, the averaging and
// the squared norm of the result.
//
// Every rank's flat fp32 gradient lives in symmetric memory, so each GPU holds a pointer to every
// peer's buffer. Rank r owns slice r. In one launch it reads its slice from all W ranks with plain
// peer loads (16 bytes per thread, W loads in flight), scales each by that rank's clip coefficient,
// averages, accumulates the squared norm and writes the averaged slice back into all W buffers with
// peer stores: reduce-scatter, all-gather and the norm in a single pass over the data. The block
// that finishes last publishes this rank's partial squared norm and a sequence flag into every peer's
// control block. A second, tiny kernel waits (bounded) until all W flags of this step arrived, which
// also means every peer's slice has landed here, and writes sqrt(sum of partials).
//
// No multimem / NVLS and no TMA is used: plain loads and stores keep the kernel safe when a peer
// process has gone away between steps, and it travels to any number of GPUs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "common.cuh"

using torch::Tensor;

namespace df3 {
namespace {

constexpr int kMaxWorld = 16;
constexpr int64_t kDefaultSpinLimit = 20 * 1000 * 1000;  // polls (each sleeps ~64 ns) of a local word: about two seconds, then give up

// Layout of the symmetric control block of one rank (all offsets in bytes).
constexpr int kCoefOff = 0;      // float: this rank's clip coefficient, read by peers
constexpr int kSlotsOff = 64;    // double[kMaxWorld]: partial squared norms, slot s written by rank s
constexpr int kFlagsOff = 256;   // unsigned long long[kMaxWorld]: sequence numbers, slot s written by rank s
constexpr int kCtrlBytes = 512;

struct Peers {
  float* grad[kMaxWorld];
  unsigned char* ctrl[kMaxWorld];
};

// local scratch: [0] double block accumulator, [1] as unsigned: blocks done
__global__ void __launch_bounds__(512) peer_reduce_kernel(Peers peers, double* __restrict__ acc, unsigned int* __restrict__ done,
                                                        long long begin4, long long end4, int rank, int world,
                                                        unsigned long long seq) {
  __shared__ float red[32];
  float coef[kMaxWorld];
#pragma unroll
  for (int r = 0; r < kMaxWorld; ++r)
    coef[r] = r < world ? *reinterpret_cast<const volatile float*>(peers.ctrl[r] + kCoefOff) : 0.f;
  const float inv_world = 1.f / (float)world;
  float sumsq = 0.f;
  for (long long i = begin4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < end4; i += (long long)gridDim.x * blockDim.x) {
    float4 v[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < world) v[r] = reinterpret_cast<const float4*>(peers.grad[r])[i];
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < world) {
        s.x += coef[r] * v[r].x; s.y += coef[r] * v[r].y; s.z += coef[r] * v[r].z; s.w += coef[r] * v[r].w;
      }
    s.x *= inv_world; s.y *= inv_world; s.z *= inv_world; s.w *= inv_world;
    sumsq += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r)
      if (r < world) reinterpret_cast<float4*>(peers.grad[r])[i] = s;
  }
  const float block_total = block_sum(sumsq, red);
  __threadfence_system();  // this block's peer stores are visible before it counts itself done
  if (threadIdx.x == 0) {
    atomicAdd(acc, (double)block_total);
    __threadfence();
    const unsigned int before = atomicAdd(done, 1u);
    if (before == gridDim.x - 1) {  // last block of this rank: publish partial norm, then the flag
      __threadfence();
      const double total = *reinterpret_cast<volatile double*>(acc);
      for (int r = 0; r < world; ++r) reinterpret_cast<volatile double*>(peers.ctrl[r] + kSlotsOff)[rank] = total;
      __threadfence_system();
      for (int r = 0; r < world; ++r) reinterpret_cast<volatile unsigned long long*>(peers.ctrl[r] + kFlagsOff)[rank] = seq;
      *acc = 0.0;
      *done = 0u;
    }
  }
}

// Waits for the flags of all ranks, then norm = sqrt(sum of partial squared norms). status: kTimeoutPeerFlag on give-up.
__global__ void peer_norm_kernel(const unsigned char* __restrict__ ctrl, float* __restrict__ norm_out, int* __restrict__ status,
                                 int world, unsigned long long seq, unsigned int spin_limit) {
  const int r = threadIdx.x;
  bool ok = true;
  if (r < world) {
    const volatile unsigned long long* flag = reinterpret_cast<const volatile unsigned long long*>(ctrl + kFlagsOff) + r;
    uint32_t spins = 0;
    while (*flag < seq) {
      if (++spins > spin_limit) { ok = false; break; }
      __nanosleep(64);
    }
  }
  const int all_ok = __syncthreads_and(ok ? 1 : 0);
  if (threadIdx.x == 0) {
    if (!all_ok) {
      atomicCAS(status, kOk, kTimeoutPeerFlag);
      *norm_out = __int_as_float(0x7fc00000);  // NaN: the step is skipped by the caller's finite check
    } else {
      __threadfence_system();
      double total = 0.0;
      for (int s = 0; s < world; ++s) total += reinterpret_cast<const volatile double*>(ctrl + kSlotsOff)[s];
      *norm_out = (float)sqrt(total);
    }
  }
}

// grad: this rank's symmetric flat gradient (numel % 4 == 0); grad_ptrs / ctrl_ptrs: peer addresses by rank;
// scratch: local 16 zero bytes (double + counter); returns the norm of the averaged gradient (fp32 scalar tensor).
Tensor df3_peer_allreduce_mean(Tensor grad, const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& ctrl_ptrs,
                               Tensor scratch, Tensor status, int64_t rank, int64_t world, int64_t seq, int64_t spin_limit) {
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == torch::kFloat32 && grad.is_contiguous() && grad.numel() % 4 == 0,
              "peer_allreduce_mean: contiguous fp32 CUDA buffer, numel % 4 == 0");
  TORCH_CHECK(world >= 1 && world <= kMaxWorld && (int64_t)grad_ptrs.size() == world && (int64_t)ctrl_ptrs.size() == world &&
              rank >= 0 && rank < world, "peer_allreduce_mean: world size / pointer lists");
  TORCH_CHECK(scratch.is_cuda() && scratch.numel() * scratch.element_size() >= 16 && status.scalar_type() == torch::kInt32,
              "peer_allreduce_mean: scratch of 16 bytes and an int32 status word");
  TORCH_CHECK((uintptr_t)grad_ptrs[rank] == (uintptr_t)grad.data_ptr(), "peer_allreduce_mean: own pointer mismatch");
  c10::cuda::CUDAGuard guard(grad.device());
  Peers peers{};
  for (int r = 0; r < world; ++r) {
    peers.grad[r] = reinterpret_cast<float*>(grad_ptrs[r]);
    peers.ctrl[r] = reinterpret_cast<unsigned char*>(ctrl_ptrs[r]);
  }
  const long long n4 = grad.numel() / 4;
  const long long per = (n4 + world - 1) / world;
  const long long begin4 = std::min<long long>(n4, per * rank), end4 = std::min<long long>(n4, per * (rank + 1));
  Tensor norm = torch::empty({}, grad.options());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  auto* acc = reinterpret_cast<double*>(scratch.data_ptr());
  auto* done = reinterpret_cast<unsigned int*>(reinterpret_cast<unsigned char*>(scratch.data_ptr()) + 8);
  const int blocks = 148 * 2;
  peer_reduce_kernel<<<blocks, 512, 0, stream>>>(peers, acc, done, begin4, end4, (int)rank, (int)world, (unsigned long long)seq);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  peer_norm_kernel<<<1, 32, 0, stream>>>(peers.ctrl[rank], norm.data_ptr<float>(), status.data_ptr<int>(), (int)world,
                                        (unsigned long long)seq,
                                        (unsigned int)(spin_limit > 0 ? spin_limit : kDefaultSpinLimit));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return norm;
}

}  // namespace
}  // namespace df3

void df3_register_peer(torch::Library& m) {
  m.def("peer_allreduce_mean(Tensor(a!) grad, int[] grad_ptrs, int[] ctrl_ptrs, Tensor(b!) scratch, Tensor(c!) status, int rank, "
        "int world, int seq, int spin_limit=0) -> Tensor", &df3::df3_peer_allreduce_mean);
}
