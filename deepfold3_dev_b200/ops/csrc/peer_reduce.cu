// Gradient all-reduce over NVLink peer memory, fused with the per-rank clip scaling, the averaging and
// the squared norm of the result.
//
// Every rank's flat fp32 gradient lives in symmetric memory, so each GPU holds a pointer to every
// peer's buffer. Rank r owns slice r. In one launch it reads its slice from all W ranks with plain
// peer loads (16 bytes per thread, W loads in flight), scales each by that rank's clip coefficient,
// averages, accumulates the squared norm and writes the averaged slice back into all W buffers with
// peer stores: reduce-scatter, all-gather and the norm in a single pass over the data. The block
// that finishes last publishes this rank's partial squared norm and a sequence flag into every peer's
// control block. A one-warp kernel in front makes "every rank's gradient is final" known (its own bounded
// arrive / wait on the control blocks, no library barrier), and a second one behind waits (bounded) until
// all W flags of this step arrived, which also means every peer's slice has landed here, and writes
// sqrt(sum of partials). peer_fused_step_kernel further down folds all of it, the skip consensus and the
// AdamW + EMA update into one cooperative launch.
//
// No multimem / NVLS and no TMA is used: plain loads and stores keep the kernel safe when a peer
// process has gone away between steps, and it travels to any number of GPUs.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <cstring>
#include <initializer_list>

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
constexpr int kArriveOff = 384;  // unsigned long long[kMaxWorld]: entry sequence numbers, slot s written by rank s
constexpr int kCtrlBytes = 1024;

struct Peers {
  float* grad[kMaxWorld];
  unsigned char* ctrl[kMaxWorld];
};

// local scratch: [0] double block accumulator, [1] as unsigned: blocks done
__global__ void __launch_bounds__(512) peer_reduce_kernel(Peers peers, double* __restrict__ acc, unsigned int* __restrict__ done,
                                                        const int* __restrict__ status, long long begin4, long long end4, int rank,
                                                        int world, unsigned long long seq) {
  __shared__ float red[32];
  if (*reinterpret_cast<const volatile int*>(status) != kOk) return;  // the entry wait ran out: touch no peer memory
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

// Entry of a reduction: tell every peer that this rank's gradient and clip coefficient are final (sequence number into
// the peer's control block), then wait, bounded, for the same word from every peer. A wait that runs out records
// kTimeoutPeerFlag; the kernels that follow on the stream see the status and leave peer memory alone.
__global__ void peer_entry_kernel(Peers peers, int* __restrict__ status, int rank, int world, unsigned long long seq,
                                  unsigned int spin_limit) {
  const int r = threadIdx.x;
  bool ok = true;
  if (r < world) {
    __threadfence_system();
    reinterpret_cast<volatile unsigned long long*>(peers.ctrl[r] + kArriveOff)[rank] = seq;
    const volatile unsigned long long* flag = reinterpret_cast<const volatile unsigned long long*>(peers.ctrl[rank] + kArriveOff) + r;
    uint32_t spins = 0;
    while (*flag < seq) {
      if (++spins > spin_limit) { ok = false; break; }
      __nanosleep(64);
    }
  }
  if (!__syncthreads_and(ok ? 1 : 0) && threadIdx.x == 0) atomicCAS(status, kOk, kTimeoutPeerFlag);
  __threadfence_system();
}

// Waits for the flags of all ranks, then norm = sqrt(sum of partial squared norms). status: kTimeoutPeerFlag on give-up.
__global__ void peer_norm_kernel(const unsigned char* __restrict__ ctrl, float* __restrict__ norm_out, int* __restrict__ status,
                                 int world, unsigned long long seq, unsigned int spin_limit) {
  const int r = threadIdx.x;
  bool ok = *reinterpret_cast<const volatile int*>(status) == kOk;  // an entry wait that ran out ends the step
  if (ok && r < world) {
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
  const unsigned int spin = (unsigned int)(spin_limit > 0 ? spin_limit : kDefaultSpinLimit);
  peer_entry_kernel<<<1, 32, 0, stream>>>(peers, status.data_ptr<int>(), (int)rank, (int)world, (unsigned long long)seq, spin);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  peer_reduce_kernel<<<blocks, 512, 0, stream>>>(peers, acc, done, status.data_ptr<int>(), begin4, end4, (int)rank, (int)world,
                                                 (unsigned long long)seq);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  peer_norm_kernel<<<1, 32, 0, stream>>>(peers.ctrl[rank], norm.data_ptr<float>(), status.data_ptr<int>(), (int)world,
                                        (unsigned long long)seq, spin);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return norm;
}


// ---------------------------------------------------------------------------------------------------------------
// One kernel for the whole data-parallel optimizer step (what the reference does with two barriers, two all-gathers,
// an all-reduce, a clip, fused AdamW and a foreach lerp: training/optim.py:576-765, training/ema.py:77-90):
//
//   phase 0  entry: this rank tells every peer "my gradient, clip coefficient and loss flag are final" (a sequence
//            number stored into each peer's control block) and waits, bounded, for the same word from all peers
//   phase 1  reduce-scatter + scale + average + squared norm + all-gather of the gradient, as peer_reduce_kernel;
//            the last block publishes the partial norm, this rank's loss flag and local norm, then its done flag
//   phase 2  every block waits, bounded, for all done flags; all ranks now hold the same reduced gradient, the same
//            norm and the same per-rank flags, so each takes the same skip / clip decision on the device and, unless
//            the step is skipped, runs AdamW + EMA + bf16 mirror over its (replicated) parameters; the gradient
//            buffer is zeroed on the way for the next accumulation window
//
// No NCCL call and no host read sits between backward and the next forward; the host learns the outcome from a
// small result block that it copies back asynchronously. All blocks wait on flags that other blocks of the same
// grid publish, so the launch is cooperative (the whole grid is resident). World size 1 runs the same kernel.
constexpr int kInfoOff = 512;     // float2[kMaxWorld]: (loss flag, local norm) of rank s, written by rank s
constexpr int kCtrlBytesV2 = 1024;
constexpr int kLossFlagOff = 4;   // float: this rank's non-finite-loss flag
constexpr int kLocalNormOff = 8;  // float: this rank's pre-clip gradient norm

struct StepArgs {
  float4* p; float4* m; float4* v; float4* ema; const float4* decay; uint2* p16;
  float lr, b1, b2, eps, bc1, bc2_sqrt, ema_w;
  float clip_norm;        // <= 0: no clipping
  float skip_threshold;   // <= 0: off
  int per_rank_clip;
  long long n4;
};

// Bounded wait until every rank's word at `off` reached seq. Returns false on timeout (uniform over the block).
__device__ __forceinline__ bool wait_all_ranks(const unsigned char* ctrl, int off, int world, unsigned long long seq, unsigned int spin_limit) {
  bool ok = true;
  if ((int)threadIdx.x < world) {
    const volatile unsigned long long* flag = reinterpret_cast<const volatile unsigned long long*>(ctrl + off) + threadIdx.x;
    unsigned int spins = 0;
    while (*flag < seq) {
      if (++spins > spin_limit) { ok = false; break; }
      __nanosleep(64);
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__global__ void __launch_bounds__(512) peer_fused_step_kernel(Peers peers, StepArgs a, double* __restrict__ acc,
                                                            unsigned int* __restrict__ done, float* __restrict__ result,
                                                            int* __restrict__ status, long long begin4, long long end4, int rank,
                                                            int world, unsigned long long seq, unsigned int spin_limit) {
  __shared__ float red[32];
  unsigned char* my_ctrl = peers.ctrl[rank];
  // ---- phase 0
  if (blockIdx.x == 0 && (int)threadIdx.x < world) {
    __threadfence_system();
    reinterpret_cast<volatile unsigned long long*>(peers.ctrl[threadIdx.x] + kArriveOff)[rank] = seq;
  }
  if (!wait_all_ranks(my_ctrl, kArriveOff, world, seq, spin_limit)) {
    if (threadIdx.x == 0) {
      atomicCAS(status, kOk, kTimeoutPeerFlag);
      if (blockIdx.x == 0) { result[0] = 0.f; result[1] = 3.f; result[2] = __int_as_float(0x7fc00000); }
    }
    return;  // nothing of any peer was read or written
  }
  __threadfence_system();
  // ---- phase 1
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
  __threadfence_system();
  if (threadIdx.x == 0) {
    atomicAdd(acc, (double)block_total);
    __threadfence();
    const unsigned int before = atomicAdd(done, 1u);
    if (before == gridDim.x - 1) {
      __threadfence();
      const double total = *reinterpret_cast<volatile double*>(acc);
      const float lf = *reinterpret_cast<const volatile float*>(my_ctrl + kLossFlagOff);
      const float ln = *reinterpret_cast<const volatile float*>(my_ctrl + kLocalNormOff);
      for (int r = 0; r < world; ++r) {
        reinterpret_cast<volatile double*>(peers.ctrl[r] + kSlotsOff)[rank] = total;
        volatile float* info = reinterpret_cast<volatile float*>(peers.ctrl[r] + kInfoOff) + 2 * rank;
        info[0] = lf;
        info[1] = ln;
      }
      __threadfence_system();
      for (int r = 0; r < world; ++r) reinterpret_cast<volatile unsigned long long*>(peers.ctrl[r] + kFlagsOff)[rank] = seq;
      *acc = 0.0;
      *done = 0u;
    }
  }
  // ---- phase 2
  if (!wait_all_ranks(my_ctrl, kFlagsOff, world, seq, spin_limit)) {
    if (threadIdx.x == 0) {
      atomicCAS(status, kOk, kTimeoutPeerFlag);
      if (blockIdx.x == 0) { result[0] = 0.f; result[1] = 3.f; result[2] = __int_as_float(0x7fc00000); }
    }
    return;
  }
  __threadfence_system();
  double total = 0.0;
  bool bad_loss = false, bad_grad = false;
  for (int s = 0; s < world; ++s) {
    total += reinterpret_cast<const volatile double*>(my_ctrl + kSlotsOff)[s];
    const volatile float* info = reinterpret_cast<const volatile float*>(my_ctrl + kInfoOff) + 2 * s;
    const float lf = info[0], ln = info[1];
    bad_loss = bad_loss || !(lf == 0.f);
    if (a.per_rank_clip) bad_grad = bad_grad || !isfinite(ln) || (a.skip_threshold > 0.f && ln > a.skip_threshold);
  }
  const float norm = (float)sqrt(total);
  bad_grad = bad_grad || !isfinite(norm) || (!a.per_rank_clip && a.skip_threshold > 0.f && norm > a.skip_threshold);
  const bool skip = bad_loss || bad_grad;
  float scale = 1.f;
  if (!a.per_rank_clip && a.clip_norm > 0.f) scale = fminf(1.f, a.clip_norm / (norm + 1e-6f));
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    result[0] = skip ? 0.f : 1.f;
    result[1] = bad_loss ? 1.f : (bad_grad ? 2.f : 0.f);
    result[2] = norm;
    result[3] = scale;
    for (int s = 0; s < world; ++s) {
      const volatile float* info = reinterpret_cast<const volatile float*>(my_ctrl + kInfoOff) + 2 * s;
      result[4 + s] = info[0];
      result[4 + kMaxWorld + s] = info[1];
    }
  }
  float4* g = reinterpret_cast<float4*>(peers.grad[rank]);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n4; i += (long long)gridDim.x * blockDim.x) {
    if (skip) {
      g[i] = zero;
      continue;
    }
    float4 pp = a.p[i], gg = g[i], mm = a.m[i], vv = a.v[i], dd = a.decay[i];
    g[i] = zero;
    float* P = &pp.x; float* G = &gg.x; float* M = &mm.x; float* V = &vv.x; float* D = &dd.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float gk = G[k] * scale;
      float pk = P[k] * (1.f - a.lr * D[k]);
      M[k] = M[k] + (gk - M[k]) * (1.f - a.b1);
      V[k] = V[k] * a.b2 + gk * gk * (1.f - a.b2);
      pk -= (a.lr / a.bc1) * M[k] / (sqrtf(V[k]) / a.bc2_sqrt + a.eps);
      P[k] = pk;
    }
    a.p[i] = pp; a.m[i] = mm; a.v[i] = vv;
    if (a.p16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp.x, pp.y), hi = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 w;
      w.x = *reinterpret_cast<uint32_t*>(&lo);
      w.y = *reinterpret_cast<uint32_t*>(&hi);
      a.p16[i] = w;
    }
    if (a.ema) {
      float4 ee = a.ema[i];
      ee.x += (pp.x - ee.x) * a.ema_w; ee.y += (pp.y - ee.y) * a.ema_w;
      ee.z += (pp.z - ee.z) * a.ema_w; ee.w += (pp.w - ee.w) * a.ema_w;
      a.ema[i] = ee;
    }
  }
}

// The whole optimizer step of one rank. `ctrl` of this rank must already hold its clip coefficient (offset 0), loss
// flag (offset 4) and local norm (offset 8), written by earlier work on the same stream. `result` (>= 4 + 2 * 16
// floats): [advanced, reason (0 none, 1 loss, 2 gradient, 3 wait ran out), norm of the averaged gradient, clip scale,
// loss flags by rank, local norms by rank].
void df3_peer_fused_step(Tensor grad, const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& ctrl_ptrs, Tensor scratch,
                         Tensor status, Tensor result, Tensor p, Tensor m, Tensor v, const c10::optional<Tensor>& ema,
                         const Tensor& decay, const c10::optional<Tensor>& p16, int64_t rank, int64_t world, int64_t seq,
                         double lr, double b1, double b2, double eps, double bc1, double bc2, double ema_w, double clip_norm,
                         double skip_threshold, bool per_rank_clip, int64_t spin_limit) {
  TORCH_CHECK(grad.is_cuda() && grad.scalar_type() == torch::kFloat32 && grad.is_contiguous() && grad.numel() % 4 == 0,
              "peer_fused_step: contiguous fp32 CUDA gradient, numel % 4 == 0");
  TORCH_CHECK(world >= 1 && world <= kMaxWorld && (int64_t)grad_ptrs.size() == world && (int64_t)ctrl_ptrs.size() == world &&
              rank >= 0 && rank < world, "peer_fused_step: world size / pointer lists");
  TORCH_CHECK((uintptr_t)grad_ptrs[rank] == (uintptr_t)grad.data_ptr(), "peer_fused_step: own pointer mismatch");
  for (const Tensor* t : std::initializer_list<const Tensor*>{&p, &m, &v, &decay})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->is_contiguous() && t->numel() == grad.numel(),
                "peer_fused_step: parameter, moment and decay buffers match the gradient");
  TORCH_CHECK(result.is_cuda() && result.scalar_type() == torch::kFloat32 && result.numel() >= 4 + 2 * kMaxWorld &&
              scratch.numel() * scratch.element_size() >= 16 && status.scalar_type() == torch::kInt32, "peer_fused_step: result / scratch / status");
  c10::cuda::CUDAGuard guard(grad.device());
  Peers peers{};
  for (int r = 0; r < world; ++r) {
    peers.grad[r] = reinterpret_cast<float*>(grad_ptrs[r]);
    peers.ctrl[r] = reinterpret_cast<unsigned char*>(ctrl_ptrs[r]);
  }
  StepArgs a{};
  a.p = reinterpret_cast<float4*>(p.data_ptr<float>());
  a.m = reinterpret_cast<float4*>(m.data_ptr<float>());
  a.v = reinterpret_cast<float4*>(v.data_ptr<float>());
  a.ema = (ema.has_value() && ema->defined()) ? reinterpret_cast<float4*>(ema->data_ptr<float>()) : nullptr;
  a.decay = reinterpret_cast<const float4*>(decay.data_ptr<float>());
  a.p16 = (p16.has_value() && p16->defined()) ? reinterpret_cast<uint2*>(p16->data_ptr()) : nullptr;
  a.lr = (float)lr; a.b1 = (float)b1; a.b2 = (float)b2; a.eps = (float)eps; a.bc1 = (float)bc1; a.bc2_sqrt = (float)std::sqrt(bc2);
  a.ema_w = (float)ema_w; a.clip_norm = (float)clip_norm; a.skip_threshold = (float)skip_threshold;
  a.per_rank_clip = per_rank_clip ? 1 : 0;
  a.n4 = grad.numel() / 4;
  const long long n4 = a.n4;
  const long long per = (n4 + world - 1) / world;
  long long begin4 = std::min<long long>(n4, per * rank), end4 = std::min<long long>(n4, per * (rank + 1));
  int device = grad.device().index(), sms = 148, occ = 1;
  C10_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  C10_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, peer_fused_step_kernel, 512, 0));
  TORCH_CHECK(occ >= 1, "peer_fused_step: kernel does not fit on an SM");
  const int blocks = sms * std::min(occ, 2);
  auto* acc = reinterpret_cast<double*>(scratch.data_ptr());
  auto* done = reinterpret_cast<unsigned int*>(reinterpret_cast<unsigned char*>(scratch.data_ptr()) + 8);
  float* res = result.data_ptr<float>();
  int* st = status.data_ptr<int>();
  int rank_i = (int)rank, world_i = (int)world;
  unsigned long long seq_u = (unsigned long long)seq;
  unsigned int spin = (unsigned int)(spin_limit > 0 ? spin_limit : kDefaultSpinLimit);
  void* args[] = {&peers, &a, &acc, &done, &res, &st, &begin4, &end4, &rank_i, &world_i, &seq_u, &spin};
  // cooperative: every block waits on words that other blocks of this grid publish, so all of them must be resident
  C10_CUDA_CHECK(cudaLaunchCooperativeKernel((void*)peer_fused_step_kernel, dim3(blocks), dim3(512), args, 0,
                                             at::cuda::getCurrentCUDAStream()));
}

// ---- peer-memory bootstrap without any library: plain device allocations shared through CUDA IPC handles ------------
// The handles (64 bytes each) travel between the ranks over the process group; opening one maps the peer's buffer
// into this process and enables peer access over NVLink.
Tensor df3_peer_alloc(int64_t nbytes, int64_t device) {
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  void* ptr = nullptr;
  C10_CUDA_CHECK(cudaMalloc(&ptr, (size_t)nbytes));
  C10_CUDA_CHECK(cudaMemset(ptr, 0, (size_t)nbytes));
  auto deleter = [](void* q) { cudaFree(q); };
  return torch::from_blob(ptr, {nbytes}, deleter, torch::dtype(torch::kUInt8).device(torch::kCUDA, (c10::DeviceIndex)device));
}

Tensor df3_peer_ipc_handle(const Tensor& buf) {
  TORCH_CHECK(buf.is_cuda(), "peer_ipc_handle: CUDA buffer from peer_alloc");
  cudaIpcMemHandle_t h;
  C10_CUDA_CHECK(cudaIpcGetMemHandle(&h, buf.data_ptr()));
  Tensor out = torch::empty({(int64_t)sizeof(h)}, torch::dtype(torch::kUInt8));
  std::memcpy(out.data_ptr(), &h, sizeof(h));
  return out;
}

int64_t df3_peer_ipc_open(const Tensor& handle, int64_t device) {
  TORCH_CHECK(!handle.is_cuda() && handle.numel() == (int64_t)sizeof(cudaIpcMemHandle_t), "peer_ipc_open: 64-byte host handle");
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data_ptr(), sizeof(h));
  void* ptr = nullptr;
  C10_CUDA_CHECK(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return (int64_t)(uintptr_t)ptr;  // stays mapped for the life of the process
}

}  // namespace
}  // namespace df3

void df3_register_peer(torch::Library& m) {
  m.def("peer_fused_step(Tensor(a!) grad, int[] grad_ptrs, int[] ctrl_ptrs, Tensor(b!) scratch, Tensor(c!) status, Tensor(d!) result, "
        "Tensor(e!) p, Tensor(f!) m, Tensor(g!) v, Tensor(h!)? ema, Tensor decay, Tensor(i!)? p16, int rank, int world, int seq, "
        "float lr, float b1, float b2, float eps, float bc1, float bc2, float ema_w, float clip_norm, float skip_threshold, "
        "bool per_rank_clip, int spin_limit=0) -> ()", &df3::df3_peer_fused_step);
  m.def("peer_alloc(int nbytes, int device) -> Tensor", &df3::df3_peer_alloc);
  m.def("peer_ipc_handle(Tensor buf) -> Tensor", &df3::df3_peer_ipc_handle);
  m.def("peer_ipc_open(Tensor handle, int device) -> int", &df3::df3_peer_ipc_open);
  m.def("peer_allreduce_mean(Tensor(a!) grad, int[] grad_ptrs, int[] ctrl_ptrs, Tensor(b!) scratch, Tensor(c!) status, int rank, "
        "int world, int seq, int spin_limit=0) -> Tensor", &df3::df3_peer_allreduce_mean);
}
