// Re-layout of a sharded tensor across the GPUs of one node through NVLink peer memory: all-to-all (rows <-> channels,
// shard transpose) and all-gather, as one strided "push" pattern.
//
// Every rank owns a receive heap and a control block that all ranks have mapped. One exchange is three launches on the
// caller's stream:
//   1. entry   one warp: stores this exchange's sequence number into every peer's control block and waits, bounded,
//              for the same word from every peer. Once it returns, every peer has finished (in stream order) whatever
//              read its own heap before, so the heaps may be overwritten.
//   2. push    every rank stores its contribution straight into its final place in each peer's heap, 16 bytes per
//              thread, four stores in flight; the order of destinations is rotated by rank so that no two ranks
//              target the same GPU at the same moment. The last block fences and publishes the done flag to all peers.
//   3. collect every block waits, bounded, for all done flags and copies its part of the heap into the result tensor,
//              which leaves the heap free for the next exchange.
// The pattern is described by three loop levels with source and destination strides plus a contiguous inner run; the
// source offset advances by `src_q` per destination rank, the destination offset is fixed by the sending rank.
//
// Plain stores and loads only (no multimem, no TMA), and no wait is unbounded: a wait that runs out records
// kTimeoutPeerFlag in the status word, the later launches of the exchange see it and touch no peer memory.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "common.cuh"

using torch::Tensor;

namespace df3 {
namespace {

constexpr int kMaxWorld = 16;
constexpr int64_t kDefaultSpinLimit = 20 * 1000 * 1000;
constexpr int kDoneOff = 256;    // unsigned long long[kMaxWorld]: done sequence numbers, slot s written by rank s
constexpr int kArriveOff = 384;  // unsigned long long[kMaxWorld]: entry sequence numbers, slot s written by rank s

struct XPeers {
  uint4* heap[kMaxWorld];
  unsigned char* ctrl[kMaxWorld];
};

// all extents and strides in 16-byte vectors
struct XPlan {
  uint32_t n0, n1, n2, inner;
  long long ss0, ss1, ss2, ds0, ds1, ds2, src_q, dst_base;
  long long src_vecs, dst_vecs;   // extents of the source tensor and of one rank's result (read by the debug build's checks)
};

__global__ void exchange_entry_kernel(XPeers peers, int* __restrict__ status, int rank, int world, unsigned long long seq,
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

__device__ __forceinline__ void locate(const XPlan& pl, uint32_t per_q, uint32_t idx, int rank, int world, int& q, long long& s,
                                       long long& d) {
  const uint32_t k = idx / per_q;
  uint32_t rem = idx - k * per_q;
  q = rank + (int)k;
  if (q >= world) q -= world;
  const uint32_t v = rem % pl.inner;
  rem /= pl.inner;
  const uint32_t i2 = rem % pl.n2;
  rem /= pl.n2;
  const uint32_t i1 = rem % pl.n1;
  const uint32_t i0 = rem / pl.n1;
  s = (long long)q * pl.src_q + i0 * pl.ss0 + i1 * pl.ss1 + i2 * pl.ss2 + v;
  d = pl.dst_base + i0 * pl.ds0 + i1 * pl.ds1 + i2 * pl.ds2 + v;
}

__global__ void __launch_bounds__(512) exchange_push_kernel(const uint4* __restrict__ src, XPeers peers, XPlan pl,
                                                          int* __restrict__ status, unsigned int* __restrict__ done,
                                                          uint32_t per_q, int rank, int world, unsigned long long seq) {
  if (*reinterpret_cast<const volatile int*>(status) != kOk) return;
  const unsigned long long total = (unsigned long long)per_q * world;
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  constexpr int kUnroll = 4;
  for (unsigned long long base = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; base < total; base += stride * kUnroll) {
    uint4 v[kUnroll];
    int q[kUnroll];
    long long d[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const unsigned long long idx = base + u * stride;
      q[u] = -1;
      if (idx < total) {
        long long s;
        locate(pl, per_q, (uint32_t)idx, rank, world, q[u], s, d[u]);
        if (in_bounds(s, pl.src_vecs, status) && in_bounds(d[u], pl.dst_vecs, status)) v[u] = src[s];
        else q[u] = -1;
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      if (q[u] >= 0) peers.heap[q[u]][d[u]] = v[u];
  }
  __threadfence_system();  // this block's peer stores are visible before it counts itself done
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int before = atomicAdd(done, 1u);
    if (before == gridDim.x - 1) {
      __threadfence_system();
      for (int r = 0; r < world; ++r) reinterpret_cast<volatile unsigned long long*>(peers.ctrl[r] + kDoneOff)[rank] = seq;
      *done = 0u;
    }
  }
}

__global__ void __launch_bounds__(512) exchange_collect_kernel(const uint4* __restrict__ heap, uint4* __restrict__ out,
                                                             unsigned long long total, const unsigned char* __restrict__ ctrl,
                                                             int* __restrict__ status, int world, unsigned long long seq,
                                                             unsigned int spin_limit) {
  bool ok = *reinterpret_cast<const volatile int*>(status) == kOk;
  if (ok && (int)threadIdx.x < world) {
    const volatile unsigned long long* flag = reinterpret_cast<const volatile unsigned long long*>(ctrl + kDoneOff) + threadIdx.x;
    uint32_t spins = 0;
    while (*flag < seq) {
      if (++spins > spin_limit) { ok = false; break; }
      __nanosleep(64);
    }
  }
  if (!__syncthreads_and(ok ? 1 : 0)) {
    if (threadIdx.x == 0) atomicCAS(status, kOk, kTimeoutPeerFlag);
    return;
  }
  __threadfence_system();
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
    out[i] = __ldcv(heap + i);  // written by other GPUs: bypass whatever this SM may have cached from an earlier exchange
}

}  // namespace

// src: this rank's contiguous contribution; out: the result tensor (contiguous); heap_ptrs / ctrl_ptrs: the receive heap
// and control block of every rank as mapped here. counts / sstr / dstr / inner / src_q / dst_base are in elements of src.
void df3_peer_exchange(const Tensor& src, Tensor out, const std::vector<int64_t>& heap_ptrs, const std::vector<int64_t>& ctrl_ptrs,
                       int64_t heap_bytes, Tensor scratch, Tensor status, int64_t rank, int64_t world, int64_t seq,
                       const std::vector<int64_t>& counts, const std::vector<int64_t>& sstr, const std::vector<int64_t>& dstr,
                       int64_t inner, int64_t src_q, int64_t dst_base, int64_t spin_limit) {
  TORCH_CHECK(src.is_cuda() && out.is_cuda() && src.is_contiguous() && out.is_contiguous() && src.scalar_type() == out.scalar_type(),
              "peer_exchange: contiguous CUDA tensors of one dtype");
  TORCH_CHECK(world >= 2 && world <= kMaxWorld && (int64_t)heap_ptrs.size() == world && (int64_t)ctrl_ptrs.size() == world && rank >= 0 &&
              rank < world, "peer_exchange: world size / pointer lists");
  TORCH_CHECK(counts.size() == 3 && sstr.size() == 3 && dstr.size() == 3, "peer_exchange: three loop levels");
  TORCH_CHECK(scratch.is_cuda() && scratch.numel() * scratch.element_size() >= 4 && status.scalar_type() == torch::kInt32,
              "peer_exchange: 4 scratch bytes and an int32 status word");
  const int64_t es = src.element_size();
  TORCH_CHECK(16 % es == 0, "peer_exchange: element size must divide 16");
  const int64_t per16 = 16 / es;
  auto vec = [&](int64_t elems, const char* what) {
    TORCH_CHECK(elems % per16 == 0, "peer_exchange: ", what, " (", elems, " elements) is not a multiple of 16 bytes");
    return elems / per16;
  };
  XPlan pl{};
  pl.n0 = (uint32_t)counts[0]; pl.n1 = (uint32_t)counts[1]; pl.n2 = (uint32_t)counts[2];
  pl.inner = (uint32_t)vec(inner, "inner run");
  pl.ss0 = vec(sstr[0], "source stride"); pl.ss1 = vec(sstr[1], "source stride"); pl.ss2 = vec(sstr[2], "source stride");
  pl.ds0 = vec(dstr[0], "destination stride"); pl.ds1 = vec(dstr[1], "destination stride"); pl.ds2 = vec(dstr[2], "destination stride");
  pl.src_q = vec(src_q, "per-rank source offset");
  pl.dst_base = vec(dst_base, "destination offset");
  pl.src_vecs = src.numel() * es / 16;
  pl.dst_vecs = out.numel() * es / 16;
  TORCH_CHECK(counts[0] > 0 && counts[1] > 0 && counts[2] > 0 && pl.inner > 0, "peer_exchange: empty pattern");
  const int64_t per_q = counts[0] * counts[1] * counts[2] * (int64_t)pl.inner;
  TORCH_CHECK(per_q * world < (int64_t)1 << 32, "peer_exchange: more than 2^32 vectors in one exchange");
  TORCH_CHECK(per_q * world * 16 == out.numel() * es, "peer_exchange: the pattern does not cover the result exactly");
  TORCH_CHECK(out.numel() * es <= heap_bytes, "peer_exchange: result larger than the receive heap");
  TORCH_CHECK(per_q * world * 16 <= src.numel() * es * world, "peer_exchange: pattern reads beyond the source");
  TORCH_CHECK((uintptr_t)src.data_ptr() % 16 == 0 && (uintptr_t)out.data_ptr() % 16 == 0, "peer_exchange: 16-byte aligned tensors");
  // bounds of the addressed ranges (host arithmetic on the launch's own numbers)
  const int64_t last_s = (world - 1) * pl.src_q + (counts[0] - 1) * pl.ss0 + (counts[1] - 1) * pl.ss1 + (counts[2] - 1) * pl.ss2 + pl.inner;
  const int64_t last_d = pl.dst_base + (counts[0] - 1) * pl.ds0 + (counts[1] - 1) * pl.ds1 + (counts[2] - 1) * pl.ds2 + pl.inner;
  TORCH_CHECK(last_s * 16 <= src.numel() * es, "peer_exchange: source pattern out of range");
  TORCH_CHECK(last_d * 16 <= out.numel() * es, "peer_exchange: destination pattern out of range");
  c10::cuda::CUDAGuard guard(src.device());
  XPeers peers{};
  for (int r = 0; r < world; ++r) {
    peers.heap[r] = reinterpret_cast<uint4*>(heap_ptrs[r]);
    peers.ctrl[r] = reinterpret_cast<unsigned char*>(ctrl_ptrs[r]);
  }
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const unsigned int spin = (unsigned int)(spin_limit > 0 ? spin_limit : kDefaultSpinLimit);
  const unsigned long long total = (unsigned long long)per_q * world;
  const int blocks = (int)std::min<unsigned long long>(148 * 4, (total + 511) / 512);
  exchange_entry_kernel<<<1, 32, 0, stream>>>(peers, status.data_ptr<int>(), (int)rank, (int)world, (unsigned long long)seq, spin);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  exchange_push_kernel<<<blocks, 512, 0, stream>>>(reinterpret_cast<const uint4*>(src.data_ptr()), peers, pl, status.data_ptr<int>(),
                                                   reinterpret_cast<unsigned int*>(scratch.data_ptr()), (uint32_t)per_q, (int)rank,
                                                   (int)world, (unsigned long long)seq);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  exchange_collect_kernel<<<blocks, 512, 0, stream>>>(peers.heap[rank], reinterpret_cast<uint4*>(out.data_ptr()), total, peers.ctrl[rank],
                                                      status.data_ptr<int>(), (int)world, (unsigned long long)seq, spin);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace df3

void df3_register_peer_exchange(torch::Library& m) {
  m.def("peer_exchange(Tensor src, Tensor(a!) out, int[] heap_ptrs, int[] ctrl_ptrs, int heap_bytes, Tensor(b!) scratch, "
        "Tensor(c!) status, int rank, int world, int seq, int[] counts, int[] sstr, int[] dstr, int inner, int src_q, int dst_base, "
        "int spin_limit=0) -> ()", &df3::df3_peer_exchange);
}
