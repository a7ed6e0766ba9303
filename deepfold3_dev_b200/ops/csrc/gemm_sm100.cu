// bf16 GEMM for sm_100a on the 5th-generation tensor cores, with the epilogues the model needs fused in.
//
//   C[b, m, n] = epilogue( sum_k A[b, m, k] * W[b or 0, n, k] )
//
// One CTA computes a 128 x BN tile. Warp 0 is the TMA producer (cp.async.bulk.tensor into 128-byte
// swizzled shared memory, no cluster multicast), warp 1 allocates tensor memory and issues
// tcgen05.mma from one elected thread, warps 2-5 read the fp32 accumulator back with tcgen05.ld and
// run the epilogue. Stages are handed over with mbarriers; every wait is bounded and reports through
// a status word (df3::Status) instead of hanging.
//
// Epilogues:
//   kPlain       out = (acc + bias[n]) * row_mask[m]
//   kGated       out = sigmoid(acc_gate) * acc_proj * row_mask[m]   (gate and proj rows stacked in W)
//   kSwiGLU      out = silu(acc_gate) * acc_proj
//   kSigmoidMul  out = sigmoid(acc + bias[n]) * mul[m, n]
//   kSwiGLUBwd   out[m, n] = g b s (1 + a (1 - s)),  out[m, N + n] = g a s      with a = acc_gate, b = acc_proj,
//                s = sigmoid(a), g = mul[m, n]: the gradient of the pre-activation, which is recomputed here
//   kGatedBwd    out[m, n] = g r b s (1 - s),        out[m, N + n] = g r s       with r = row_mask[m]
// Output is bf16, row-major [b, m, n] or channel-major [b, n, m] (one plane per output channel, the
// layout the triangle contraction consumes).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <mutex>
#include <unordered_map>

#include "sm100_ptx.cuh"

using torch::Tensor;

namespace df3 {

// The driver entry point is looked up at run time so that the library loads on machines without a driver.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    C10_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q));
    TORCH_CHECK(sym != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is not available");
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// bf16 tensor map of any rank up to 5 with 128-byte swizzle; dims/strides innermost first, strides in elements.
CUtensorMap make_map_nd(const void* base, int rank, const int64_t* dims, const int64_t* strides_elems, const int* box) {
  CUtensorMap m;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = (cuuint64_t)dims[i];
    gbox[i] = (cuuint32_t)box[i];
    estr[i] = 1;
    if (i > 0) gstrides[i - 1] = (cuuint64_t)strides_elems[i] * 2;
  }
  const CUresult r = encode_tiled()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdims,
                                    gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    std::string msg = "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r) + ": dims";
    for (int i = 0; i < rank; ++i) msg += " " + std::to_string(dims[i]) + "(stride " + std::to_string(strides_elems[i]) + ")";
    TORCH_CHECK(false, msg);
  }
  return m;
}

// One int per device that kernels report bounded-wait failures through.
Tensor status_word(int device) {
  static std::mutex mutex;
  static std::unordered_map<int, Tensor> words;
  std::lock_guard<std::mutex> lock(mutex);
  auto it = words.find(device);
  if (it != words.end()) return it->second;
  Tensor t = torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
  words.emplace(device, t);
  return t;
}

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kThreads = 192;

enum Epi : int { kPlain = 0, kGated = 1, kSwiGLU = 2, kSigmoidMul = 3, kSwiGLUBwd = 4, kGatedBwd = 5 };

struct GemmParams {
  __nv_bfloat16* C;
  const float* bias;          // [n] or null
  const float* row_mask;      // [batch * M] or null
  const __nv_bfloat16* mul;   // [batch, M, N] (row stride ld_mul) or null
  int* status;
  long long c_batch_stride;   // elements
  long long mul_batch_stride;
  int ldc;                    // row stride (row-major) or plane stride (channel-major), elements
  int ld_mul;
  int M, N, K;                // N = output channels (half the accumulator width for the gated epilogues)
  int m_tiles, n_tiles;
  int stages;
  int b_batched;              // W has a batch axis
  int proj_row_offset;        // first row of the proj half inside the stacked weight
  int channel_major;
};

template <int BN>
struct Smem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
};

__device__ __forceinline__ bool wait_quiet(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 20); ++i)
    if (ptx::mbar_try_wait(bar, parity)) return true;
  return false;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 32 consecutive outputs of one row, already final values.
__device__ __forceinline__ void store_row32(const GemmParams& p, long long batch, int row, int n0, const float* v) {
  if (row >= p.M) return;
  if (p.channel_major) {
    __nv_bfloat16* base = p.C + batch * p.c_batch_stride + (long long)n0 * p.ldc + row;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n0 + j < p.N) base[(long long)j * p.ldc] = __float2bfloat16_rn(v[j]);
    return;
  }
  __nv_bfloat16* dst = p.C + batch * p.c_batch_stride + (long long)row * p.ldc + n0;
  if (n0 + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint4 q;
      q.x = pack_bf16(v[g * 8 + 0], v[g * 8 + 1]);
      q.y = pack_bf16(v[g * 8 + 2], v[g * 8 + 3]);
      q.z = pack_bf16(v[g * 8 + 4], v[g * 8 + 5]);
      q.w = pack_bf16(v[g * 8 + 6], v[g * 8 + 7]);
      reinterpret_cast<uint4*>(dst)[g] = q;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n0 + j < p.N) dst[j] = __float2bfloat16_rn(v[j]);
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads) gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                                                       const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  using S = Smem<BN>;
  constexpr bool kDual = (EPI == kGated || EPI == kSwiGLU || EPI == kSwiGLUBwd || EPI == kGatedBwd);
  constexpr bool kBwd = (EPI == kSwiGLUBwd || EPI == kGatedBwd);
  constexpr int kOutPerTile = kDual ? BN / 2 : BN;  // output columns one CTA produces
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + (size_t)p.stages * S::kStageBytes);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_ready = empty + p.stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x % p.n_tiles;
  const int m_tile = (blockIdx.x / p.n_tiles) % p.m_tiles;
  const int batch = blockIdx.x / (p.n_tiles * p.m_tiles);
  const int num_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
    }
    ptx::mbar_init(acc_ready, 1);
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, BN);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (ptx::elect_one()) {
      ptx::prefetch_tensormap(&tmA);
      ptx::prefetch_tensormap(&tmB);
      int issued = 0;
      bool ok = true;
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % p.stages;
        const uint32_t ph = (uint32_t)(kb / p.stages) & 1u;
        if (!ptx::mbar_wait(&empty[s], ph ^ 1u, p.status, kTimeoutStageEmpty)) { ok = false; break; }
        uint8_t* a_s = tiles + (size_t)s * S::kStageBytes;
        uint8_t* b_s = a_s + S::kABytes;
        ptx::mbar_expect_tx(&full[s], S::kStageBytes);
        ptx::tma_load_3d(a_s, &tmA, &full[s], kb * BK, m_tile * BM, batch);
        const int bz = p.b_batched ? batch : 0;
        if (kDual) {
          ptx::tma_load_3d(b_s, &tmB, &full[s], kb * BK, n_tile * (BN / 2), bz);
          ptx::tma_load_3d(b_s + S::kBBytes / 2, &tmB, &full[s], kb * BK, p.proj_row_offset + n_tile * (BN / 2), bz);
        } else {
          ptx::tma_load_3d(b_s, &tmB, &full[s], kb * BK, n_tile * BN, bz);
        }
        issued = kb + 1;
      }
      if (!ok) {  // give up: let the copies already in flight land before the CTA's shared memory goes away
        const int first = issued > p.stages ? issued - p.stages : 0;
        for (int kb = first; kb < issued; ++kb) wait_quiet(&full[kb % p.stages], (uint32_t)(kb / p.stages) & 1u);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = ptx::idesc_bf16_f32(BM, BN);
      bool ok = true;
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % p.stages;
        const uint32_t ph = (uint32_t)(kb / p.stages) & 1u;
        if (!ptx::mbar_wait(&full[s], ph, p.status, kTimeoutTmaFull)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t a_addr = ptx::smem_u32(tiles + (size_t)s * S::kStageBytes);
        const uint64_t a_desc = ptx::smem_desc_k_sw128(a_addr);
        const uint64_t b_desc = ptx::smem_desc_k_sw128(a_addr + S::kABytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)  // 16 bf16 = 32 bytes per MMA along K: descriptor address advances by 2
          ptx::umma_bf16(tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, (kb | k) != 0);
        ptx::umma_commit(&empty[s]);
      }
      if (ok) ptx::umma_commit(acc_ready);
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    if (ptx::mbar_wait(acc_ready, 0, p.status, kTimeoutMmaDone)) {
      ptx::tc_fence_after();
      const int row = m_tile * BM + q * 32 + lane;
      const uint32_t t_row = tmem + ((uint32_t)(q * 32) << 16);
      const float rm = (p.row_mask != nullptr && row < p.M) ? p.row_mask[(long long)batch * p.M + row] : 1.f;
      float a[32], b[32];
#pragma unroll 1
      for (int c = 0; c < kOutPerTile / 32; ++c) {
        const int n0 = n_tile * kOutPerTile + c * 32;
        if (n0 >= p.N) break;
        ptx::tmem_ld_32x32(t_row + c * 32, a);
        if (kDual) ptx::tmem_ld_32x32(t_row + BN / 2 + c * 32, b);
        ptx::tmem_ld_wait();
        if (EPI == kPlain) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float bv = (p.bias != nullptr && n0 + j < p.N) ? p.bias[n0 + j] : 0.f;
            a[j] = (a[j] + bv) * rm;
          }
        } else if (EPI == kGated) {
#pragma unroll
          for (int j = 0; j < 32; ++j) a[j] = sigmoidf_(a[j]) * b[j] * rm;
        } else if (EPI == kSwiGLU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) a[j] = a[j] * sigmoidf_(a[j]) * b[j];
        } else if (kBwd) {
          const __nv_bfloat16* grow = p.mul + batch * p.mul_batch_stride + (long long)row * p.ld_mul + n0;
          float g[32];
          if (row < p.M && n0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(grow) & 15) == 0) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              const uint4 w = reinterpret_cast<const uint4*>(grow)[q4];
              const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(&ww[e]);
                g[q4 * 8 + 2 * e] = __low2float(pr);
                g[q4 * 8 + 2 * e + 1] = __high2float(pr);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) g[j] = (row < p.M && n0 + j < p.N) ? __bfloat162float(grow[j]) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float sg = sigmoidf_(a[j]);
            const float gj = g[j] * rm;
            const float da = EPI == kSwiGLUBwd ? gj * b[j] * sg * (1.f + a[j] * (1.f - sg)) : gj * b[j] * sg * (1.f - sg);
            const float dbv = EPI == kSwiGLUBwd ? gj * a[j] * sg : gj * sg;
            a[j] = da;
            b[j] = dbv;
          }
          store_row32(p, batch, row, n0, a);
          GemmParams p2 = p;
          p2.C = p.C + p.N;  // second half of the [M, 2 N] output; bounds are those of the first half
          store_row32(p2, batch, row, n0, b);
          continue;
        } else {
          const __nv_bfloat16* mrow = p.mul + batch * p.mul_batch_stride + (long long)row * p.ld_mul + n0;
          if (row < p.M && n0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(mrow) & 15) == 0) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint4 w = reinterpret_cast<const uint4*>(mrow)[g];
              const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(&ww[e]);
                const int j = g * 8 + 2 * e;
                const float b0 = p.bias ? p.bias[n0 + j] : 0.f, b1 = p.bias ? p.bias[n0 + j + 1] : 0.f;
                a[j] = sigmoidf_(a[j] + b0) * __low2float(pr);
                a[j + 1] = sigmoidf_(a[j + 1] + b1) * __high2float(pr);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const bool in = row < p.M && n0 + j < p.N;
              const float bv = (p.bias != nullptr && in) ? p.bias[n0 + j] : 0.f;
              const float mv = in ? __bfloat162float(mrow[j]) : 0.f;
              a[j] = sigmoidf_(a[j] + bv) * mv;
            }
          }
        }
        store_row32(p, batch, row, n0, a);
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, BN);
  }
}

// ---- host ---------------------------------------------------------------------------------------
CUtensorMap make_map(const void* base, int64_t inner, int64_t rows, int64_t batch, int64_t row_stride,
                     int64_t batch_stride, int box_rows) {
  const int64_t dims[3] = {inner, rows, batch};
  const int64_t strides[3] = {1, row_stride, batch_stride};
  const int box[3] = {BK, box_rows, 1};
  return make_map_nd(base, 3, dims, strides, box);
}

template <int BN, int EPI>
void launch(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int64_t batch, cudaStream_t stream) {
  using S = Smem<BN>;
  const int num_k = (p.K + BK - 1) / BK;
  // enough stages to cover a short K loop without spending shared memory that a second resident CTA could use
  const int stages = num_k < 2 ? 2 : (num_k > 4 ? 4 : num_k);
  p.stages = stages;
  const size_t smem = (size_t)stages * S::kStageBytes + 1024 + 256;
  static bool attr_set = false;
  if (!attr_set) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set = true;
  }
  const long long ctas = (long long)p.m_tiles * p.n_tiles * batch;
  TORCH_CHECK(ctas > 0 && ctas < (1ll << 31), "gemm: grid too large");
  gemm_kernel<BN, EPI><<<(unsigned)ctas, kThreads, smem, stream>>>(ta, tb, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// a: [batch, M, K] view (last dim contiguous); w: [wb, Nw, K]; returns [batch, M, N] or [batch, N, M].
Tensor gemm_impl(const Tensor& a3, const Tensor& w3, const c10::optional<Tensor>& bias,
                 const c10::optional<Tensor>& row_mask, const c10::optional<Tensor>& mul, int epi, bool channel_major) {
  TORCH_CHECK(a3.is_cuda() && a3.scalar_type() == torch::kBFloat16 && w3.scalar_type() == torch::kBFloat16,
              "gemm: bf16 CUDA tensors expected");
  TORCH_CHECK(a3.dim() == 3 && w3.dim() == 3 && a3.stride(2) == 1 && w3.stride(2) == 1, "gemm: [b, rows, k] operands");
  const int64_t batch = a3.size(0), M = a3.size(1), K = a3.size(2);
  const int64_t wb = w3.size(0), Nw = w3.size(1);
  TORCH_CHECK(w3.size(2) == K && (wb == 1 || wb == batch), "gemm: operand shapes disagree");
  TORCH_CHECK(K % 8 == 0 && a3.stride(1) % 8 == 0 && w3.stride(1) % 8 == 0, "gemm: K and row strides must be multiples of 8");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(a3.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(w3.data_ptr()) % 16 == 0,
              "gemm: operands must be 16-byte aligned");
  TORCH_CHECK(batch == 1 || a3.stride(0) % 8 == 0, "gemm: batch stride must be a multiple of 8");
  const bool dual = (epi == kGated || epi == kSwiGLU || epi == kSwiGLUBwd || epi == kGatedBwd);
  const bool bwd = (epi == kSwiGLUBwd || epi == kGatedBwd);
  TORCH_CHECK(!bwd || !channel_major, "gemm: the backward epilogues store row-major");
  TORCH_CHECK(!dual || Nw % 2 == 0, "gemm: stacked gate/proj weight expected");
  const int64_t N = dual ? Nw / 2 : Nw;
  TORCH_CHECK(M < (1ll << 31) && N < (1 << 24) && K < (1 << 24), "gemm: size out of range");
  c10::cuda::CUDAGuard guard(a3.device());
  auto opts = a3.options();
  Tensor out = channel_major ? torch::empty({batch, N, M}, opts) : torch::empty({batch, M, bwd ? 2 * N : N}, opts);
  if (out.numel() == 0) return out;

  // accumulator width: the widest tile that the output needs
  int BN;
  if (dual) BN = N >= 128 ? 256 : (N >= 64 ? 128 : 64);
  else BN = N > 64 ? 128 : (N > 32 ? 64 : 32);
  const int out_per_tile = dual ? BN / 2 : BN;

  GemmParams p{};
  p.C = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  Tensor bias_f, mask_f, mul_c;
  if (bias.has_value() && bias->defined()) {
    bias_f = bias->to(torch::kFloat32).contiguous();
    TORCH_CHECK(bias_f.numel() == N, "gemm: bias length");
    p.bias = bias_f.data_ptr<float>();
  }
  if (row_mask.has_value() && row_mask->defined()) {
    mask_f = row_mask->to(torch::kFloat32).contiguous();
    TORCH_CHECK(mask_f.numel() == batch * M, "gemm: row mask length");
    p.row_mask = mask_f.data_ptr<float>();
  }
  if (epi == kSigmoidMul || bwd) {
    TORCH_CHECK(mul.has_value() && mul->defined(), "gemm: sigmoid-mul epilogue needs the multiplicand");
    mul_c = mul->contiguous();
    TORCH_CHECK(mul_c.scalar_type() == torch::kBFloat16 && mul_c.numel() == batch * M * N, "gemm: multiplicand shape");
    p.mul = reinterpret_cast<const __nv_bfloat16*>(mul_c.data_ptr());
    p.ld_mul = (int)N;
    p.mul_batch_stride = M * N;
  }
  Tensor status = status_word(a3.device().index());
  p.status = status.data_ptr<int>();
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.m_tiles = (int)((M + BM - 1) / BM);
  p.n_tiles = (int)((N + out_per_tile - 1) / out_per_tile);
  p.b_batched = wb > 1;
  p.proj_row_offset = (int)N;
  p.channel_major = channel_major;
  p.ldc = channel_major ? (int)M : (int)(bwd ? 2 * N : N);
  p.c_batch_stride = M * (bwd ? 2 * N : N);

  const int box_b = dual ? BN / 2 : BN;
  const CUtensorMap ta = make_map(a3.data_ptr(), K, M, batch, a3.stride(1), batch > 1 ? a3.stride(0) : M * a3.stride(1), BM);
  const CUtensorMap tb = make_map(w3.data_ptr(), K, Nw, wb, w3.stride(1), wb > 1 ? w3.stride(0) : Nw * w3.stride(1), box_b);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
#define DF3_LAUNCH(BN_, EPI_) launch<BN_, EPI_>(ta, tb, p, batch, stream)
  switch (epi) {
    case kPlain:
      if (BN == 128) DF3_LAUNCH(128, kPlain); else if (BN == 64) DF3_LAUNCH(64, kPlain); else DF3_LAUNCH(32, kPlain);
      break;
    case kSigmoidMul:
      if (BN == 128) DF3_LAUNCH(128, kSigmoidMul); else if (BN == 64) DF3_LAUNCH(64, kSigmoidMul); else DF3_LAUNCH(32, kSigmoidMul);
      break;
    case kGated:
      if (BN == 256) DF3_LAUNCH(256, kGated); else if (BN == 128) DF3_LAUNCH(128, kGated); else DF3_LAUNCH(64, kGated);
      break;
    case kSwiGLU:
      if (BN == 256) DF3_LAUNCH(256, kSwiGLU); else if (BN == 128) DF3_LAUNCH(128, kSwiGLU); else DF3_LAUNCH(64, kSwiGLU);
      break;
    case kSwiGLUBwd:
      if (BN == 256) DF3_LAUNCH(256, kSwiGLUBwd); else if (BN == 128) DF3_LAUNCH(128, kSwiGLUBwd); else DF3_LAUNCH(64, kSwiGLUBwd);
      break;
    case kGatedBwd:
      if (BN == 256) DF3_LAUNCH(256, kGatedBwd); else if (BN == 128) DF3_LAUNCH(128, kGatedBwd); else DF3_LAUNCH(64, kGatedBwd);
      break;
    default:
      TORCH_CHECK(false, "gemm: unknown epilogue ", epi);
  }
#undef DF3_LAUNCH
  return out;
}

// x: [..., K] with any leading shape; weight [N(or 2N), K]. Leading axes are flattened into rows.
Tensor df3_gemm(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, const c10::optional<Tensor>& row_mask,
                const c10::optional<Tensor>& mul, int64_t epi, bool channel_major) {
  TORCH_CHECK(x.dim() >= 2 && w.dim() == 2, "gemm: x [..., K], w [N, K]");
  Tensor xc = x.contiguous();
  const int64_t K = xc.size(-1);
  Tensor a3 = xc.view({1, -1, K});
  Tensor w3 = w.contiguous().view({1, w.size(0), K});
  Tensor out = gemm_impl(a3, w3, bias, row_mask, mul, (int)epi, channel_major);
  if (channel_major) return out.view({out.size(1), out.size(2)});
  auto shape = xc.sizes().vec();
  shape.back() = out.size(2);
  return out.view(shape);
}

// a: [B, M, K], b: [B, N, K] -> [B, M, N]: sum over the shared last axis (both K-major).
Tensor df3_bmm_nt(const Tensor& a, const Tensor& b) {
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3 && a.size(0) == b.size(0), "bmm_nt: [B, M, K] x [B, N, K]");
  Tensor ac = a.stride(2) == 1 ? a : a.contiguous();
  Tensor bc = b.stride(2) == 1 ? b : b.contiguous();
  return gemm_impl(ac, bc, c10::nullopt, c10::nullopt, c10::nullopt, kPlain, false);
}

// Backward of y = x w^T (+ b) with bf16 operands: dx = dy w (in x's dtype), dw = dy^T x and db = sum dy in fp32.
// One call from Python instead of six small ones; the products run on the library GEMM.
std::tuple<Tensor, Tensor, Tensor> df3_linear_bwd(const Tensor& dy, const Tensor& x, const Tensor& w16, bool need_dx, bool need_dw,
                                                   bool need_db) {
  const int64_t n = w16.size(0), k = w16.size(1);
  Tensor d2 = dy.reshape({-1, n});
  if (d2.scalar_type() != torch::kBFloat16) d2 = d2.to(torch::kBFloat16);
  Tensor dx, dw, db;
  if (need_dx) {
    dx = at::mm(d2, w16).view(x.sizes());
    if (dx.scalar_type() != x.scalar_type()) dx = dx.to(x.scalar_type());
  }
  if (need_dw) {
    Tensor x2 = x.reshape({-1, k});
    if (x2.scalar_type() != torch::kBFloat16) x2 = x2.to(torch::kBFloat16);
    dw = at::mm(d2.t(), x2).to(torch::kFloat32);
  }
  if (need_db) db = d2.sum(0, false, torch::kFloat32);
  auto undef = [&](Tensor& t) { if (!t.defined()) t = torch::empty({0}, dy.options()); };
  undef(dx); undef(dw); undef(db);
  return {dx, dw, db};
}

// Reads the status word of the current device (synchronises) and clears it.
int64_t df3_gemm_status() {
  int device = 0;
  C10_CUDA_CHECK(cudaGetDevice(&device));
  Tensor s = status_word(device);
  const int64_t v = s.item<int>();
  if (v != 0) s.zero_();
  return v;
}

}  // namespace
}  // namespace df3

void df3_register_gemm(torch::Library& m) {
  m.def("gemm(Tensor x, Tensor w, Tensor? bias, Tensor? row_mask, Tensor? mul, int epi, bool channel_major) -> Tensor",
        &df3::df3_gemm);
  m.def("bmm_nt(Tensor a, Tensor b) -> Tensor", &df3::df3_bmm_nt);
  m.def("gemm_status() -> int", &df3::df3_gemm_status);
  m.def("linear_bwd(Tensor dy, Tensor x, Tensor w16, bool need_dx, bool need_dw, bool need_db) -> (Tensor, Tensor, Tensor)",
        &df3::df3_linear_bwd);
}

const char* df3_gemm_features() { return "gemm,gated_dual_linear,transition,pair_bias_attention,linear_planes,sigmoid_gate_mul,peer_reduce"; }
