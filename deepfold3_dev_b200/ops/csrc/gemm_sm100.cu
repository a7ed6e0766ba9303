// bf16 GEMM for sm_100a on the 5th-generation tensor cores, with the epilogues the model needs fused in.
//
//   C[b, m, n] = epilogue( sum_k A[b, m, k] * W[b or 0, n, k] )
//
// One CTA computes a 128 x BN tile. Warp 0 is the TMA producer (cp.async.bulk.tensor into 128-byte
// swizzled shared memory, each copy for this CTA alone), warp 1 allocates tensor memory and issues
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

#include <algorithm>
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
  // cuTensorMapEncodeTiled is a driver call and wants a context bound to the calling thread. A thread whose first CUDA
  // work is this call (an autograd worker starting a backward pass with one of these kernels) has none yet: the runtime
  // binds the primary context lazily, on its own calls. cudaSetDevice binds it.
  thread_local bool bound = false;
  if (!bound) {
    int dev = 0;
    C10_CUDA_CHECK(cudaGetDevice(&dev));
    C10_CUDA_CHECK(cudaSetDevice(dev));
    bound = true;
  }
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
constexpr int kThreads = 320;      // TMA warp, MMA warp, eight epilogue warps (two per tensor-memory lane quarter)
constexpr int kEpiThreads = 256;
constexpr int kMaxResidentK = 4;   // k blocks of the weight tile a CTA may keep in shared memory for its whole life
constexpr int kGroupM = 8;  // tiles walk the output in bands of 8 tile rows so that concurrent CTAs share operands in L2

enum Epi : int { kPlain = 0, kGated = 1, kSwiGLU = 2, kSigmoidMul = 3, kSwiGLUBwd = 4, kGatedBwd = 5, kGatedT = 6 };

struct GemmParams {
  void* C;                    // bf16 or fp32
  const float* bias;          // per output column n (or per output row m when bias_on_m) or null
  const float* row_mask;      // per output row m (or per column n when mask_on_n), one entry per batch row, or null
  const __nv_bfloat16* mul;   // [batch, M, N] (row stride ld_mul) or null
  int* status;
  long long c_batch_stride;   // elements
  long long c_split_stride;   // elements between the partial results of a split-K launch
  long long mul_batch_stride;
  long long ldc;              // row stride (row-major) or plane stride (channel-major), elements
  int ld_mul;
  int M, N, K;                // N = output channels (half the accumulator width for the dual-B epilogues)
  int m_tiles, n_tiles, batch, splits;
  int kb_total, kb_per_split; // k blocks of 64
  int stages;
  int b_resident;             // the CTA's B tile (all of K) stays in shared memory; the ring then holds A only
  int b_batched, a_batched;   // operand has a batch axis
  int proj_row_offset;        // first row of the proj half inside the stacked weight
  int channel_major;          // legacy transposed store of the row-major tile (small shapes only)
  int a_mn, b_mn;             // operand is MN-major (its M / N index is the contiguous one)
  int c_fp32;
  int tma_store;              // bf16 row-major output with 16-byte aligned rows: tiles leave through shared memory and TMA
  int bias_on_m, mask_on_n;
  long long mask_batch_stride;
  long long c_elems;          // elements of the whole output (read by the debug build's bounds checks)
};

template <int BN, bool DUAL_A>
struct Smem {
  static constexpr int kABytes = (DUAL_A ? 2 : 1) * BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// 32 consecutive outputs of one row, already final values.
__device__ __forceinline__ void store_row32(const GemmParams& p, void* cbase, long long batch_off, int row, int n0, const float* v) {
  if (row >= p.M) return;
  if (p.c_fp32) {
    float* dst = reinterpret_cast<float*>(cbase) + batch_off + (long long)row * p.ldc + n0;
    if (n0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
      for (int g = 0; g < 8; ++g) reinterpret_cast<float4*>(dst)[g] = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (n0 + j < p.N) dst[j] = v[j];
    }
    return;
  }
  __nv_bfloat16* cb = reinterpret_cast<__nv_bfloat16*>(cbase) + batch_off;
  if (p.channel_major) {
    __nv_bfloat16* base = cb + (long long)n0 * p.ldc + row;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (n0 + j < p.N) base[(long long)j * p.ldc] = __float2bfloat16_rn(v[j]);
    return;
  }
  __nv_bfloat16* dst = cb + (long long)row * p.ldc + n0;
  if (p.c_elems > 0 && !in_bounds(batch_off + (long long)row * p.ldc + n0 + (n0 + 32 <= p.N ? 31 : p.N - n0 - 1), p.c_elems, p.status)) return;
  if (n0 + 32 <= p.N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
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

__device__ __forceinline__ void load_row32(const __nv_bfloat16* src, bool row_ok, int n0, int N, float* g) {
  if (row_ok && n0 + 32 <= N && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const uint4 w = reinterpret_cast<const uint4*>(src)[q4];
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
    for (int j = 0; j < 32; ++j) g[j] = (row_ok && n0 + j < N) ? __bfloat162float(src[j]) : 0.f;
  }
}

struct TileCoord {
  int split, batch, m_tile, n_tile;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, long long t) {
  TileCoord c;
  const long long per_batch = (long long)p.m_tiles * p.n_tiles;
  const long long bt = t / per_batch;
  const int r = (int)(t - bt * per_batch);
  c.batch = (int)(bt % p.batch);
  c.split = (int)(bt / p.batch);
  const int band = kGroupM * p.n_tiles;
  const int g = r / band, q = r - g * band;
  const int gm = min(kGroupM, p.m_tiles - g * kGroupM);
  c.m_tile = g * kGroupM + q % gm;
  c.n_tile = q / gm;
  return c;
}

// Tile i of this CTA. Streaming mode: tiles blockIdx.x, blockIdx.x + gridDim.x, ... in banded order. Resident-B mode
// (tall products against a small weight): the CTA keeps one n tile for its whole life and walks down the rows, so the
// weight tile is fetched once per CTA instead of once per output tile.
__device__ __forceinline__ bool tile_at(const GemmParams& p, long long i, TileCoord& c) {
  if (p.b_resident) {
    const int G = gridDim.x / p.n_tiles;
    const long long u = blockIdx.x / p.n_tiles + i * G;
    if (u >= (long long)p.m_tiles * p.batch) return false;
    c.split = 0;
    c.n_tile = blockIdx.x % p.n_tiles;
    c.m_tile = (int)(u % p.m_tiles);
    c.batch = (int)(u / p.m_tiles);
    return true;
  }
  const long long t = blockIdx.x + i * gridDim.x;
  if (t >= (long long)p.m_tiles * p.n_tiles * p.batch * p.splits) return false;
  c = decode_tile(p, t);
  return true;
}

// Persistent kernel: each CTA walks tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... The accumulator is double
// buffered in tensor memory, so the epilogue warps drain tile t while the MMA warp already works on tile t + 1, and
// the shared-memory ring keeps running across tile boundaries.
// The plain and sigmoid-gate epilogues at tile widths up to 128 are compiled for two CTAs per SM (at most 102
// registers per thread): on the pair-shaped products (K = 128, a few thousand row tiles) the epilogue is the critical
// path, and with ten warps per SM its tensor-memory and shared-memory latencies are exposed; a second CTA fills them.
template <int BN, int EPI>
constexpr int min_ctas_per_sm() { return ((EPI == kPlain || EPI == kSigmoidMul) && BN <= 128) ? 2 : 1; }

template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, min_ctas_per_sm<BN, EPI>()) gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                                                       const __grid_constant__ CUtensorMap tmB,
                                                       const __grid_constant__ CUtensorMap tmC, GemmParams p) {
  constexpr bool kDualA = (EPI == kGatedT);   // gate and proj rows of the stacked weight as two A tiles: transposed (channel-major) output
  using S = Smem<BN, kDualA>;
  constexpr bool kDual = (EPI == kGated || EPI == kSwiGLU || EPI == kSwiGLUBwd || EPI == kGatedBwd);
  constexpr bool kBwd = (EPI == kSwiGLUBwd || EPI == kGatedBwd);
  constexpr int kOutPerTile = kDual ? BN / 2 : BN;  // output columns one tile produces
  constexpr int kAccCols = (kDualA ? 2 : 1) * BN;   // tensor-memory columns of one accumulator buffer
  constexpr uint32_t kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
  static_assert(kTmemCols <= 512, "accumulator buffers exceed tensor memory");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = p.b_resident ? S::kABytes : S::kStageBytes;
  uint8_t* b_res = tiles + (size_t)p.stages * stage_bytes;   // resident weight tile: kb_total blocks of kBBytes
  uint8_t* c_stage = b_res + (p.b_resident ? (size_t)p.kb_total * S::kBBytes : 0);   // two 128 x 64 bf16 boxes when tma_store
  uint64_t* full = reinterpret_cast<uint64_t*>(c_stage + (p.tma_store ? 2 * 16384 : 0));
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;   // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint64_t* b_full = acc_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&acc_full[s], 1);
      ptx::mbar_init(&acc_empty[s], kEpiThreads);
    }
    ptx::mbar_init(b_full, 1);
    ptx::fence_barrier_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
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
      long long it = 0;  // k blocks issued so far by this CTA (the ring position)
      bool ok = true;
      TileCoord c;
      auto load_b = [&](uint8_t* b_s, uint64_t* bar, int kb, int n_tile, int bz) {
        if (p.b_mn) {
#pragma unroll
          for (int blk = 0; blk < BN / 64; ++blk) ptx::tma_load_3d(b_s + blk * 8192, &tmB, bar, n_tile * BN + blk * 64, kb * BK, bz);
        } else if (kDual) {
          ptx::tma_load_3d(b_s, &tmB, bar, kb * BK, n_tile * (BN / 2), bz);
          ptx::tma_load_3d(b_s + S::kBBytes / 2, &tmB, bar, kb * BK, p.proj_row_offset + n_tile * (BN / 2), bz);
        } else {
          ptx::tma_load_3d(b_s, &tmB, bar, kb * BK, n_tile * BN, bz);
        }
      };
      if (p.b_resident && tile_at(p, 0, c)) {
        ptx::mbar_expect_tx(b_full, (uint32_t)(p.kb_total * S::kBBytes));
        for (int kb = 0; kb < p.kb_total; ++kb) load_b(b_res + (size_t)kb * S::kBBytes, b_full, kb, c.n_tile, 0);
      }
      for (long long i = 0; ok && tile_at(p, i, c); ++i) {
        const int kb0 = c.split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        const int az = p.a_batched ? c.batch : 0, bz = p.b_batched ? c.batch : 0;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = (int)(it % p.stages);
          const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
          if (!ptx::mbar_wait(&empty[s], ph ^ 1u, p.status, kTimeoutStageEmpty)) { ok = false; break; }
          uint8_t* a_s = tiles + (size_t)s * stage_bytes;
          uint8_t* b_s = a_s + S::kABytes;
          ptx::mbar_expect_tx(&full[s], (uint32_t)stage_bytes);
          if (p.a_mn) {  // [k][m] with m contiguous: two 64-wide column blocks of 64 k rows
            ptx::tma_load_3d(a_s, &tmA, &full[s], c.m_tile * BM, kb * BK, az);
            ptx::tma_load_3d(a_s + 8192, &tmA, &full[s], c.m_tile * BM + 64, kb * BK, az);
          } else {
            ptx::tma_load_3d(a_s, &tmA, &full[s], kb * BK, c.m_tile * BM, az);
            if (kDualA) ptx::tma_load_3d(a_s + BM * BK * 2, &tmA, &full[s], kb * BK, p.proj_row_offset + c.m_tile * BM, az);
          }
          if (!p.b_resident) load_b(b_s, &full[s], kb, c.n_tile, bz);
        }
      }
      if (!ok) {  // give up: let the copies already in flight land before the CTA's shared memory goes away
        const long long first = it > p.stages ? it - p.stages : 0;
        for (long long k = first; k < it; ++k) ptx::mbar_wait_quiet(&full[k % p.stages], (uint32_t)(k / p.stages) & 1u);
        if (p.b_resident) ptx::mbar_wait_quiet(b_full, 0);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      const uint32_t idesc = ptx::idesc_bf16_f32(BM, BN) | (p.a_mn ? ptx::kIdescAMnMajor : 0u) | (p.b_mn ? ptx::kIdescBMnMajor : 0u);
      long long it = 0;
      bool ok = true;
      TileCoord c;
      if (p.b_resident && tile_at(p, 0, c)) ok = ptx::mbar_wait(b_full, 0, p.status, kTimeoutTmaFull);
      for (long long local = 0; ok && tile_at(p, local, c); ++local) {
        const int kb0 = c.split * p.kb_per_split, kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        const int ab = (int)(local & 1);
        if (!ptx::mbar_wait(&acc_empty[ab], (uint32_t)((local >> 1) & 1) ^ 1u, p.status, kTimeoutStageEmpty)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t acc = tmem + ab * kAccCols;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = (int)(it % p.stages);
          const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
          if (!ptx::mbar_wait(&full[s], ph, p.status, kTimeoutTmaFull)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t a_addr = ptx::smem_u32(tiles + (size_t)s * stage_bytes);
          const uint32_t b_addr = p.b_resident ? ptx::smem_u32(b_res + (size_t)kb * S::kBBytes) : a_addr + S::kABytes;
          const uint64_t a_desc = p.a_mn ? ptx::smem_desc_mn_sw128(a_addr, 8192) : ptx::smem_desc_k_sw128(a_addr);
          const uint64_t b_desc = p.b_mn ? ptx::smem_desc_mn_sw128(b_addr, 8192) : ptx::smem_desc_k_sw128(b_addr);
          // 16 bf16 along K per MMA: 32 bytes inside the swizzled row (K-major) or 16 rows of 128 bytes (MN-major)
          const uint64_t a_step = p.a_mn ? (2048 >> 4) : 2, b_step = p.b_mn ? (2048 >> 4) : 2;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint32_t accum = (kb != kb0 || k != 0) ? 1u : 0u;
            ptx::umma_bf16(acc, a_desc + a_step * k, b_desc + b_step * k, idesc, accum);
            if (kDualA) {
              const uint64_t a2 = ptx::smem_desc_k_sw128(a_addr + BM * BK * 2);
              ptx::umma_bf16(acc + BN, a2 + 2 * k, b_desc + b_step * k, idesc, accum);
            }
          }
          ptx::umma_commit(&empty[s]);
        }
        if (ok) ptx::umma_commit(&acc_full[ab]);
      }
    }
  } else {
    const int q = warp & 3;           // TMEM lane quarter this warp may read
    const int chalf = (warp - 2) >> 2;  // which half of the 32-column chunks this warp takes
    constexpr bool kCanTmaStore = kOutPerTile >= 64;
    const bool tma_out = kCanTmaStore && p.tma_store;
    const bool issuer = threadIdx.x == 64;  // first epilogue thread: issues and tracks the TMA stores
    const int row_in_tile = q * 32 + lane;
    // this thread's 128-byte line inside a staged 128 x 64 box; 16-byte chunks are XOR-swizzled by the row
    uint8_t* stage_row = c_stage + (row_in_tile >> 3) * 1024 + (row_in_tile & 7) * 128;
    const int swz = row_in_tile & 7;
    auto stage32 = [&](int buf, const float* v) {  // 32 values -> this thread's half of the staged line
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 w;
        w.x = pack_bf16(v[g * 8 + 0], v[g * 8 + 1]);
        w.y = pack_bf16(v[g * 8 + 2], v[g * 8 + 3]);
        w.z = pack_bf16(v[g * 8 + 4], v[g * 8 + 5]);
        w.w = pack_bf16(v[g * 8 + 6], v[g * 8 + 7]);
        *reinterpret_cast<uint4*>(stage_row + buf * 16384 + (((chalf * 4 + g) ^ swz) << 4)) = w;
      }
    };
    int boxes = 0;  // 64-column boxes staged so far by this CTA (buffer = boxes & 1 for single-output epilogues)
    bool ok = true;
    TileCoord c;
    for (long long local = 0; ok && tile_at(p, local, c); ++local) {
      const int ab = (int)(local & 1);
      if (kBwd || EPI == kSigmoidMul) {
        // the epilogue's second operand of the next tile: ask for this thread's 128 bytes of it now, so that they are
        // in L2 by the time the rows are read (the reads are one dependent load per chunk, nothing else hides them)
        TileCoord nx;
        if (tile_at(p, local + 1, nx)) {
          const int prow = nx.m_tile * BM + row_in_tile;
          const int pcol = nx.n_tile * kOutPerTile + chalf * 64;
          if (prow < p.M && pcol < p.N) {
            const __nv_bfloat16* src = p.mul + (long long)nx.batch * p.mul_batch_stride + (long long)prow * p.ld_mul + pcol;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
          }
        }
      }
      if (!ptx::mbar_wait(&acc_full[ab], (uint32_t)(local >> 1) & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
      ptx::tc_fence_after();
      const int row = c.m_tile * BM + row_in_tile;
      const uint32_t t_row = tmem + ab * kAccCols + ((uint32_t)(q * 32) << 16);
      const long long batch = c.batch;
      const long long c_off = batch * p.c_batch_stride + (long long)c.split * p.c_split_stride;
      const float* mask_b = p.row_mask ? p.row_mask + batch * p.mask_batch_stride : nullptr;
      const float rm = (mask_b != nullptr && !p.mask_on_n && row < p.M) ? mask_b[row] : 1.f;
      const float bm = (p.bias != nullptr && p.bias_on_m && row < p.M) ? p.bias[row] : 0.f;
      float a[32], b[32];
#pragma unroll 1
      for (int cc = (kOutPerTile >= 64 ? chalf : 0); cc < kOutPerTile / 32; cc += (kOutPerTile >= 64 ? 2 : 1)) {
        const int n0 = c.n_tile * kOutPerTile + cc * 32;
        const bool live = n0 < p.N && !(kOutPerTile < 64 && chalf != 0);   // uniform over the warp
        if (!live && !tma_out) break;
        if (live) {
          ptx::tmem_ld_32x32(t_row + cc * 32, a);
          if (kDual) ptx::tmem_ld_32x32(t_row + BN / 2 + cc * 32, b);
          if (kDualA) ptx::tmem_ld_32x32(t_row + BN + cc * 32, b);
          ptx::tmem_ld_wait();
          if (EPI == kPlain) {
            if (p.bias != nullptr && !p.bias_on_m) {
#pragma unroll
              for (int j = 0; j < 32; ++j) a[j] += (n0 + j < p.N) ? p.bias[n0 + j] : 0.f;
            }
            if (mask_b != nullptr && p.mask_on_n) {
#pragma unroll
              for (int j = 0; j < 32; ++j) a[j] = (a[j] + bm) * ((n0 + j < p.N) ? mask_b[n0 + j] : 0.f);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) a[j] = (a[j] + bm) * rm;
            }
          } else if (EPI == kGated) {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] = sigmoid_fast(a[j]) * b[j] * rm;
          } else if (EPI == kGatedT) {
            // rows are output channels, columns are the input rows: the mask runs along the columns
            if (mask_b != nullptr && n0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(mask_b + n0) & 15) == 0)) {
#pragma unroll
              for (int g4 = 0; g4 < 8; ++g4) {
                const float4 mk = *reinterpret_cast<const float4*>(mask_b + n0 + 4 * g4);
                a[4 * g4 + 0] = sigmoid_fast(a[4 * g4 + 0]) * b[4 * g4 + 0] * mk.x;
                a[4 * g4 + 1] = sigmoid_fast(a[4 * g4 + 1]) * b[4 * g4 + 1] * mk.y;
                a[4 * g4 + 2] = sigmoid_fast(a[4 * g4 + 2]) * b[4 * g4 + 2] * mk.z;
                a[4 * g4 + 3] = sigmoid_fast(a[4 * g4 + 3]) * b[4 * g4 + 3] * mk.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float mk = mask_b ? ((n0 + j < p.N) ? mask_b[n0 + j] : 0.f) : 1.f;
                a[j] = sigmoid_fast(a[j]) * b[j] * mk;
              }
            }
          } else if (EPI == kSwiGLU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) a[j] = a[j] * sigmoid_fast(a[j]) * b[j];
          } else if (kBwd) {
            const __nv_bfloat16* grow = p.mul + batch * p.mul_batch_stride + (long long)row * p.ld_mul + n0;
            float g[32];
            load_row32(grow, row < p.M, n0, p.N, g);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float sg = sigmoid_fast(a[j]);
              const float gj = g[j] * rm;
              const float da = EPI == kSwiGLUBwd ? gj * b[j] * sg * (1.f + a[j] * (1.f - sg)) : gj * b[j] * sg * (1.f - sg);
              const float dbv = EPI == kSwiGLUBwd ? gj * a[j] * sg : gj * sg;
              a[j] = da;
              b[j] = dbv;
            }
          } else {  // kSigmoidMul
            const __nv_bfloat16* mrow = p.mul + batch * p.mul_batch_stride + (long long)row * p.ld_mul + n0;
            float g[32];
            load_row32(mrow, row < p.M, n0, p.N, g);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float bv = (p.bias != nullptr && n0 + j < p.N) ? p.bias[n0 + j] : 0.f;
              a[j] = sigmoid_fast(a[j] + bv) * g[j];
            }
          }
        }
        if (tma_out) {
          // the 64-column box this chunk belongs to leaves through shared memory: both column halves (the two warps of a
          // lane quarter) stage their 32 columns, then one thread hands the box to the TMA unit, which clips it at the
          // tensor's bounds. The backward epilogues stage two boxes (both output halves) per round.
          if ((c.n_tile * kOutPerTile + (cc & ~1) * 32) >= p.N) break;  // whole box beyond the output: the same for all threads
          const int buf = kBwd ? 0 : (boxes & 1);
          if (issuer) { if (kBwd) ptx::tma_store_wait_read<0>(); else ptx::tma_store_wait_read<1>(); }
          ptx::named_barrier(1, kEpiThreads);   // the buffer's previous box has been read out
          stage32(buf, a);
          if (kBwd) stage32(1, b);
          ptx::fence_proxy_async();
          ptx::named_barrier(1, kEpiThreads);   // the box is complete
          if (issuer) {
            const int x0 = c.n_tile * kOutPerTile + (cc & ~1) * 32;
            ptx::tma_store_3d(&tmC, c_stage + buf * 16384, x0, c.m_tile * BM, c.batch);
            if (kBwd) ptx::tma_store_3d(&tmC, c_stage + 16384, p.N + x0, c.m_tile * BM, c.batch);
            ptx::tma_store_commit();
          }
          ++boxes;
        } else if (kBwd) {
          store_row32(p, p.C, c_off, row, n0, a);
          store_row32(p, reinterpret_cast<__nv_bfloat16*>(p.C) + p.N, c_off, row, n0, b);  // second half of the [M, 2 N] output
        } else {
          store_row32(p, p.C, c_off, row, n0, a);
        }
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(&acc_empty[ab]);
    }
    if (tma_out && issuer) ptx::tma_store_wait_read<0>();  // shared memory stays valid until the last box has been read
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

// out[e] = sum over the splits of partial[s][e] (+ nothing else: split launches use the plain epilogue without bias).
template <typename OutT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, OutT* __restrict__ out, long long n,
                                                            int splits) {
  const long long e = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (e >= n) return;
  if (e + 4 <= n) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + (long long)s * n + e);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    out[e] = from_float<OutT>(acc.x); out[e + 1] = from_float<OutT>(acc.y);
    out[e + 2] = from_float<OutT>(acc.z); out[e + 3] = from_float<OutT>(acc.w);
  } else {
    for (long long k = e; k < n; ++k) {
      float acc = 0.f;
      for (int s = 0; s < splits; ++s) acc += partial[(long long)s * n + k];
      out[k] = from_float<OutT>(acc);
    }
  }
}

// ---- host ---------------------------------------------------------------------------------------
int sm_count() {
  static int n = [] {
    int dev = 0, v = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

// K-major operand [batch, rows, K]: box = 64 k x box_rows; MN-major operand [batch, K, cols]: box = 64 cols x 64 k.
CUtensorMap operand_map(const Tensor& t3, bool mn_major, int box_rows) {
  const int64_t inner = t3.size(2), rows = t3.size(1), batch = t3.size(0);
  const int64_t dims[3] = {inner, rows, batch};
  const int64_t strides[3] = {1, t3.stride(1), batch > 1 ? t3.stride(0) : rows * t3.stride(1)};
  const int box[3] = {BK, mn_major ? BK : box_rows, 1};
  return make_map_nd(t3.data_ptr(), 3, dims, strides, box);
}

// bf16 output [batch, rows, cols] (contiguous) as a store target: boxes of 64 columns x 128 rows
CUtensorMap output_map(const Tensor& out, int64_t rows, int64_t cols, int64_t batch) {
  const int64_t dims[3] = {cols, rows, batch};
  const int64_t strides[3] = {1, cols, rows * cols};
  const int box[3] = {64, BM, 1};
  return make_map_nd(out.data_ptr(), 3, dims, strides, box);
}

template <int BN, int EPI>
void launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmParams& p, cudaStream_t stream) {
  using S = Smem<BN, EPI == kGatedT>;
  const int per_tile_k = p.kb_per_split;
  const long long tiles = (long long)p.m_tiles * p.n_tiles * p.batch * p.splits;
  TORCH_CHECK(tiles > 0 && tiles < (1ll << 40), "gemm: grid too large");
  constexpr int acc_cols = (EPI == kGatedT ? 2 : 1) * BN * 2;
  const int sms = sm_count();
  // Tall product against a small broadcast weight (the pair-shaped linears: K <= 256, hundreds of row tiles): each CTA
  // keeps its weight tile in shared memory and streams row tiles through a ring that holds A only. Otherwise every
  // output tile would fetch the weight tile again and the L2-to-SM traffic of the weights would exceed the traffic of
  // the activations.
  p.b_resident = (!p.b_batched && p.splits == 1 && p.kb_total <= kMaxResidentK && EPI != kGatedT &&
                  (long long)p.m_tiles * p.batch >= 4ll * sms / std::max(1, p.n_tiles) && p.n_tiles <= sms) ? 1 : 0;
  constexpr bool dual_b = (EPI == kGated || EPI == kSwiGLU || EPI == kSwiGLUBwd || EPI == kGatedBwd);
  if ((dual_b ? BN / 2 : BN) < 64) p.tma_store = 0;  // narrow tiles store from registers
  const size_t extra = (p.tma_store ? 2 * 16384 : 0) + 1024 + 256;
  int stages;
  size_t smem;
  if (p.b_resident) {
    // a short ring when that lets two CTAs share an SM (K = 128: weight 32 KiB + two A blocks + the store boxes)
    stages = (min_ctas_per_sm<BN, EPI>() == 2 && 2 * S::kABytes + (size_t)p.kb_total * S::kBBytes + extra <= 110 * 1024) ? 2 : 6;
    smem = (size_t)stages * S::kABytes + (size_t)p.kb_total * S::kBBytes + extra;
  } else {
    // a deep ring when the K loop is long; short loops still get enough stages for the loads of the next tile to run
    // ahead of the epilogue, but few enough for two CTAs per SM when the accumulators allow it
    stages = per_tile_k >= 8 ? 6 : (acc_cols <= 256 && 3 * S::kStageBytes + extra <= 110 * 1024 ? 3 : 4);
    while (stages > 2 && (size_t)stages * S::kStageBytes + extra > 226 * 1024) --stages;
    smem = (size_t)stages * S::kStageBytes + extra;
  }
  p.stages = stages;
  static bool attr_set = false;
  if (!attr_set) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set = true;
  }
  // one CTA per SM, or two when both the shared memory and the tensor-memory columns allow it
  const int per_sm = (smem <= 110 * 1024 && acc_cols <= 256 && min_ctas_per_sm<BN, EPI>() == 2) ? 2 : 1;
  long long ctas = std::min<long long>(tiles, (long long)sms * per_sm);
  if (p.b_resident) {
    const long long groups = std::max<long long>(1, std::min<long long>((long long)sms * per_sm / p.n_tiles, (long long)p.m_tiles * p.batch));
    ctas = groups * p.n_tiles;
  }
  gemm_kernel<BN, EPI><<<(unsigned)ctas, kThreads, smem, stream>>>(ta, tb, tc, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

struct GemmOpts {
  Tensor out;                        // optional preallocated contiguous [batch, M, N] result of the plain epilogue
  bool a_mn = false, b_mn = false;   // a3 is [batch, K, M] / w3 is [wb, K, N] (contiguous M / N) instead of [.., rows, K]
  bool out_fp32 = false;
  bool channel_major = false;        // return [batch, N, M]
  int splits = 1;                    // split the K loop; partial sums are added in a fixed order afterwards
};

// a: [batch or 1, M, K] (or [.., K, M] when a_mn); w: [wb, Nw, K] (or [wb, K, Nw] when b_mn); returns [batch, M, N]
// (or [batch, N, M] when channel_major), bf16 or fp32.
Tensor gemm_impl(const Tensor& a3, const Tensor& w3, const c10::optional<Tensor>& bias, const c10::optional<Tensor>& row_mask,
                 const c10::optional<Tensor>& mul, int epi, GemmOpts o) {
  TORCH_CHECK(a3.is_cuda() && a3.scalar_type() == torch::kBFloat16 && w3.scalar_type() == torch::kBFloat16,
              "gemm: bf16 CUDA tensors expected");
  TORCH_CHECK(a3.dim() == 3 && w3.dim() == 3 && a3.stride(2) == 1 && w3.stride(2) == 1, "gemm: 3-D operands with a contiguous last axis");
  const int64_t ab = a3.size(0), wb = w3.size(0);
  const int64_t M = o.a_mn ? a3.size(2) : a3.size(1), K = o.a_mn ? a3.size(1) : a3.size(2);
  const int64_t Nw = o.b_mn ? w3.size(2) : w3.size(1), Kw = o.b_mn ? w3.size(1) : w3.size(2);
  const int64_t batch = std::max(ab, wb);
  TORCH_CHECK(Kw == K && (wb == 1 || wb == batch) && (ab == 1 || ab == batch), "gemm: operand shapes disagree");
  TORCH_CHECK(a3.size(2) % 8 == 0 && w3.size(2) % 8 == 0 && a3.stride(1) % 8 == 0 && w3.stride(1) % 8 == 0,
              "gemm: contiguous extents and row strides must be multiples of 8");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(a3.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(w3.data_ptr()) % 16 == 0,
              "gemm: operands must be 16-byte aligned");
  TORCH_CHECK((ab == 1 || a3.stride(0) % 8 == 0) && (wb == 1 || w3.stride(0) % 8 == 0), "gemm: batch strides must be multiples of 8");
  const bool dual = (epi == kGated || epi == kSwiGLU || epi == kSwiGLUBwd || epi == kGatedBwd);
  const bool bwd = (epi == kSwiGLUBwd || epi == kGatedBwd);
  TORCH_CHECK(!bwd || !o.channel_major, "gemm: the backward epilogues store row-major");
  TORCH_CHECK(!dual || Nw % 2 == 0, "gemm: stacked gate/proj weight expected");
  TORCH_CHECK(epi == kPlain || (!o.a_mn && !o.b_mn && !o.out_fp32 && o.splits == 1), "gemm: fused epilogues take K-major operands");
  const int64_t N = dual ? Nw / 2 : Nw;
  TORCH_CHECK(M < (1ll << 31) && N < (1ll << 31) && K < (1 << 24), "gemm: size out of range");
  c10::cuda::CUDAGuard guard(a3.device());
  auto opts = a3.options();
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();

  // Channel-major output of the plain and gated epilogues: compute the transposed product instead (the weight becomes
  // the A operand, so a tensor-memory lane is an output channel and every thread stores contiguous runs of one plane).
  if (o.channel_major && (epi == kPlain || epi == kGated) && !o.a_mn && !o.b_mn && M >= 64) {
    TORCH_CHECK(ab == batch || batch == 1, "gemm: channel-major output with a broadcast input");
    Tensor out = torch::empty({batch, N, M}, opts);
    if (out.numel() == 0) return out;
    GemmParams p{};
    p.C = out.data_ptr();
    p.c_elems = out.numel();
    Tensor bias_f, mask_f;
    if (bias.has_value() && bias->defined()) {
      bias_f = bias->to(torch::kFloat32).contiguous();
      TORCH_CHECK(bias_f.numel() == N, "gemm: bias length");
      p.bias = bias_f.data_ptr<float>();
      p.bias_on_m = 1;
    }
    if (row_mask.has_value() && row_mask->defined()) {
      mask_f = row_mask->to(torch::kFloat32).contiguous();
      TORCH_CHECK(mask_f.numel() == batch * M, "gemm: row mask length");
      p.row_mask = mask_f.data_ptr<float>();
      p.mask_on_n = 1;
      p.mask_batch_stride = M;
    }
    Tensor status = status_word(a3.device().index());
    p.status = status.data_ptr<int>();
    p.M = (int)N; p.N = (int)M; p.K = (int)K;   // roles swapped
    constexpr int BN = 128;
    p.m_tiles = (int)((N + BM - 1) / BM);
    p.n_tiles = (int)((M + BN - 1) / BN);
    p.batch = (int)batch; p.splits = 1;
    p.kb_total = p.kb_per_split = (int)((K + BK - 1) / BK);
    p.a_batched = wb > 1; p.b_batched = ab > 1;
    p.proj_row_offset = (int)N;
    p.ldc = M;
    p.c_batch_stride = N * M;
    const CUtensorMap ta = operand_map(w3, false, BM);
    const CUtensorMap tb = operand_map(a3, false, BN);
    p.tma_store = (M % 8 == 0) ? 1 : 0;
    const CUtensorMap tc = p.tma_store ? output_map(out, N, M, batch) : ta;
    if (epi == kPlain) launch<BN, kPlain>(ta, tb, tc, p, stream); else launch<BN, kGatedT>(ta, tb, tc, p, stream);
    return out;
  }

  // accumulator width: the widest tile that the output needs
  int BN;
  if (dual) BN = N >= 128 ? 256 : (N >= 64 ? 128 : 64);
  else BN = (epi == kPlain && N > 128 && K >= 512 && M * batch > 2048 && M >= 256) ? 256 : (N > 64 ? 128 : (N > 32 ? 64 : 32));
  if (o.b_mn && BN < 64) BN = 64;
  const int out_per_tile = dual ? BN / 2 : BN;

  GemmParams p{};
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
    p.mask_batch_stride = M;
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
  p.batch = (int)batch;
  p.kb_total = (int)((K + BK - 1) / BK);
  int splits = std::max(1, std::min(o.splits, p.kb_total));
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
  p.splits = splits;
  p.a_batched = ab > 1; p.b_batched = wb > 1;
  p.proj_row_offset = (int)N;
  p.a_mn = o.a_mn; p.b_mn = o.b_mn;
  const int64_t out_cols = bwd ? 2 * N : N;
  if (o.out.defined())
    TORCH_CHECK(epi == kPlain && !o.channel_major && o.out.is_contiguous() && o.out.numel() == batch * M * N &&
                o.out.scalar_type() == (o.out_fp32 ? torch::kFloat32 : torch::kBFloat16), "gemm: preallocated output shape / dtype");
  Tensor out, partial;
  if (splits > 1) {
    TORCH_CHECK(!o.channel_major && epi == kPlain && !p.bias && !p.row_mask, "gemm: split-K takes the plain epilogue");
    partial = torch::empty({splits, batch, M, N}, opts.dtype(torch::kFloat32));
    out = o.out.defined() ? o.out : torch::empty({batch, M, N}, o.out_fp32 ? opts.dtype(torch::kFloat32) : opts);
    p.C = partial.data_ptr();
    p.c_fp32 = 1;
    p.c_split_stride = batch * M * N;
  } else {
    out = o.out.defined() ? o.out
          : o.channel_major ? torch::empty({batch, N, M}, opts)
                            : torch::empty({batch, M, out_cols}, o.out_fp32 ? opts.dtype(torch::kFloat32) : opts);
    p.C = out.data_ptr();
    p.c_elems = out.numel();
    p.c_fp32 = o.out_fp32;
  }
  if (out.numel() == 0) return out;
  p.channel_major = o.channel_major;
  p.ldc = o.channel_major ? M : out_cols;
  p.c_batch_stride = M * out_cols;

  const CUtensorMap ta = operand_map(a3, o.a_mn, BM);
  const CUtensorMap tb = operand_map(w3, o.b_mn, dual ? BN / 2 : BN);
  p.tma_store = (splits == 1 && !p.c_fp32 && !o.channel_major && out_cols % 8 == 0 && N % 8 == 0 &&
                 reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0) ? 1 : 0;
  const CUtensorMap tc = p.tma_store ? output_map(out, M, out_cols, batch) : ta;
#define DF3_LAUNCH(BN_, EPI_) launch<BN_, EPI_>(ta, tb, tc, p, stream)
  switch (epi) {
    case kPlain:
      if (BN == 256) DF3_LAUNCH(256, kPlain); else if (BN == 128) DF3_LAUNCH(128, kPlain); else if (BN == 64) DF3_LAUNCH(64, kPlain); else DF3_LAUNCH(32, kPlain);
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
  if (splits > 1) {
    const long long n = out.numel();
    const unsigned grid = (unsigned)((n / 4 + 256) / 256);
    if (o.out_fp32)
      splitk_reduce_kernel<float><<<grid, 256, 0, stream>>>(partial.data_ptr<float>(), out.data_ptr<float>(), n, splits);
    else
      splitk_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(partial.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), n, splits);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
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
  GemmOpts o;
  o.channel_major = channel_major;
  Tensor out = gemm_impl(a3, w3, bias, row_mask, mul, (int)epi, o);
  if (channel_major) return out.view({out.size(1), out.size(2)});
  auto shape = xc.sizes().vec();
  shape.back() = out.size(2);
  return out.view(shape);
}

Tensor as3d(const Tensor& t) {
  Tensor c = t.dim() == 2 ? t.unsqueeze(0) : t;
  TORCH_CHECK(c.dim() == 3, "bmm: 2-D or 3-D operands");
  if (c.stride(2) != 1 || c.stride(1) % 8 != 0 || (c.size(0) > 1 && c.stride(0) % 8 != 0) ||
      reinterpret_cast<uintptr_t>(c.data_ptr()) % 16 != 0)
    c = c.contiguous();
  return c.scalar_type() == torch::kBFloat16 ? c : c.to(torch::kBFloat16);
}

// a: [B, M, K], b: [B, N, K] -> [B, M, N]: sum over the shared last axis (both K-major).
Tensor df3_bmm_nt(const Tensor& a, const Tensor& b) {
  TORCH_CHECK(a.dim() == 3 && b.dim() == 3 && a.size(0) == b.size(0), "bmm_nt: [B, M, K] x [B, N, K]");
  return gemm_impl(as3d(a), as3d(b), c10::nullopt, c10::nullopt, c10::nullopt, kPlain, GemmOpts{});
}

// General product on the tcgen05 kernel: out[b, m, n] = sum_k A[b, m, k] B[b, k, n] with either operand given transposed.
//   a: [B or 1, M, K], or [B or 1, K, M] with trans_a;  b: [B or 1, K, N], or [B or 1, N, K] with trans_b.
// No operand is copied as long as its last axis is contiguous. `splits` > 1 cuts the K loop into that many pieces whose
// fp32 partial results are added in a fixed order (long-K products with few output tiles: weight gradients); 0 picks
// a count that fills the GPU.
Tensor df3_matmul(const Tensor& a, const Tensor& b, bool trans_a, bool trans_b, bool out_fp32, int64_t splits,
                  const c10::optional<Tensor>& out_given = c10::nullopt) {
  Tensor a3 = as3d(a), b3 = as3d(b);
  GemmOpts o;
  if (out_given.has_value() && out_given->defined()) o.out = *out_given;
  o.a_mn = trans_a;          // [K, M] with M contiguous
  o.b_mn = !trans_b;         // [K, N] with N contiguous
  o.out_fp32 = out_fp32;
  const int64_t M = trans_a ? a3.size(2) : a3.size(1), K = trans_a ? a3.size(1) : a3.size(2);
  const int64_t N = trans_b ? b3.size(1) : b3.size(2);
  if (splits == 0) {
    const int64_t tiles = ((M + 127) / 128) * ((N + 127) / 128) * std::max(a3.size(0), b3.size(0));
    const int64_t kb = (K + BK - 1) / BK;
    splits = 1;
    if (tiles < sm_count() && kb >= 16) splits = std::min<int64_t>(std::max<int64_t>(1, sm_count() / tiles), kb / 4);
  }
  o.splits = (int)std::max<int64_t>(1, splits);
  Tensor out = gemm_impl(a3, b3, c10::nullopt, c10::nullopt, c10::nullopt, kPlain, o);
  if (o.out.defined()) return out;
  return (a.dim() == 2 && b.dim() == 2) ? out.squeeze(0) : out;
}

// Backward of y = x w^T (+ b) with bf16 operands: dx = dy w (in x's dtype), dw = dy^T x and db = sum dy in fp32.
// Both products run on the tcgen05 kernel without transposing anything: dy is the K-major A operand of dx and the
// MN-major A operand of dw; w and x are MN-major B operands. dw is a split-K launch with an order-fixed reduction.
// The same product for any extents: an operand whose last two extents are not multiples of 8 (TMA rows have to be
// 16-byte multiples) is zero-padded, which leaves the product unchanged, and the result is cut back. With `out` the
// result lands in that tensor (directly when no padding was needed).
Tensor matmul_any_impl(const Tensor& a, const Tensor& b, bool trans_a, bool trans_b, bool out_fp32, int64_t splits,
                       const c10::optional<Tensor>& out = c10::nullopt) {
  auto pad8 = [](const Tensor& t) {
    const int64_t r = (8 - t.size(-2) % 8) % 8, c = (8 - t.size(-1) % 8) % 8;
    return (r || c) ? at::constant_pad_nd(t, {0, c, 0, r}, 0) : t;
  };
  const Tensor a8 = pad8(a.contiguous()), b8 = pad8(b.contiguous());
  const bool padded = a8.data_ptr() != a.data_ptr() || b8.data_ptr() != b.data_ptr() || !a.is_contiguous() || !b.is_contiguous();
  const int64_t rows = trans_a ? a.size(-1) : a.size(-2), cols = trans_b ? b.size(-2) : b.size(-1);
  if (out.has_value() && out->defined() && a8.size(-1) == a.size(-1) && a8.size(-2) == a.size(-2) && b8.size(-1) == b.size(-1) &&
      b8.size(-2) == b.size(-2) && out->is_contiguous())
    return df3_matmul(a8, b8, trans_a, trans_b, out_fp32, splits, out);
  (void)padded;
  Tensor full = df3_matmul(a8, b8, trans_a, trans_b, out_fp32, splits);
  Tensor cut = full.narrow(-2, 0, rows).narrow(-1, 0, cols);
  if (out.has_value() && out->defined()) {
    out->copy_(cut.view(out->sizes()));
    return *out;
  }
  return cut.contiguous();
}

std::tuple<Tensor, Tensor, Tensor> df3_linear_bwd(const Tensor& dy, const Tensor& x, const Tensor& w16, bool need_dx, bool need_dw,
                                                   bool need_db) {
  const int64_t n = w16.size(0), k = w16.size(1);
  Tensor d2 = dy.reshape({-1, n});
  if (d2.scalar_type() != torch::kBFloat16) d2 = d2.to(torch::kBFloat16);
  Tensor dx, dw, db;
  const bool any_rows = d2.size(0) > 0;
  if (need_dx) {
    dx = any_rows ? matmul_any_impl(d2, w16, false, false, false, 1) : torch::zeros({0, k}, d2.options());
    dx = dx.view(x.sizes());
    if (dx.scalar_type() != x.scalar_type()) dx = dx.to(x.scalar_type());
  }
  if (need_dw) {
    Tensor x2 = x.reshape({-1, k});
    if (x2.scalar_type() != torch::kBFloat16) x2 = x2.to(torch::kBFloat16);
    dw = any_rows ? matmul_any_impl(d2, x2, true, false, true, 0) : torch::zeros({n, k}, d2.options().dtype(torch::kFloat32));
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

Tensor df3_matmul_any(const Tensor& a, const Tensor& b, bool trans_a, bool trans_b, bool out_fp32, int64_t splits,
                      const c10::optional<Tensor>& out) {
  return matmul_any_impl(a, b, trans_a, trans_b, out_fp32, splits, out);
}
}  // namespace df3

void df3_register_gemm(torch::Library& m) {
  m.def("gemm(Tensor x, Tensor w, Tensor? bias, Tensor? row_mask, Tensor? mul, int epi, bool channel_major) -> Tensor",
        &df3::df3_gemm);
  m.def("bmm_nt(Tensor a, Tensor b) -> Tensor", &df3::df3_bmm_nt);
  m.def("matmul(Tensor a, Tensor b, bool trans_a, bool trans_b, bool out_fp32, int splits, Tensor(a!)? out=None) -> Tensor",
        &df3::df3_matmul);
  m.def("gemm_status() -> int", &df3::df3_gemm_status);
  m.def("linear_bwd(Tensor dy, Tensor x, Tensor w16, bool need_dx, bool need_dw, bool need_db) -> (Tensor, Tensor, Tensor)",
        &df3::df3_linear_bwd);
}

const char* df3_gemm_features() {
  return "gemm,matmul,gated_dual_linear,transition,pair_bias_attention,linear_planes,sigmoid_gate_mul,peer_reduce,peer_exchange,window_attention";
}
