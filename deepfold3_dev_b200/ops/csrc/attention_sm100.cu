// Pair-biased softmax attention, forward, for sm_100a:
//
//   out[b, r, h, i, :] = softmax_j( scale * q[b,r,h,i,:] . k[b,r,h,j,:] + bias[b,h,i,j] + 1e9 * (mask[b,r,j] - 1) ) v[b,r,h,j,:]
//
// q/k/v are strided 5-D views [B, R, H, N, D] (last axis contiguous), so the row and the column
// flavour of triangle attention, the single-representation attention and the diffusion transformer
// (R = samples) all read the projection outputs in place. The bias is shared by the R rows.
//
// One CTA owns 128 queries of one (b, r, h) and streams the keys in blocks of 128:
//   warp 0      TMA producer: Q once, then K blocks into a two-stage ring and V blocks into one stage (5-D tensor maps,
//               128-byte swizzle)
//   warp 1      tcgen05.mma issuer: S = Q K^T into tensor memory, later O_blk = P V
//   warps 2-9   two threads per query row (64 keys and half of the output columns each): S from tensor memory,
//               bias + mask, online softmax in base 2, P (bf16) into swizzled shared memory as the A operand of the
//               second MMA, O accumulated in registers; the pair exchanges row maximum and row sum through shared memory
// Every wait is bounded; a wait that runs out records a df3::Status code and the CTA leaves cleanly.
#include <ATen/cuda/CUDAContext.h>
#include <algorithm>
#include <vector>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "sm100_ptx.cuh"

using torch::Tensor;

namespace df3 {
bool attention_bwd_fused_supported(int64_t N, int64_t D);  // attention_bwd_sm100.cu
std::tuple<Tensor, Tensor, Tensor, Tensor> attention_bwd_fused(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
                                                               const Tensor& d_out, const c10::optional<Tensor>& bias,
                                                               const c10::optional<Tensor>& mask, const Tensor& lse, double scale,
                                                               bool want_dbias, const c10::optional<Tensor>& dq_out,
                                                               const c10::optional<Tensor>& dk_out, const c10::optional<Tensor>& dv_out);
Tensor status_word(int device);                       // gemm_sm100.cu
Tensor df3_matmul_any(const Tensor& a, const Tensor& b, bool trans_a, bool trans_b, bool out_fp32, int64_t splits,
                      const c10::optional<Tensor>& out);  // gemm_sm100.cu: the tcgen05 product for any extents
CUtensorMap make_map_nd(const void* base, int rank, const int64_t* dims, const int64_t* strides_elems,
                        const int* box);              // gemm_sm100.cu

CUtensorMap qkv_map(const Tensor& t) {  // [B, R, H, N, D] view -> 5-D map (d, n, h, r, b), box 64 x 128
  const int64_t dims[5] = {t.size(4), t.size(3), t.size(2), t.size(1), t.size(0)};
  const int64_t strides[5] = {1, t.stride(3), t.stride(2), t.stride(1), t.stride(0)};
  const int box[5] = {64, 128, 1, 1, 1};
  return make_map_nd(t.data_ptr(), 5, dims, strides, box);
}

bool strides_ok(const Tensor& t) {
  if (t.stride(4) != 1 || reinterpret_cast<uintptr_t>(t.data_ptr()) % 16 != 0) return false;
  for (int d = 0; d < 4; ++d)
    if (t.size(d) > 1 && (t.stride(d) % 8 != 0 || t.stride(d) <= 0)) return false;
  return true;
}

namespace {

constexpr int BQ = 128;   // queries per CTA
constexpr int BKEY = 128; // keys per block
constexpr int kTileBytes = 128 * 128;  // 128 rows x 128 bytes (64 bf16): Q, K or V tile
constexpr int kThreads = 320;         // TMA warp, MMA warp, eight softmax warps
constexpr int kSoftmaxThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  __nv_bfloat16* out;
  float* out32;            // [B, R, H, N, D] contiguous fp32 copy of the output for the backward's row sums, or null
  float* lse;              // [2, B, R, H, N] or null: row maximum and log2 of the row sum, both in base 2
  const void* bias;        // [B, H, N, N] or null
  const float* mask;       // [B, R, N] or null (1 keep, 0 drop)
  int* status;
  long long o_sb, o_sr, o_sh, o_sn;           // out strides (elements)
  long long bias_sb, bias_sh, bias_si;        // bias strides (last axis contiguous)
  long long mask_sb, mask_sr;                 // mask strides (last axis contiguous)
  int B, R, H, N, D;       // N: keys per (b, r, h)
  int NQ;                  // queries per (b, r, h); equals N for self-attention, 32 against 128 keys for atom windows
  int q_tiles;
  int bias_is_bf16;
  int bias_tma;            // bias tiles are staged through shared memory by TMA (bf16, contiguous keys, N % 8 == 0)
  float scale_log2;        // scale * log2(e)
};

using ptx::pack2_bf16;
using ptx::smem_desc_mn_sw128;
using ptx::tma_load_4d;
using ptx::tma_load_5d;
using ptx::tmem_st_32x32;
using ptx::tmem_st_wait;
__device__ __forceinline__ uint32_t pack2(float lo, float hi) { return pack2_bf16(lo, hi); }

// instruction descriptor of the second MMA: A (P) K-major, B (V) MN-major
__host__ __device__ constexpr uint32_t idesc_pv(int m, int n) { return ptx::idesc_bf16_f32(m, n) | (1u << 16); }

template <int DN>  // head width rounded up to 16: 16, 32, 48 or 64
__global__ void __launch_bounds__(kThreads, 2) attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                   const __grid_constant__ CUtensorMap tmK,
                                                                   const __grid_constant__ CUtensorMap tmV,
                                                                   const __grid_constant__ CUtensorMap tmBias, AttnParams p) {
  // shared memory: Q | K stage 0 | K stage 1 | V | P (two 64-key atoms) | barriers | key term | row exchange
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_s = smem;
  uint8_t* k_s = smem + kTileBytes;                  // two stages
  uint8_t* v_s = smem + 3 * kTileBytes;              // one stage: V of block j + 1 is fetched while softmax j + 1 runs
  uint8_t* p_s = smem + 4 * kTileBytes;              // 128 x 128 bf16: two 64-key atoms of 16 KiB
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTileBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 6;
  uint64_t* s_ready = bars + 7;
  uint64_t* p_ready = bars + 8;
  uint64_t* o_ready = bars + 9;
  uint64_t* x_ready = bars + 10;  // [2]: row-maximum exchange between the two threads of a row, by block parity
  uint64_t* bias_full = bars + 13;  // the bias tile of the next block sits in the P buffer (each thread reads its own
                                    // 128 bytes in pass 1 and overwrites exactly those with P in pass 2)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  // one copy for the eight softmax warps: each warp writes all 128 (identical) values itself before it reads them,
  // and no warp starts the next key block before every warp has finished reading this one (o_ready follows p_ready)
  float* key_add = reinterpret_cast<float*>(bars + 16);  // [128]
  float* xchg = key_add + 128;                           // [2 parities][2 halves][128 rows]
  constexpr uint32_t kTmemCols = 256;  // S: columns [0, 128), O block: [128, 128 + DN)
  constexpr int DH = DN / 2;           // output columns per thread

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int idx = blockIdx.x;
  const int qt = idx % p.q_tiles; idx /= p.q_tiles;
  const int h = idx % p.H; idx /= p.H;
  const int r = idx % p.R;
  const int b = idx / p.R;
  const int nb = (p.N + BKEY - 1) / BKEY;

  if ((ptx::smem_u32(smem) & 1023u) != 0) {  // the swizzle pattern assumes 1024-byte aligned tiles
    if (threadIdx.x == 0) atomicCAS(p.status, kOk, kBadShape);
    return;
  }
  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&k_full[s], 1);
      ptx::mbar_init(&k_empty[s], 1);
      ptx::mbar_init(&x_ready[s], kSoftmaxThreads);
    }
    ptx::mbar_init(v_full, 1);
    ptx::mbar_init(v_empty, 1);
    ptx::mbar_init(s_ready, 1);
    ptx::mbar_init(p_ready, kSoftmaxThreads);
    ptx::mbar_init(o_ready, 1);
    ptx::mbar_init(bias_full, 1);
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
  const uint32_t tmem_s = tmem, tmem_o = tmem + 128;

  if (warp == 0) {
    if (ptx::elect_one()) {
      ptx::prefetch_tensormap(&tmQ);
      ptx::prefetch_tensormap(&tmK);
      ptx::prefetch_tensormap(&tmV);
      ptx::mbar_expect_tx(q_full, kTileBytes);
      tma_load_5d(q_s, &tmQ, q_full, 0, qt * BQ, h, r, b);
      int k_issued = 0, v_issued = 0, bias_issued = 0;
      bool ok = true;
      if (p.bias_tma) ptx::prefetch_tensormap(&tmBias);
      for (int j = 0; j < nb; ++j) {
        const int s = j & 1;
        if (!ptx::mbar_wait(&k_empty[s], (uint32_t)((j >> 1) & 1) ^ 1u, p.status, kTimeoutStageEmpty)) { ok = false; break; }
        ptx::mbar_expect_tx(&k_full[s], kTileBytes);
        tma_load_5d(k_s + s * kTileBytes, &tmK, &k_full[s], 0, j * BKEY, h, r, b);
        k_issued = j + 1;
        if (p.bias_tma) {
          // the P buffer is free once the second MMA of the previous block has finished reading it
          if (j > 0 && !ptx::mbar_wait(o_ready, (uint32_t)(j - 1) & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
          ptx::mbar_expect_tx(bias_full, 2 * kTileBytes);
          tma_load_4d(p_s, &tmBias, bias_full, j * BKEY, qt * BQ, h, p.bias_sb ? b : 0);
          tma_load_4d(p_s + kTileBytes, &tmBias, bias_full, j * BKEY + 64, qt * BQ, h, p.bias_sb ? b : 0);
          bias_issued = j + 1;
        }
        if (!ptx::mbar_wait(v_empty, (uint32_t)(j & 1) ^ 1u, p.status, kTimeoutStageEmpty)) { ok = false; break; }
        ptx::mbar_expect_tx(v_full, kTileBytes);
        tma_load_5d(v_s, &tmV, v_full, 0, j * BKEY, h, r, b);
        v_issued = j + 1;
      }
      if (!ok) {  // let copies in flight land before shared memory is released
        for (int i = 0; i < (1 << 20) && !ptx::mbar_try_wait(q_full, 0); ++i) {}
        for (int j = k_issued > 2 ? k_issued - 2 : 0; j < k_issued; ++j)
          for (int i = 0; i < (1 << 20) && !ptx::mbar_try_wait(&k_full[j & 1], (uint32_t)(j >> 1) & 1u); ++i) {}
        if (v_issued > 0)
          for (int i = 0; i < (1 << 20) && !ptx::mbar_try_wait(v_full, (uint32_t)(v_issued - 1) & 1u); ++i) {}
        if (bias_issued > 0)
          for (int i = 0; i < (1 << 20) && !ptx::mbar_try_wait(bias_full, (uint32_t)(bias_issued - 1) & 1u); ++i) {}
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      constexpr uint32_t idesc_s = ptx::idesc_bf16_f32(BQ, BKEY);
      constexpr uint32_t idesc_o = idesc_pv(BQ, DN);
      const uint64_t q_desc = ptx::smem_desc_k_sw128(ptx::smem_u32(q_s));
      const uint64_t p_desc = ptx::smem_desc_k_sw128(ptx::smem_u32(p_s));
      const uint64_t v_desc = smem_desc_mn_sw128(ptx::smem_u32(v_s));
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        if (!ptx::mbar_wait(&k_full[s], (uint32_t)(j >> 1) & 1u, p.status, kTimeoutTmaFull)) return false;
        ptx::tc_fence_after();
        const uint64_t k_desc = ptx::smem_desc_k_sw128(ptx::smem_u32(k_s + s * kTileBytes));
#pragma unroll
        for (int kk = 0; kk < DN / 16; ++kk) ptx::umma_bf16(tmem_s, q_desc + 2 * kk, k_desc + 2 * kk, idesc_s, kk != 0);
        ptx::umma_commit(s_ready);
        ptx::umma_commit(&k_empty[s]);
        return true;
      };
      bool ok = ptx::mbar_wait(q_full, 0, p.status, kTimeoutTmaFull);
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < nb; ++j) {
        if (!ptx::mbar_wait(p_ready, (uint32_t)j & 1u, p.status, kTimeoutMmaDone)) break;
        if (!ptx::mbar_wait(v_full, (uint32_t)j & 1u, p.status, kTimeoutTmaFull)) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKEY / 16; ++kk) {
          // P: keys 16 kk .. 16 kk + 15 sit in atom kk / 4 (16 KiB apart) at byte 32 (kk % 4) of each row;
          // V: 16 keys = 2048 bytes further down the tile
          const uint64_t pa = p_desc + (uint64_t)((kk >> 2) * (16384 >> 4) + (kk & 3) * 2);
          ptx::umma_bf16(tmem_o, pa, v_desc + (uint64_t)(kk * (2048 >> 4)), idesc_o, kk != 0);
        }
        ptx::umma_commit(o_ready);
        ptx::umma_commit(v_empty);
        if (j + 1 < nb) ok = issue_s(j + 1);
      }
    }
  } else {
    // two threads per query row: warps 2-5 take keys [0, 64) of each block and output columns [0, DN/2),
    // warps 6-9 the other halves; the pair meets through shared memory for the row maximum and the row sum
    const int qd = warp & 3;                 // tensor-memory lane quarter of this warp
    const int half = (warp - 2) >> 2;
    const int row_in_tile = qd * 32 + lane;
    const int i = qt * BQ + row_in_tile;     // query index
    const bool row_ok = i < p.NQ;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const float* mask_row = p.mask ? p.mask + b * p.mask_sb + r * p.mask_sr : nullptr;
    const uint8_t* bias_row = nullptr;
    if (p.bias && row_ok)
      bias_row = reinterpret_cast<const uint8_t*>(p.bias) +
                 (b * p.bias_sb + h * p.bias_sh + (long long)i * p.bias_si) * (p.bias_is_bf16 ? 2 : 4);
    float m_run = -INFINITY, l_run = 0.f;
    float o_acc[DH];
#pragma unroll
    for (int d = 0; d < DH; ++d) o_acc[d] = 0.f;
    // this row's 128-byte line inside this thread's P atom: 8-row groups are 1024 bytes, chunks XOR-swizzled by the row
    uint8_t* p_row = p_s + half * 16384 + (row_in_tile >> 3) * 1024 + (row_in_tile & 7) * 128;
    const int swz = row_in_tile & 7;
    bool ok = true;
    float v[32];
    for (int j = 0; j < nb && ok; ++j) {
      if (!ptx::mbar_wait(s_ready, (uint32_t)j & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
      ptx::tc_fence_after();
      const int key0 = j * BKEY;
      // additive key term (mask, out-of-range keys) of this block; skipped altogether when every key of the block counts
      __syncwarp();
      bool plain_block = true;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int key = key0 + lane + 32 * t;
        float add = -INFINITY;
        if (key < p.N) add = mask_row ? 1e9f * kLog2e * (mask_row[key] - 1.f) : 0.f;
        key_add[lane + 32 * t] = add;
        plain_block = plain_block && (add == 0.f);
      }
      plain_block = __all_sync(0xffffffffu, plain_block);
      __syncwarp();
      if (p.bias_tma && !ptx::mbar_wait(bias_full, (uint32_t)j & 1u, p.status, kTimeoutTmaFull)) { ok = false; break; }
      // pass 1: logits in base 2 with bias and mask, maximum over this thread's 64 keys; logits parked back in tensor memory
      float m_half = -INFINITY;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * half + cc;
        ptx::tmem_ld_32x32(tmem_s + lane_off + c * 32, v);
        ptx::tmem_ld_wait();
        const int kbase = key0 + c * 32;
        if (p.bias_tma) {  // this row's 64 bytes of the staged tile (out-of-range keys were zero-filled)
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint4 w = *reinterpret_cast<const uint4*>(p_row + (((cc * 4 + g) ^ swz) << 4));
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(&ww[e]);
              v[g * 8 + 2 * e] = v[g * 8 + 2 * e] * p.scale_log2 + __low2float(pr) * kLog2e;
              v[g * 8 + 2 * e + 1] = v[g * 8 + 2 * e + 1] * p.scale_log2 + __high2float(pr) * kLog2e;
            }
          }
        } else if (bias_row == nullptr) {
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = v[t] * p.scale_log2;
        } else if (p.bias_is_bf16 && kbase + 32 <= p.N && ((reinterpret_cast<uintptr_t>(bias_row) + 2 * kbase) & 15) == 0) {
          const uint4* src = reinterpret_cast<const uint4*>(bias_row + 2 * kbase);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint4 w = src[g];
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(&ww[e]);
              v[g * 8 + 2 * e] = v[g * 8 + 2 * e] * p.scale_log2 + __low2float(pr) * kLog2e;
              v[g * 8 + 2 * e + 1] = v[g * 8 + 2 * e + 1] * p.scale_log2 + __high2float(pr) * kLog2e;
            }
          }
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            const int key = kbase + t;
            float add = 0.f;
            if (key < p.N)
              add = p.bias_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias_row)[key])
                                   : reinterpret_cast<const float*>(bias_row)[key];
            v[t] = v[t] * p.scale_log2 + add * kLog2e;
          }
        }
        if (plain_block) {
#pragma unroll
          for (int t = 0; t < 32; ++t) m_half = fmaxf(m_half, v[t]);
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) {
            v[t] += key_add[c * 32 + t];
            m_half = fmaxf(m_half, v[t]);
          }
        }
        tmem_st_32x32(tmem_s + lane_off + c * 32, v);
      }
      // the row maximum needs the other half of the row
      float* x_mine = xchg + ((j & 1) * 2 + half) * 128 + row_in_tile;
      const float* x_other = xchg + ((j & 1) * 2 + (half ^ 1)) * 128 + row_in_tile;
      *x_mine = m_half;
      ptx::mbar_arrive(&x_ready[j & 1]);
      tmem_st_wait();
      if (!ptx::mbar_wait(&x_ready[j & 1], (uint32_t)(j >> 1) & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
      const float m_new = fmaxf(m_run, fmaxf(m_half, *x_other));
      const float alpha = exp2f(m_run - m_new);  // 0 on the first block
      float l_blk = 0.f;
      // pass 2: probabilities, partial row sum, P as bf16 into this thread's 64-key atom of the A-operand tile
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * half + cc;
        ptx::tmem_ld_32x32(tmem_s + lane_off + c * 32, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; ++t) {
          v[t] = exp2f(v[t] - m_new);
          l_blk += v[t];
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = cc * 4 + g;  // 16-byte chunk inside the 128-byte line
          uint4 w;
          w.x = pack2(v[g * 8 + 0], v[g * 8 + 1]);
          w.y = pack2(v[g * 8 + 2], v[g * 8 + 3]);
          w.z = pack2(v[g * 8 + 4], v[g * 8 + 5]);
          w.w = pack2(v[g * 8 + 6], v[g * 8 + 7]);
          *reinterpret_cast<uint4*>(p_row + ((chunk ^ swz) << 4)) = w;
        }
      }
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      ptx::fence_proxy_async();   // P written through the generic proxy, read by the tensor core
      ptx::tc_fence_before();     // and our tensor-memory reads of S are done
      ptx::mbar_arrive(p_ready);
      if (!ptx::mbar_wait(o_ready, (uint32_t)j & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
      ptx::tc_fence_after();
#pragma unroll
      for (int c = 0; c < DH / 8; ++c) {
        float t8[8];
        uint32_t* rr = reinterpret_cast<uint32_t*>(t8);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
            : "=r"(rr[0]), "=r"(rr[1]), "=r"(rr[2]), "=r"(rr[3]), "=r"(rr[4]), "=r"(rr[5]), "=r"(rr[6]), "=r"(rr[7])
            : "r"(tmem_o + lane_off + half * DH + c * 8));
        ptx::tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 8; ++t) o_acc[c * 8 + t] = o_acc[c * 8 + t] * alpha + t8[t];
      }
    }
    // total row sum: one more exchange through the slot of the parity after the last block
    if (ok) {
      const int par = nb & 1;
      xchg[(par * 2 + half) * 128 + row_in_tile] = l_run;
      ptx::mbar_arrive(&x_ready[par]);
      ok = ptx::mbar_wait(&x_ready[par], (uint32_t)(nb >> 1) & 1u, p.status, kTimeoutMmaDone);
      if (ok) l_run += xchg[(par * 2 + (half ^ 1)) * 128 + row_in_tile];
    }
    if (ok && row_ok) {
      const float inv = 1.f / l_run;
      const int d0 = half * DH;
      __nv_bfloat16* dst = p.out + b * p.o_sb + r * p.o_sr + h * p.o_sh + (long long)i * p.o_sn + d0;
      if ((p.D & 7) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int g = 0; g < DH / 8; ++g) {
          if (d0 + g * 8 < p.D) {
            uint4 w;
            w.x = pack2(o_acc[g * 8 + 0] * inv, o_acc[g * 8 + 1] * inv);
            w.y = pack2(o_acc[g * 8 + 2] * inv, o_acc[g * 8 + 3] * inv);
            w.z = pack2(o_acc[g * 8 + 4] * inv, o_acc[g * 8 + 5] * inv);
            w.w = pack2(o_acc[g * 8 + 6] * inv, o_acc[g * 8 + 7] * inv);
            reinterpret_cast<uint4*>(dst)[g] = w;
          }
        }
      } else {
#pragma unroll
        for (int d = 0; d < DH; ++d)
          if (d0 + d < p.D) dst[d] = __float2bfloat16_rn(o_acc[d] * inv);
      }
      if (p.out32) {  // unrounded copy: delta = rowsum(dO o O) of the backward must not see the bf16 rounding of O
        float* d32 = p.out32 + ((((long long)b * p.R + r) * p.H + h) * p.NQ + i) * p.D + d0;
#pragma unroll
        for (int d = 0; d < DH; ++d)
          if (d0 + d < p.D) d32[d] = o_acc[d] * inv;
      }
      if (p.lse && half == 0) {
        // kept apart: for a fully masked row the maximum is about -1.4e9, where adding log2(sum) would round away
        const long long at = (((long long)b * p.R + r) * p.H + h) * p.NQ + i;
        p.lse[at] = m_run;
        p.lse[(long long)p.B * p.R * p.H * p.NQ + at] = log2f(l_run);
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

// Backward helper over one chunk of rows: turns raw q.k and dO.v products into P and dS in place and
// accumulates the bias gradient. One thread per (h, i, j), looping over the rows of the chunk, so the
// sum over rows needs no atomics.
//   s_io  [Rc, H, N, N] bf16: in q.k (unscaled)          out P = exp2(log2e (scale q.k + bias + mask) - row_max - row_log2sum)
//   dp_io [Rc, H, N, N] bf16: in dO.v                    out dS * scale, dS = P (dP - delta)
//   dbias [H, N, N] fp32 += sum_r dS
template <typename BiasT>
__global__ void __launch_bounds__(256) attention_bwd_elem_kernel(
    __nv_bfloat16* __restrict__ s_io, __nv_bfloat16* __restrict__ dp_io, const BiasT* __restrict__ bias, long long bias_sh,
    long long bias_si, const float* __restrict__ mask, long long mask_sr, const float* __restrict__ row_max,
    const float* __restrict__ row_log2sum, const float* __restrict__ delta, float* __restrict__ dbias, int Rc, int H, int N,
    float scale) {
  // one thread per (h, i, pair of keys): N is even (head rows are 16-byte aligned), so a pair never crosses a row
  const long long per_row = (long long)H * N * N;
  const long long e = 2 * ((long long)blockIdx.x * blockDim.x + threadIdx.x);
  if (e >= per_row) return;
  const int j = (int)(e % N);
  const int i = (int)((e / N) % N);
  const int h = (int)(e / ((long long)N * N));
  float bv0 = 0.f, bv1 = 0.f;
  if (bias) {
    const BiasT* bp = bias + h * bias_sh + (long long)i * bias_si + j;
    bv0 = to_float<BiasT>(bp[0]) * kLog2e;
    bv1 = to_float<BiasT>(bp[1]) * kLog2e;
  }
  const float scale_log2 = scale * kLog2e;
  float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 4
  for (int r = 0; r < Rc; ++r) {
    const long long off = r * per_row + e;
    const long long row = ((long long)r * H + h) * N + i;
    float m0 = 0.f, m1 = 0.f;
    if (mask) {
      m0 = 1e9f * kLog2e * (mask[r * mask_sr + j] - 1.f);
      m1 = 1e9f * kLog2e * (mask[r * mask_sr + j + 1] - 1.f);
    }
    const __nv_bfloat162 sv = *reinterpret_cast<const __nv_bfloat162*>(s_io + off);
    const __nv_bfloat162 dv = *reinterpret_cast<const __nv_bfloat162*>(dp_io + off);
    const float mx = row_max[row], ls = row_log2sum[row], dl = delta[row];
    // the same base-2 logit as the forward kernel forms, so masked and unmasked keys line up with its row maximum
    // a logit cannot exceed its row maximum: the clamp only acts on fully masked rows, where the 1e9 offset leaves
    // 128-wide rounding steps and the recomputed logit may land one step above the stored maximum
    const float p0 = exp2f(fminf(((__low2float(sv) * scale_log2 + bv0) + m0) - mx, 0.f) - ls);
    const float p1 = exp2f(fminf(((__high2float(sv) * scale_log2 + bv1) + m1) - mx, 0.f) - ls);
    const float d0 = p0 * (__low2float(dv) - dl), d1 = p1 * (__high2float(dv) - dl);
    acc0 += d0;
    acc1 += d1;
    *reinterpret_cast<__nv_bfloat162*>(s_io + off) = __floats2bfloat162_rn(p0, p1);
    *reinterpret_cast<__nv_bfloat162*>(dp_io + off) = __floats2bfloat162_rn(d0 * scale, d1 * scale);
  }
  if (dbias) {
    float2 cur = *reinterpret_cast<float2*>(dbias + e);
    cur.x += acc0;
    cur.y += acc1;
    *reinterpret_cast<float2*>(dbias + e) = cur;
  }
}

void df3_attention_bwd_elem(Tensor s_io, Tensor dp_io, const c10::optional<Tensor>& bias, const c10::optional<Tensor>& mask,
                            const Tensor& row_max, const Tensor& row_log2sum, const Tensor& delta,
                            const c10::optional<Tensor>& dbias, double scale) {
  TORCH_CHECK(s_io.dim() == 4 && s_io.is_contiguous() && dp_io.is_contiguous() && s_io.sizes() == dp_io.sizes() &&
              s_io.scalar_type() == torch::kBFloat16 && dp_io.scalar_type() == torch::kBFloat16, "attention_bwd_elem: [Rc, H, N, N] bf16");
  const int Rc = (int)s_io.size(0), H = (int)s_io.size(1), N = (int)s_io.size(2);
  for (const Tensor* t : {&row_max, &row_log2sum, &delta})
    TORCH_CHECK(t->is_contiguous() && t->numel() == (int64_t)Rc * H * N && t->scalar_type() == torch::kFloat32,
                "attention_bwd_elem: row_max / row_log2sum / delta [Rc, H, N] fp32");
  c10::cuda::CUDAGuard guard(s_io.device());
  const float* mp = nullptr;
  long long mask_sr = 0;
  Tensor m;
  if (mask.has_value() && mask->defined()) {
    m = mask->to(torch::kFloat32);
    TORCH_CHECK(m.dim() == 2 && m.size(1) == N && (m.size(0) == Rc || m.size(0) == 1), "attention_bwd_elem: mask [Rc or 1, N]");
    if (m.stride(1) != 1) m = m.contiguous();
    mp = m.data_ptr<float>();
    mask_sr = m.size(0) == 1 ? 0 : m.stride(0);
  }
  float* dbp = nullptr;
  if (dbias.has_value() && dbias->defined()) {
    TORCH_CHECK(dbias->is_contiguous() && dbias->scalar_type() == torch::kFloat32 && dbias->numel() == (int64_t)H * N * N, "attention_bwd_elem: dbias [H, N, N] fp32");
    dbp = dbias->data_ptr<float>();
  }
  const long long per_row = (long long)H * N * N;
  TORCH_CHECK(N % 2 == 0, "attention_bwd_elem: an even number of keys is expected");
  const unsigned grid = (unsigned)((per_row / 2 + 255) / 256);
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  auto* sp = reinterpret_cast<__nv_bfloat16*>(s_io.data_ptr());
  auto* dp = reinterpret_cast<__nv_bfloat16*>(dp_io.data_ptr());
  if (bias.has_value() && bias->defined()) {
    Tensor b = *bias;
    TORCH_CHECK(b.dim() == 3 && b.size(0) == H && b.size(1) == N && b.size(2) == N, "attention_bwd_elem: bias [H, N, N]");
    if (b.stride(2) != 1 || (b.scalar_type() != torch::kBFloat16 && b.scalar_type() != torch::kFloat32)) b = b.to(torch::kFloat32).contiguous();
    if (b.scalar_type() == torch::kBFloat16)
      attention_bwd_elem_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(sp, dp, reinterpret_cast<const __nv_bfloat16*>(b.data_ptr()), b.stride(0), b.stride(1), mp, mask_sr, row_max.data_ptr<float>(), row_log2sum.data_ptr<float>(), delta.data_ptr<float>(), dbp, Rc, H, N, (float)scale);
    else
      attention_bwd_elem_kernel<float><<<grid, 256, 0, stream>>>(sp, dp, b.data_ptr<float>(), b.stride(0), b.stride(1), mp, mask_sr, row_max.data_ptr<float>(), row_log2sum.data_ptr<float>(), delta.data_ptr<float>(), dbp, Rc, H, N, (float)scale);
  } else {
    attention_bwd_elem_kernel<float><<<grid, 256, 0, stream>>>(sp, dp, nullptr, 0, 0, mp, mask_sr, row_max.data_ptr<float>(), row_log2sum.data_ptr<float>(), delta.data_ptr<float>(), dbp, Rc, H, N, (float)scale);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// delta[b, r, h, n] = sum_d out * d_out, straight from the (strided) bf16 tensors.
__global__ void attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                       long long o_sb, long long o_sr, long long o_sh, long long o_sn, long long g_sb, long long g_sr,
                                       long long g_sh, long long g_sn, int R, int H, int N, int D, long long total) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int n = (int)(e % N);
  const int h = (int)((e / N) % H);
  const int r = (int)((e / ((long long)N * H)) % R);
  const long long b = e / ((long long)N * H * R);
  const __nv_bfloat16* po = o + b * o_sb + r * o_sr + h * o_sh + (long long)n * o_sn;
  const __nv_bfloat16* pg = d_o + b * g_sb + r * g_sr + h * g_sh + (long long)n * g_sn;
  float acc = 0.f;
  if ((D & 7) == 0 && (reinterpret_cast<uintptr_t>(po) & 15) == 0 && (reinterpret_cast<uintptr_t>(pg) & 15) == 0) {
    for (int d = 0; d < D; d += 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(po + d), c = *reinterpret_cast<const uint4*>(pg + d);
      const uint32_t aa[4] = {a.x, a.y, a.z, a.w}, cc[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&aa[k]), y = *reinterpret_cast<const __nv_bfloat162*>(&cc[k]);
        acc += __low2float(x) * __low2float(y) + __high2float(x) * __high2float(y);
      }
    }
  } else {
    for (int d = 0; d < D; ++d) acc += __bfloat162float(po[d]) * __bfloat162float(pg[d]);
  }
  delta[e] = acc;
}

// Whole backward of the attention op: row chunks sized for L2, five library GEMMs and one fused
// elementwise kernel per chunk. Returns dq, dk, dv as contiguous [B, R, H, N, D] and dbias [Bb, H, N, N] fp32.
std::tuple<Tensor, Tensor, Tensor, Tensor> df3_attention_bwd(const Tensor& q, const Tensor& k, const Tensor& v,
                                                             const Tensor& out, const Tensor& d_out,
                                                             const c10::optional<Tensor>& bias,
                                                             const c10::optional<Tensor>& mask, const Tensor& lse,
                                                             double scale, bool want_dbias, int64_t chunk_bytes) {
  const int64_t B = q.size(0), R = q.size(1), H = q.size(2), N = q.size(3), D = q.size(4);
  if (chunk_bytes >= 0 && attention_bwd_fused_supported(N, D))  // a negative chunk size asks for the chunked form
    return attention_bwd_fused(q, k, v, out, d_out, bias, mask, lse, scale, want_dbias, c10::nullopt, c10::nullopt, c10::nullopt);
  if (chunk_bytes < 0) chunk_bytes = -chunk_bytes;
  c10::cuda::CUDAGuard guard(q.device());
  auto bf = q.options();
  Tensor qc = q.contiguous(), kc = k.contiguous(), vc = v.contiguous();
  Tensor doc = d_out.to(torch::kBFloat16).contiguous();
  Tensor delta = torch::empty({B, R, H, N}, bf.dtype(torch::kFloat32));
  if (out.scalar_type() == torch::kBFloat16 && out.stride(4) == 1 && delta.numel() > 0) {
    const long long total = delta.numel();
    attention_delta_kernel<<<(unsigned)((total + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(out.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(doc.data_ptr()),
        delta.data_ptr<float>(), out.stride(0), out.stride(1), out.stride(2), out.stride(3), doc.stride(0), doc.stride(1),
        doc.stride(2), doc.stride(3), (int)R, (int)H, (int)N, (int)D, total);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else {
    delta = (doc.to(torch::kFloat32) * out.to(torch::kFloat32)).sum(-1);
  }
  Tensor dq = torch::empty({B, R, H, N, D}, bf), dk = torch::empty({B, R, H, N, D}, bf), dv = torch::empty({B, R, H, N, D}, bf);
  const bool has_bias = bias.has_value() && bias->defined();
  const bool has_mask = mask.has_value() && mask->defined();
  Tensor dbias;
  if (want_dbias && has_bias) dbias = torch::zeros({bias->size(0), H, N, N}, bf.dtype(torch::kFloat32));
  int64_t rc = chunk_bytes / std::max<int64_t>(1, H * N * N * 2);
  rc = std::max<int64_t>(1, std::min<int64_t>(R, rc));
  Tensor s = torch::empty({rc, H, N, N}, bf), dp = torch::empty({rc, H, N, N}, bf);
  for (int64_t b = 0; b < B; ++b) {
    c10::optional<Tensor> bb, db;
    if (has_bias) bb = bias->select(0, bias->size(0) > 1 ? b : 0);
    if (dbias.defined()) db = dbias.select(0, dbias.size(0) > 1 ? b : 0);
    for (int64_t r0 = 0; r0 < R; r0 += rc) {
      const int64_t n = std::min(rc, R - r0);
      Tensor q3 = qc[b].narrow(0, r0, n).reshape({n * H, N, D});
      Tensor k3 = kc[b].narrow(0, r0, n).reshape({n * H, N, D});
      Tensor v3 = vc[b].narrow(0, r0, n).reshape({n * H, N, D});
      Tensor o3 = doc[b].narrow(0, r0, n).reshape({n * H, N, D});
      Tensor s3 = s.narrow(0, 0, n).view({n * H, N, N});
      Tensor p3 = dp.narrow(0, 0, n).view({n * H, N, N});
      df3_matmul_any(q3, k3, false, true, false, 1, s3);   // S = Q K^T
      df3_matmul_any(o3, v3, false, true, false, 1, p3);   // dP = dO V^T
      c10::optional<Tensor> mm;
      if (has_mask) {
        Tensor mb = mask->select(0, mask->size(0) > 1 ? b : 0);
        mm = mb.size(0) > 1 ? mb.narrow(0, r0, n) : mb;
      }
      df3_attention_bwd_elem(s.narrow(0, 0, n), dp.narrow(0, 0, n), bb, mm, lse[0][b].narrow(0, r0, n).contiguous(),
                             lse[1][b].narrow(0, r0, n).contiguous(), delta[b].narrow(0, r0, n).contiguous(), db, scale);
      Tensor dv3 = dv[b].narrow(0, r0, n).view({n * H, N, D});
      Tensor dq3 = dq[b].narrow(0, r0, n).view({n * H, N, D});
      Tensor dk3 = dk[b].narrow(0, r0, n).view({n * H, N, D});
      df3_matmul_any(s3, o3, true, false, false, 1, dv3);  // dV = P^T dO
      df3_matmul_any(p3, k3, false, false, false, 1, dq3); // dQ = dS K
      df3_matmul_any(p3, q3, true, false, false, 1, dk3);  // dK = dS^T Q
    }
  }
  if (!dbias.defined()) dbias = torch::empty({0}, bf.dtype(torch::kFloat32));
  return {dq, dk, dv, dbias};
}

std::tuple<Tensor, Tensor, Tensor> attention_fwd_impl(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in,
                                                      const c10::optional<Tensor>& bias_in, const c10::optional<Tensor>& mask_in,
                                                      double scale, bool want_lse, bool want_out32) {
  TORCH_CHECK(q_in.dim() == 5 && k_in.dim() == 5 && v_in.sizes() == k_in.sizes(), "attention: [B, R, H, N, D] q, k, v");
  for (int d : {0, 1, 2, 4}) TORCH_CHECK(q_in.size(d) == k_in.size(d), "attention: q and k differ outside the token axis");
  TORCH_CHECK(q_in.is_cuda() && q_in.scalar_type() == torch::kBFloat16 && k_in.scalar_type() == torch::kBFloat16 &&
              v_in.scalar_type() == torch::kBFloat16, "attention: bf16 CUDA tensors");
  const int64_t B = q_in.size(0), R = q_in.size(1), H = q_in.size(2), NQ = q_in.size(3), N = k_in.size(3), D = q_in.size(4);
  TORCH_CHECK(D % 8 == 0 && D <= 64, "attention: head width must be a multiple of 8, at most 64");
  c10::cuda::CUDAGuard guard(q_in.device());
  Tensor q = strides_ok(q_in) ? q_in : q_in.contiguous();
  Tensor k = strides_ok(k_in) ? k_in : k_in.contiguous();
  Tensor v = strides_ok(v_in) ? v_in : v_in.contiguous();
  // the output takes q's dimension order in memory (q is usually a non-dense view of a packed projection, for which
  // empty_like would fall back to the logical order and force a transposing copy on the way back to [.., tokens, H * D])
  Tensor out;
  {
    std::vector<int64_t> order = {0, 1, 2, 3, 4};
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return q.stride(a) > q.stride(b); });
    std::vector<int64_t> sizes_perm(5), inverse(5);
    for (int i = 0; i < 5; ++i) {
      sizes_perm[i] = q.size(order[i]);
      inverse[order[i]] = i;
    }
    out = torch::empty(sizes_perm, q.options()).permute(inverse);
    if (out.stride(4) != 1) out = torch::empty(q.sizes(), q.options());
  }
  Tensor lse = torch::empty({want_lse ? 2 : 0, B, R, H, NQ}, q.options().dtype(torch::kFloat32));
  Tensor out32 = want_out32 ? torch::empty({B, R, H, NQ, D}, q.options().dtype(torch::kFloat32)) : torch::empty({0}, q.options().dtype(torch::kFloat32));
  if (out.numel() == 0 || N == 0) return {out.zero_(), lse, out32};

  AttnParams p{};
  p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.lse = want_lse ? lse.data_ptr<float>() : nullptr;
  p.out32 = want_out32 ? out32.data_ptr<float>() : nullptr;
  p.o_sb = out.stride(0); p.o_sr = out.stride(1); p.o_sh = out.stride(2); p.o_sn = out.stride(3);
  Tensor bias, mask;
  if (bias_in.has_value() && bias_in->defined()) {
    bias = *bias_in;
    TORCH_CHECK(bias.dim() == 4 && bias.size(1) == H && bias.size(2) == NQ && bias.size(3) == N &&
                (bias.size(0) == B || bias.size(0) == 1), "attention: bias [B or 1, H, queries, keys]");
    if (bias.scalar_type() != torch::kBFloat16 && bias.scalar_type() != torch::kFloat32) bias = bias.to(torch::kFloat32);
    if (bias.stride(3) != 1) bias = bias.contiguous();
    p.bias = bias.data_ptr();
    p.bias_is_bf16 = bias.scalar_type() == torch::kBFloat16;
    p.bias_sb = bias.size(0) == 1 ? 0 : bias.stride(0);
    p.bias_sh = bias.stride(1);
    p.bias_si = bias.stride(2);
  }
  if (mask_in.has_value() && mask_in->defined()) {
    mask = mask_in->to(torch::kFloat32);
    TORCH_CHECK(mask.dim() == 3 && mask.size(2) == N && (mask.size(0) == B || mask.size(0) == 1) &&
                (mask.size(1) == R || mask.size(1) == 1), "attention: key mask [B or 1, R or 1, N]");
    if (mask.stride(2) != 1) mask = mask.contiguous();
    p.mask = mask.data_ptr<float>();
    p.mask_sb = mask.size(0) == 1 ? 0 : mask.stride(0);
    p.mask_sr = mask.size(1) == 1 ? 0 : mask.stride(1);
  }
  Tensor status = status_word(q.device().index());
  p.status = status.data_ptr<int>();
  p.B = (int)B; p.R = (int)R; p.H = (int)H; p.N = (int)N; p.NQ = (int)NQ; p.D = (int)D;
  p.q_tiles = (int)((NQ + BQ - 1) / BQ);
  p.scale_log2 = (float)scale * kLog2e;
  const CUtensorMap tq = qkv_map(q), tk = qkv_map(k), tv = qkv_map(v);
  CUtensorMap tbias = tq;  // placeholder when the bias is not staged by TMA
  if (p.bias && p.bias_is_bf16 && N % 8 == 0 && bias.stride(3) == 1 && bias.stride(2) % 8 == 0 && bias.stride(1) % 8 == 0 &&
      (bias.size(0) == 1 || bias.stride(0) % 8 == 0) && reinterpret_cast<uintptr_t>(bias.data_ptr()) % 16 == 0) {
    const int64_t dims[4] = {N, NQ, H, bias.size(0)};
    const int64_t strides[4] = {1, bias.stride(2), bias.stride(1), bias.size(0) > 1 ? bias.stride(0) : H * bias.stride(1)};
    const int box[4] = {64, 128, 1, 1};
    tbias = make_map_nd(bias.data_ptr(), 4, dims, strides, box);
    p.bias_tma = 1;
  }
  const long long ctas = (long long)B * R * H * p.q_tiles;
  TORCH_CHECK(ctas < (1ll << 31), "attention: grid too large");
  const size_t smem = 6 * kTileBytes + 128 + 512 + 2048;
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const int dn = (int)((D + 15) / 16 * 16);
#define DF3_ATTN(DN_)                                                                                               \
  do {                                                                                                              \
    static bool attr = false;                                                                                       \
    if (!attr) {                                                                                                    \
      C10_CUDA_CHECK(cudaFuncSetAttribute(attention_fwd_kernel<DN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
      attr = true;                                                                                                  \
    }                                                                                                               \
    attention_fwd_kernel<DN_><<<(unsigned)ctas, kThreads, smem, stream>>>(tq, tk, tv, tbias, p);                           \
  } while (0)
  if (dn == 16) DF3_ATTN(16); else if (dn == 32) DF3_ATTN(32); else if (dn == 48) DF3_ATTN(48); else DF3_ATTN(64);
#undef DF3_ATTN
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {out, lse, out32};
}

std::tuple<Tensor, Tensor> df3_attention_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& bias,
                                             const c10::optional<Tensor>& mask, double scale, bool want_lse) {
  auto r = attention_fwd_impl(q, k, v, bias, mask, scale, want_lse, false);
  return {std::get<0>(r), std::get<1>(r)};
}

// Training forward: also returns the output before its rounding to bf16 ([B, R, H, N, D] fp32), which the backward
// takes as `out` so that delta = rowsum(dO o O) keeps the cancellation with dP (docs/optimizations.md:409-493 of the
// reference names the bf16 O store as the first of the roundings that destroy dS at a saturated row).
std::tuple<Tensor, Tensor, Tensor> df3_attention_fwd_train(const Tensor& q, const Tensor& k, const Tensor& v,
                                                           const c10::optional<Tensor>& bias, const c10::optional<Tensor>& mask,
                                                           double scale) {
  return attention_fwd_impl(q, k, v, bias, mask, scale, true, true);
}

}  // namespace
}  // namespace df3

void df3_register_attention(torch::Library& m) {
  m.def("attention_fwd(Tensor q, Tensor k, Tensor v, Tensor? bias, Tensor? key_mask, float scale, bool want_lse) -> (Tensor, Tensor)",
        &df3::df3_attention_fwd);
  m.def("attention_fwd_train(Tensor q, Tensor k, Tensor v, Tensor? bias, Tensor? key_mask, float scale) -> (Tensor, Tensor, Tensor)",
        &df3::df3_attention_fwd_train);
  m.def("attention_bwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor d_out, Tensor? bias, Tensor? key_mask, Tensor lse, "
        "float scale, bool want_dbias, int chunk_bytes) -> (Tensor, Tensor, Tensor, Tensor)",
        &df3::df3_attention_bwd);
  m.def("attention_bwd_into(Tensor q, Tensor k, Tensor v, Tensor out, Tensor d_out, Tensor? bias, Tensor? key_mask, Tensor lse, "
        "float scale, bool want_dbias, Tensor(a!) dq, Tensor(b!) dk, Tensor(c!) dv) -> Tensor",
        [](const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& d_out, const c10::optional<Tensor>& bias,
           const c10::optional<Tensor>& mask, const Tensor& lse, double scale, bool want_dbias, Tensor dq, Tensor dk, Tensor dv) {
          return std::get<3>(df3::attention_bwd_fused(q, k, v, out, d_out, bias, mask, lse, scale, want_dbias, dq, dk, dv));
        });
  m.def("attention_bwd_fused_supported(int n, int d) -> bool", [](int64_t n, int64_t d) { return df3::attention_bwd_fused_supported(n, d); });
  m.def("attention_bwd_elem(Tensor(a!) s_io, Tensor(b!) dp_io, Tensor? bias, Tensor? mask, Tensor row_max, Tensor row_log2sum, Tensor delta, Tensor(c!)? dbias, float scale) -> ()",
        &df3::df3_attention_bwd_elem);
}
