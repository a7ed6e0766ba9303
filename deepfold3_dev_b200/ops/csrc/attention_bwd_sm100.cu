// Pair-biased softmax attention, backward, for sm_100a: one kernel forms dQ, dK, dV and the logit
// gradient of one (batch, row, head) entirely on chip.
//
//   S  = Q K^T, dP = dO V^T                      recomputed on the tensor cores from the bf16 operands, fp32 in tensor memory
//   P  = exp2(scale log2e S + log2e bias + key term - row_max - row_log2sum)          (row statistics saved by the forward)
//   dS = P (dP - delta),  delta = rowsum(dO o O)
//   dV = P^T dO,  dK = scale dS^T Q,  dQ = scale dS K,  dbias = sum over rows r of dS
//
// The logits never leave fp32 between the accumulator and the exponential (the reference keeps the same contract:
// model/triton/evo_attention.py:602-1195, docs/optimizations.md:409-493); only the P and dS tiles that feed the
// second-stage MMAs are rounded to bf16.
//
// One CTA owns one (b, r, h). Keys are walked in blocks of 128 (outer loop), queries in tiles of 128 (inner loop), and
// each (query tile, key block) pair is processed as two 64-key halves so that the tensor cores compute the next half
// while the softmax warps work on the current one:
//   warp 0       TMA producer: K/V blocks (two stages) and Q/dO tiles (two stages), 5-D tensor maps, 128-byte swizzle
//   warp 1       tcgen05.mma issuer; owns the tensor-memory allocation (512 columns):
//                  [0, 256)   two stages of { S half 128x64, dP half 128x64 }
//                  [256, ..)  dQ accumulators of every query tile, then dK and dV of the current key block
//   warps 2-17   softmax warps, four threads per query row, each with 16 of the 64 keys of the half:
//                  S and dP out of tensor memory, P and dS in registers, both written as bf16 into 128-byte swizzled
//                  shared-memory tiles [query][key] that the second-stage MMAs read K-major (dQ += dS K) and MN-major
//                  (dV += P^T dO, dK += dS^T Q); dS also goes to a global scratch [B, R, H, N, N] for the bias gradient
// The bias gradient is the sum of that scratch over r, done by a second, order-fixed kernel: no atomics, run-to-run
// bitwise reproducible. The scratch is fp16 (saturating): at the same traffic as bf16 each term carries three more
// mantissa bits into the fp32 sum, and a logit gradient beyond the fp16 range would be a diverged step anyway.
// Every wait is bounded and reports through the status word.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_fp16.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "sm100_ptx.cuh"

using torch::Tensor;

namespace df3 {
Tensor status_word(int device);          // gemm_sm100.cu
CUtensorMap qkv_map(const Tensor& t);     // attention_sm100.cu
bool strides_ok(const Tensor& t);         // attention_sm100.cu

namespace {

constexpr int kTile = 128;             // query tile / key block
constexpr int kTileBytes = 128 * 128;  // 128 rows x 128 bytes
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kSoftmaxWarps = 16;
constexpr int kSoftmaxThreads = kSoftmaxWarps * 32;
constexpr int kBwdThreads = kSoftmaxThreads + 64;
constexpr int COLS = 64 / (kSoftmaxWarps / 4);  // keys of one half-step per thread
static_assert(COLS == 16, "the tensor-memory loads below are written for 16 columns per thread");

struct BwdParams {
  const float* lse;      // [2, B, R, H, N]: row maximum, log2 of the row sum (base 2)
  const float* delta;    // [B, R, H, N]
  const void* bias;      // [Bb, H, N, N] or null
  const float* mask;     // [B or 1, R or 1, N] or null
  __nv_bfloat16* dq;     // outputs, strided [B, R, H, N, D]
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  __half* ds;            // scratch [B, R, H, N, N] (fp16) or null
  int* status;
  long long dq_s[4], dk_s[4], dv_s[4];   // element strides of b, r, h, n (d is contiguous)
  long long bias_sb, bias_sh, bias_si;
  long long mask_sb, mask_sr;
  int B, R, H, N, D;
  int T;                 // tiles of 128 along N
  int bias_is_bf16;
  int vec_ok;            // N % 8 == 0 and 16-byte aligned bias / scratch rows: 16-byte accesses
  float scale, scale_log2;
};

// two fp32 -> packed fp16 pair, values beyond the fp16 range clamped to the largest finite one
__device__ __forceinline__ uint32_t pack2_f16_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ void store_chunk8(__nv_bfloat16* dst, const float* v, float mul, bool vec) {
  if (vec) {
    uint4 w;
    w.x = ptx::pack2_bf16(v[0] * mul, v[1] * mul);
    w.y = ptx::pack2_bf16(v[2] * mul, v[3] * mul);
    w.z = ptx::pack2_bf16(v[4] * mul, v[5] * mul);
    w.w = ptx::pack2_bf16(v[6] * mul, v[7] * mul);
    *reinterpret_cast<uint4*>(dst) = w;
  } else {
#pragma unroll
    for (int t = 0; t < 8; ++t) dst[t] = __float2bfloat16_rn(v[t] * mul);
  }
}

template <int DN>  // head width rounded up to 16
__global__ void __launch_bounds__(kBwdThreads, 1) attention_bwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                       const __grid_constant__ CUtensorMap tmK,
                                                                       const __grid_constant__ CUtensorMap tmV,
                                                                       const __grid_constant__ CUtensorMap tmDO, BwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // tiles: Q[2] dO[2] K[2] V[2] P(2 atoms) dS(2 atoms)
  uint8_t* q_s = smem;
  uint8_t* do_s = smem + 2 * kTileBytes;
  uint8_t* k_s = smem + 4 * kTileBytes;
  uint8_t* v_s = smem + 6 * kTileBytes;
  uint8_t* p_s = smem + 8 * kTileBytes;
  uint8_t* ds_s = smem + 10 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 12 * kTileBytes);
  uint64_t* kv_full = bars;         // [2]
  uint64_t* kv_empty = bars + 2;    // [2]
  uint64_t* q_full = bars + 4;      // [2]
  uint64_t* q_empty = bars + 6;     // [2]
  uint64_t* sdp_ready = bars + 8;   // [2]
  uint64_t* sdp_free = bars + 10;   // [2]
  // [2], by step parity. One barrier would not do: a softmax thread that is a whole half-step ahead of a slow one would
  // arrive a second time into the phase the slow thread has not reached yet, and the MMA warp would read an incomplete tile.
  // With two, the fast thread's next arrival goes to the other barrier, and it cannot reach the step after that before
  // the MMA warp has seen this one complete (that step's S and dP are only issued afterwards).
  uint64_t* pds_ready = bars + 12;
  uint64_t* pds_free = bars + 14;
  uint64_t* kv_acc_ready = bars + 15;
  uint64_t* kv_acc_free = bars + 16;
  uint64_t* dq_ready = bars + 17;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  float* key_add = reinterpret_cast<float*>(bars + 20);  // [T * 128]: additive key term in base 2, -inf beyond N

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int idx = blockIdx.x;
  const int h = idx % p.H; idx /= p.H;
  const int r = idx % p.R;
  const int b = idx / p.R;
  const int T = p.T;
  const int steps = 2 * T * T;

  if ((ptx::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, kOk, kBadShape);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(&kv_full[s], 1);
      ptx::mbar_init(&kv_empty[s], 1);
      ptx::mbar_init(&q_full[s], 1);
      ptx::mbar_init(&q_empty[s], 1);
      ptx::mbar_init(&sdp_ready[s], 1);
      ptx::mbar_init(&sdp_free[s], kSoftmaxThreads);
    }
    ptx::mbar_init(&pds_ready[0], kSoftmaxThreads);
    ptx::mbar_init(&pds_ready[1], kSoftmaxThreads);
    ptx::mbar_init(pds_free, 1);
    ptx::mbar_init(kv_acc_ready, 1);
    ptx::mbar_init(kv_acc_free, kSoftmaxThreads);
    ptx::mbar_init(dq_ready, 1);
    ptx::fence_barrier_init();
  }
  {
    const float* mask_row = p.mask ? p.mask + b * p.mask_sb + r * p.mask_sr : nullptr;
    for (int t = threadIdx.x; t < T * kTile; t += kBwdThreads) {
      float add = -INFINITY;
      if (t < p.N) add = mask_row ? 1e9f * kLog2e * (mask_row[t] - 1.f) : 0.f;
      key_add[t] = add;
    }
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_dq = tmem + 256;
  const uint32_t tmem_dk = tmem_dq + T * DN;
  const uint32_t tmem_dv = tmem_dk + DN;

  if (warp == 0) {
    if (ptx::elect_one()) {
      ptx::prefetch_tensormap(&tmQ);
      ptx::prefetch_tensormap(&tmK);
      ptx::prefetch_tensormap(&tmV);
      ptx::prefetch_tensormap(&tmDO);
      bool ok = true;
      int kv_issued = 0, q_issued = 0;
      for (int j = 0; j < T && ok; ++j) {
        const int kvs = j & 1;
        if (!ptx::mbar_wait(&kv_empty[kvs], (uint32_t)((j >> 1) & 1) ^ 1u, p.status, kTimeoutStageEmpty)) { ok = false; break; }
        ptx::mbar_expect_tx(&kv_full[kvs], 2 * kTileBytes);
        ptx::tma_load_5d(k_s + kvs * kTileBytes, &tmK, &kv_full[kvs], 0, j * kTile, h, r, b);
        ptx::tma_load_5d(v_s + kvs * kTileBytes, &tmV, &kv_full[kvs], 0, j * kTile, h, r, b);
        kv_issued = j + 1;
        for (int i = 0; i < T; ++i) {
          const int n = j * T + i, qs = n & 1;
          if (!ptx::mbar_wait(&q_empty[qs], (uint32_t)((n >> 1) & 1) ^ 1u, p.status, kTimeoutStageEmpty)) { ok = false; break; }
          ptx::mbar_expect_tx(&q_full[qs], 2 * kTileBytes);
          ptx::tma_load_5d(q_s + qs * kTileBytes, &tmQ, &q_full[qs], 0, i * kTile, h, r, b);
          ptx::tma_load_5d(do_s + qs * kTileBytes, &tmDO, &q_full[qs], 0, i * kTile, h, r, b);
          q_issued = n + 1;
        }
      }
      if (!ok) {  // let copies in flight land before shared memory is released
        for (int j = kv_issued > 2 ? kv_issued - 2 : 0; j < kv_issued; ++j) ptx::mbar_wait_quiet(&kv_full[j & 1], (uint32_t)(j >> 1) & 1u);
        for (int n = q_issued > 2 ? q_issued - 2 : 0; n < q_issued; ++n) ptx::mbar_wait_quiet(&q_full[n & 1], (uint32_t)(n >> 1) & 1u);
      }
    }
  } else if (warp == 1) {
    if (ptx::elect_one()) {
      constexpr uint32_t idesc_s = ptx::idesc_bf16_f32(kTile, 64);                                  // A, B K-major
      constexpr uint32_t idesc_q = ptx::idesc_bf16_f32(kTile, DN) | ptx::kIdescBMnMajor;             // A K-major, B MN-major
      constexpr uint32_t idesc_kv = ptx::idesc_bf16_f32(kTile, DN) | ptx::kIdescAMnMajor | ptx::kIdescBMnMajor;
      const uint32_t q_a = ptx::smem_u32(q_s), do_a = ptx::smem_u32(do_s), k_a = ptx::smem_u32(k_s), v_a = ptx::smem_u32(v_s);
      const uint32_t p_a = ptx::smem_u32(p_s), ds_a = ptx::smem_u32(ds_s);
      bool ok = true;
      // first-stage MMAs of step s: S half and dP half into stage s & 1
      auto issue_sdp = [&](int s) -> bool {
        const int hh = s & 1, pair = s >> 1, j = pair / T, i = pair - j * T;
        const int kvs = j & 1, qs = pair & 1;
        if (hh == 0) {
          if (i == 0 && !ptx::mbar_wait(&kv_full[kvs], (uint32_t)(j >> 1) & 1u, p.status, kTimeoutTmaFull)) return false;
          if (!ptx::mbar_wait(&q_full[qs], (uint32_t)(pair >> 1) & 1u, p.status, kTimeoutTmaFull)) return false;
        }
        if (!ptx::mbar_wait(&sdp_free[hh], (uint32_t)((s >> 1) & 1) ^ 1u, p.status, kTimeoutStageEmpty)) return false;
        ptx::tc_fence_after();
        const uint64_t qd = ptx::smem_desc_k_sw128(q_a + qs * kTileBytes);
        const uint64_t dod = ptx::smem_desc_k_sw128(do_a + qs * kTileBytes);
        const uint64_t kd = ptx::smem_desc_k_sw128(k_a + kvs * kTileBytes + hh * 8192);   // keys 64 hh .. 64 hh + 63
        const uint64_t vd = ptx::smem_desc_k_sw128(v_a + kvs * kTileBytes + hh * 8192);
        const uint32_t t_s = tmem + hh * 128, t_dp = t_s + 64;
#pragma unroll
        for (int kk = 0; kk < DN / 16; ++kk) ptx::umma_bf16(t_s, qd + 2 * kk, kd + 2 * kk, idesc_s, kk != 0);
#pragma unroll
        for (int kk = 0; kk < DN / 16; ++kk) ptx::umma_bf16(t_dp, dod + 2 * kk, vd + 2 * kk, idesc_s, kk != 0);
        ptx::umma_commit(&sdp_ready[hh]);
        return true;
      };
      ok = issue_sdp(0);
      for (int s = 0; s < steps && ok; ++s) {
        if (s + 1 < steps && !issue_sdp(s + 1)) { ok = false; break; }
        const int hh = s & 1, pair = s >> 1, j = pair / T, i = pair - j * T;
        const int kvs = j & 1, qs = pair & 1;
        if (!ptx::mbar_wait(&pds_ready[hh], (uint32_t)(s >> 1) & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
        ptx::tc_fence_after();
        // dQ_i += dS[:, 64 hh ..] K[64 hh .., :]
        {
          const uint64_t a = ptx::smem_desc_k_sw128(ds_a + hh * 16384);
          const uint64_t bdesc = ptx::smem_desc_mn_sw128(k_a + kvs * kTileBytes + hh * 8192);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            ptx::umma_bf16(tmem_dq + i * DN, a + 2 * kk, bdesc + (uint64_t)(kk * (2048 >> 4)), idesc_q, !(j == 0 && hh == 0 && kk == 0));
        }
        if (hh == 1) {
          if (i == 0 && j > 0 && !ptx::mbar_wait(kv_acc_free, (uint32_t)(j - 1) & 1u, p.status, kTimeoutStageEmpty)) { ok = false; break; }
          ptx::tc_fence_after();
          // dV_j += P^T dO_i, dK_j += dS^T Q_i: A is the [query][key] tile read MN-major (two 64-key blocks 16 KiB apart)
          const uint64_t pa = ptx::smem_desc_mn_sw128(p_a, 16384), dsa = ptx::smem_desc_mn_sw128(ds_a, 16384);
          const uint64_t dob = ptx::smem_desc_mn_sw128(do_a + qs * kTileBytes), qb = ptx::smem_desc_mn_sw128(q_a + qs * kTileBytes);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t adv = (uint64_t)(kk * (2048 >> 4));  // 16 queries further down both tiles
            ptx::umma_bf16(tmem_dv, pa + adv, dob + adv, idesc_kv, !(i == 0 && kk == 0));
          }
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint64_t adv = (uint64_t)(kk * (2048 >> 4));
            ptx::umma_bf16(tmem_dk, dsa + adv, qb + adv, idesc_kv, !(i == 0 && kk == 0));
          }
          ptx::umma_commit(pds_free);
          ptx::umma_commit(&q_empty[qs]);
          if (i == T - 1) {
            ptx::umma_commit(&kv_empty[kvs]);
            ptx::umma_commit(kv_acc_ready);
          }
        }
      }
      if (ok) ptx::umma_commit(dq_ready);
    }
  } else {
    const int w = warp - 2;
    const int qd = warp & 3;            // tensor-memory lane quarter of this warp
    const int sub = w >> 2;             // which COLS keys of a 64-key half
    const int row_in_tile = qd * 32 + lane;
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const long long brh = ((long long)b * p.R + r) * p.H + h;
    const float* row_max = p.lse + brh * p.N;
    const float* row_l2s = p.lse + (long long)p.B * p.R * p.H * p.N + brh * p.N;
    const float* delta = p.delta + brh * p.N;
    const int swz = row_in_tile & 7;
    uint8_t* p_row = p_s + (row_in_tile >> 3) * 1024 + (row_in_tile & 7) * 128;
    uint8_t* ds_row = ds_s + (row_in_tile >> 3) * 1024 + (row_in_tile & 7) * 128;
    bool ok = true;
    float mx = 0.f, ls = INFINITY, dl = 0.f;
    const uint8_t* bias_row = nullptr;
    __half* ds_out = nullptr;
    bool row_ok = false;
    float s_v[COLS], dp_v[COLS];
    for (int s = 0; s < steps && ok; ++s) {
      const int hh = s & 1, pair = s >> 1, j = pair / T, i = pair - j * T;
      if (hh == 0) {
        const int qi = i * kTile + row_in_tile;
        row_ok = qi < p.N;
        mx = row_ok ? row_max[qi] : 0.f;
        ls = row_ok ? row_l2s[qi] : INFINITY;   // rows beyond N get P = 0
        dl = row_ok ? delta[qi] : 0.f;
        bias_row = (p.bias && row_ok) ? reinterpret_cast<const uint8_t*>(p.bias) +
                                            ((p.bias_sb ? b * p.bias_sb : 0) + h * p.bias_sh + (long long)qi * p.bias_si) * (p.bias_is_bf16 ? 2 : 4)
                                      : nullptr;
        ds_out = (p.ds && row_ok) ? p.ds + (brh * p.N + qi) * p.N : nullptr;
      }
      if (!ptx::mbar_wait(&sdp_ready[hh], (uint32_t)(s >> 1) & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
      ptx::tc_fence_after();
      ptx::tmem_ld_32x16(tmem + lane_off + hh * 128 + sub * COLS, s_v);
      ptx::tmem_ld_32x16(tmem + lane_off + hh * 128 + 64 + sub * COLS, dp_v);
      ptx::tmem_ld_wait();
      ptx::tc_fence_before();
      ptx::mbar_arrive(&sdp_free[hh]);
      const int key0 = j * kTile + hh * 64 + sub * COLS;
      // base-2 logits exactly as the forward forms them: acc * scale_log2 + bias * log2e, then the key term
      if (bias_row == nullptr) {
#pragma unroll
        for (int t = 0; t < COLS; ++t) s_v[t] = s_v[t] * p.scale_log2;
      } else if (p.bias_is_bf16 && p.vec_ok && key0 + COLS <= p.N) {
        const uint4* src = reinterpret_cast<const uint4*>(bias_row + 2 * key0);
#pragma unroll
        for (int g = 0; g < COLS / 8; ++g) {
          const uint4 wv = src[g];
          const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(&ww[e]);
            s_v[g * 8 + 2 * e] = s_v[g * 8 + 2 * e] * p.scale_log2 + __low2float(pr) * kLog2e;
            s_v[g * 8 + 2 * e + 1] = s_v[g * 8 + 2 * e + 1] * p.scale_log2 + __high2float(pr) * kLog2e;
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < COLS; ++t) {
          const int key = key0 + t;
          float add = 0.f;
          if (key < p.N)
            add = p.bias_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias_row)[key])
                                 : reinterpret_cast<const float*>(bias_row)[key];
          s_v[t] = s_v[t] * p.scale_log2 + add * kLog2e;
        }
      }
      // P and dS; a logit cannot exceed its row maximum (the clamp only acts on fully masked rows, where the 1e9
      // offset leaves coarse rounding steps)
#pragma unroll
      for (int t = 0; t < COLS; ++t) {
        const float pv = exp2f(fminf((s_v[t] + key_add[key0 + t]) - mx, 0.f) - ls);
        s_v[t] = pv;
        dp_v[t] = pv * (dp_v[t] - dl);
      }
      if (hh == 0 && pair > 0 && !ptx::mbar_wait(pds_free, (uint32_t)(pair - 1) & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
#pragma unroll
      for (int g = 0; g < COLS / 8; ++g) {
        const int chunk = sub * (COLS / 8) + g;  // 16-byte chunk inside the 128-byte line of this row
        uint4 pw, dw;
        pw.x = ptx::pack2_bf16(s_v[g * 8 + 0], s_v[g * 8 + 1]);
        pw.y = ptx::pack2_bf16(s_v[g * 8 + 2], s_v[g * 8 + 3]);
        pw.z = ptx::pack2_bf16(s_v[g * 8 + 4], s_v[g * 8 + 5]);
        pw.w = ptx::pack2_bf16(s_v[g * 8 + 6], s_v[g * 8 + 7]);
        dw.x = ptx::pack2_bf16(dp_v[g * 8 + 0], dp_v[g * 8 + 1]);
        dw.y = ptx::pack2_bf16(dp_v[g * 8 + 2], dp_v[g * 8 + 3]);
        dw.z = ptx::pack2_bf16(dp_v[g * 8 + 4], dp_v[g * 8 + 5]);
        dw.w = ptx::pack2_bf16(dp_v[g * 8 + 6], dp_v[g * 8 + 7]);
        *reinterpret_cast<uint4*>(p_row + hh * 16384 + ((chunk ^ swz) << 4)) = pw;
        *reinterpret_cast<uint4*>(ds_row + hh * 16384 + ((chunk ^ swz) << 4)) = dw;
        if (ds_out != nullptr) {
          const int key = key0 + g * 8;
          if (p.vec_ok) {
            if (key < p.N) {
              uint4 hw;
              hw.x = pack2_f16_sat(dp_v[g * 8 + 0], dp_v[g * 8 + 1]);
              hw.y = pack2_f16_sat(dp_v[g * 8 + 2], dp_v[g * 8 + 3]);
              hw.z = pack2_f16_sat(dp_v[g * 8 + 4], dp_v[g * 8 + 5]);
              hw.w = pack2_f16_sat(dp_v[g * 8 + 6], dp_v[g * 8 + 7]);
              *reinterpret_cast<uint4*>(ds_out + key) = hw;
            }
          } else {
#pragma unroll
            for (int t = 0; t < 8; ++t)
              if (key + t < p.N) ds_out[key + t] = __float2half_rn(fminf(fmaxf(dp_v[g * 8 + t], -65504.f), 65504.f));
          }
        }
      }
      ptx::fence_proxy_async();   // P and dS written through the generic proxy, read by the tensor core
      ptx::mbar_arrive(&pds_ready[hh]);
      if (hh == 1 && i == T - 1) {
        // dK_j and dV_j are complete: this thread's key row, 8-column chunks sub, sub + 4, ...
        if (!ptx::mbar_wait(kv_acc_ready, (uint32_t)j & 1u, p.status, kTimeoutMmaDone)) { ok = false; break; }
        ptx::tc_fence_after();
        const int key = j * kTile + row_in_tile;
        float t8[8];
#pragma unroll 1
        for (int c = sub; c < DN / 8; c += kSoftmaxWarps / 4) {
          const bool in = key < p.N && c * 8 < p.D;
          ptx::tmem_ld_32x8(tmem_dk + lane_off + c * 8, t8);
          ptx::tmem_ld_wait();
          if (in) {
            __nv_bfloat16* dst = p.dk + b * p.dk_s[0] + r * p.dk_s[1] + h * p.dk_s[2] + (long long)key * p.dk_s[3] + c * 8;
            store_chunk8(dst, t8, p.scale, (reinterpret_cast<uintptr_t>(dst) & 15) == 0);
          }
          ptx::tmem_ld_32x8(tmem_dv + lane_off + c * 8, t8);
          ptx::tmem_ld_wait();
          if (in) {
            __nv_bfloat16* dst = p.dv + b * p.dv_s[0] + r * p.dv_s[1] + h * p.dv_s[2] + (long long)key * p.dv_s[3] + c * 8;
            store_chunk8(dst, t8, 1.f, (reinterpret_cast<uintptr_t>(dst) & 15) == 0);
          }
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(kv_acc_free);
      }
    }
    if (ok && ptx::mbar_wait(dq_ready, 0, p.status, kTimeoutMmaDone)) {
      ptx::tc_fence_after();
      float t8[8];
      for (int i = 0; i < T; ++i) {
        const int qi = i * kTile + row_in_tile;
#pragma unroll 1
        for (int c = sub; c < DN / 8; c += kSoftmaxWarps / 4) {
          ptx::tmem_ld_32x8(tmem_dq + i * DN + lane_off + c * 8, t8);
          ptx::tmem_ld_wait();
          if (qi < p.N && c * 8 < p.D) {
            __nv_bfloat16* dst = p.dq + b * p.dq_s[0] + r * p.dq_s[1] + h * p.dq_s[2] + (long long)qi * p.dq_s[3] + c * 8;
            store_chunk8(dst, t8, p.scale, (reinterpret_cast<uintptr_t>(dst) & 15) == 0);
          }
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

// dbias[bb, h, i, j] = sum over the rows r (and over b when the bias is shared by the batch) of ds[b, r, h, i, j], in a
// fixed order. One thread per 8 consecutive keys.
__global__ void __launch_bounds__(256) attention_dbias_reduce_kernel(const __half* __restrict__ ds, float* __restrict__ dbias,
                                                                     int B, int R, int H, long long nn, int per_batch, int vec) {
  const long long per_head = nn;  // N * N
  const long long groups = ((long long)H * per_head + 7) / 8;
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int bb = blockIdx.y;
  if (g >= groups) return;
  const long long e = g * 8;
  const long long hn = (long long)H * per_head;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  const int b0 = per_batch ? bb : 0, b1 = per_batch ? bb + 1 : B;
  for (int b = b0; b < b1; ++b) {
    const __half* src = ds + (long long)b * R * hn + e;
    if (vec) {
#pragma unroll 4
      for (int r = 0; r < R; ++r) {
        const uint4 w = *reinterpret_cast<const uint4*>(src + (long long)r * hn);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 pr = __half22float2(*reinterpret_cast<const __half2*>(&ww[k]));
          acc[2 * k] += pr.x;
          acc[2 * k + 1] += pr.y;
        }
      }
    } else {
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (e + k < hn) acc[k] += __half2float(src[(long long)r * hn + k]);
    }
  }
  float* dst = dbias + (long long)bb * hn + e;
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (e + k < hn) dst[k] = acc[k];
}

// fp32 O (contiguous [B, R, H, N, D]) against strided bf16 dO
__global__ void attention_delta_kernel_f32(const float* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                           long long g_sb, long long g_sr, long long g_sh, long long g_sn, int R, int H, int N, int D,
                                           long long total) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int n = (int)(e % N);
  const int h = (int)((e / N) % H);
  const int r = (int)((e / ((long long)N * H)) % R);
  const long long b = e / ((long long)N * H * R);
  const float* po = o + e * D;
  const __nv_bfloat16* pg = d_o + b * g_sb + r * g_sr + h * g_sh + (long long)n * g_sn;
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc += po[d] * __bfloat162float(pg[d]);
  delta[e] = acc;
}

__global__ void attention_delta_kernel2(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
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

}  // namespace

// Shapes the fused kernel takes: the accumulators of every query tile plus one key block must fit beside the two
// S/dP stages in the 512 tensor-memory columns.
bool attention_bwd_fused_supported(int64_t N, int64_t D) {
  if (D % 8 != 0 || D > 64 || N < 1) return false;
  const int64_t dn = (D + 15) / 16 * 16, T = (N + kTile - 1) / kTile;
  return (T + 2) * dn <= 256;
}

// q, k, v, out, d_out: [B, R, H, N, D] views; lse [2, B, R, H, N]; returns dq, dk, dv (written into dq_out / dk_out /
// dv_out when given, which may be strided views of a packed gradient) and dbias [Bb, H, N, N] fp32 (empty if not wanted).
std::tuple<Tensor, Tensor, Tensor, Tensor> attention_bwd_fused(const Tensor& q_in, const Tensor& k_in, const Tensor& v_in,
                                                               const Tensor& out, const Tensor& d_out,
                                                               const c10::optional<Tensor>& bias_in,
                                                               const c10::optional<Tensor>& mask_in, const Tensor& lse,
                                                               double scale, bool want_dbias, const c10::optional<Tensor>& dq_out,
                                                               const c10::optional<Tensor>& dk_out,
                                                               const c10::optional<Tensor>& dv_out) {
  const int64_t B = q_in.size(0), R = q_in.size(1), H = q_in.size(2), N = q_in.size(3), D = q_in.size(4);
  TORCH_CHECK(attention_bwd_fused_supported(N, D), "attention_bwd_fused: shape outside the tensor-memory budget");
  TORCH_CHECK(lse.dim() == 5 && lse.size(0) == 2 && lse.is_contiguous() && lse.scalar_type() == torch::kFloat32, "attention_bwd_fused: lse [2, B, R, H, N] fp32");
  c10::cuda::CUDAGuard guard(q_in.device());
  auto bf = q_in.options();
  Tensor q = strides_ok(q_in) ? q_in : q_in.contiguous();
  Tensor k = strides_ok(k_in) ? k_in : k_in.contiguous();
  Tensor v = strides_ok(v_in) ? v_in : v_in.contiguous();
  Tensor d_o = d_out.scalar_type() == torch::kBFloat16 ? d_out : d_out.to(torch::kBFloat16);
  if (!strides_ok(d_o)) d_o = d_o.contiguous();
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  Tensor delta = torch::empty({B, R, H, N}, bf.dtype(torch::kFloat32));
  if (out.scalar_type() == torch::kFloat32 && out.is_contiguous()) {
    const long long total = delta.numel();
    if (total > 0)
      attention_delta_kernel_f32<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
          out.data_ptr<float>(), reinterpret_cast<const __nv_bfloat16*>(d_o.data_ptr()), delta.data_ptr<float>(), d_o.stride(0),
          d_o.stride(1), d_o.stride(2), d_o.stride(3), (int)R, (int)H, (int)N, (int)D, total);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else if (out.scalar_type() == torch::kBFloat16 && out.stride(4) == 1) {
    const long long total = delta.numel();
    attention_delta_kernel2<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(out.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(d_o.data_ptr()),
        delta.data_ptr<float>(), out.stride(0), out.stride(1), out.stride(2), out.stride(3), d_o.stride(0), d_o.stride(1),
        d_o.stride(2), d_o.stride(3), (int)R, (int)H, (int)N, (int)D, total);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  } else {
    delta = (d_o.to(torch::kFloat32) * out.to(torch::kFloat32)).sum(-1).contiguous();
  }
  auto pick = [&](const c10::optional<Tensor>& given) {
    if (given.has_value() && given->defined()) {
      TORCH_CHECK(given->sizes() == q_in.sizes() && given->scalar_type() == torch::kBFloat16 && given->stride(4) == 1,
                  "attention_bwd_fused: gradient outputs are bf16 [B, R, H, N, D] views with a contiguous last axis");
      return *given;
    }
    return torch::empty({B, R, H, N, D}, bf);
  };
  Tensor dq = pick(dq_out), dk = pick(dk_out), dv = pick(dv_out);

  BwdParams p{};
  p.lse = lse.data_ptr<float>();
  p.delta = delta.data_ptr<float>();
  Tensor bias, mask, ds, dbias;
  const bool has_bias = bias_in.has_value() && bias_in->defined();
  if (has_bias) {
    bias = *bias_in;
    TORCH_CHECK(bias.dim() == 4 && bias.size(1) == H && bias.size(2) == N && bias.size(3) == N && (bias.size(0) == B || bias.size(0) == 1),
                "attention_bwd_fused: bias [B or 1, H, N, N]");
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
    TORCH_CHECK(mask.dim() == 3 && mask.size(2) == N && (mask.size(0) == B || mask.size(0) == 1) && (mask.size(1) == R || mask.size(1) == 1),
                "attention_bwd_fused: key mask [B or 1, R or 1, N]");
    if (mask.stride(2) != 1) mask = mask.contiguous();
    p.mask = mask.data_ptr<float>();
    p.mask_sb = mask.size(0) == 1 ? 0 : mask.stride(0);
    p.mask_sr = mask.size(1) == 1 ? 0 : mask.stride(1);
  }
  const bool need_ds = want_dbias && has_bias;
  if (need_ds) {
    ds = torch::empty({B, R, H, N, N}, bf.dtype(torch::kFloat16));
    p.ds = reinterpret_cast<__half*>(ds.data_ptr());
  }
  bool vec = N % 8 == 0;
  if (has_bias && p.bias_is_bf16)
    vec = vec && reinterpret_cast<uintptr_t>(bias.data_ptr()) % 16 == 0 && bias.stride(2) % 8 == 0 && bias.stride(1) % 8 == 0 &&
          (bias.size(0) == 1 || bias.stride(0) % 8 == 0);
  p.vec_ok = vec;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq.data_ptr());
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk.data_ptr());
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv.data_ptr());
  for (int d = 0; d < 4; ++d) {
    p.dq_s[d] = dq.stride(d);
    p.dk_s[d] = dk.stride(d);
    p.dv_s[d] = dv.stride(d);
  }
  Tensor status = status_word(q.device().index());
  p.status = status.data_ptr<int>();
  p.B = (int)B; p.R = (int)R; p.H = (int)H; p.N = (int)N; p.D = (int)D;
  p.T = (int)((N + kTile - 1) / kTile);
  p.scale = (float)scale;
  p.scale_log2 = (float)scale * kLog2e;
  if (q.numel() > 0) {
    const CUtensorMap tq = qkv_map(q), tk = qkv_map(k), tv = qkv_map(v), tdo = qkv_map(d_o);
    const long long ctas = (long long)B * R * H;
    TORCH_CHECK(ctas < (1ll << 31), "attention_bwd_fused: grid too large");
    const size_t smem = 12 * kTileBytes + 20 * 8 + (size_t)p.T * kTile * 4 + 16;
    const int dn = (int)((D + 15) / 16 * 16);
#define DF3_ATTN_BWD(DN_)                                                                                              \
  do {                                                                                                                 \
    static bool attr = false;                                                                                          \
    if (!attr) {                                                                                                       \
      C10_CUDA_CHECK(cudaFuncSetAttribute(attention_bwd_kernel<DN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)); \
      attr = true;                                                                                                     \
    }                                                                                                                  \
    attention_bwd_kernel<DN_><<<(unsigned)ctas, kBwdThreads, smem, stream>>>(tq, tk, tv, tdo, p);                      \
  } while (0)
    if (dn == 16) DF3_ATTN_BWD(16); else if (dn == 32) DF3_ATTN_BWD(32); else if (dn == 48) DF3_ATTN_BWD(48); else DF3_ATTN_BWD(64);
#undef DF3_ATTN_BWD
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  if (need_ds) {
    const int64_t Bb = bias.size(0);
    dbias = torch::empty({Bb, H, N, N}, bf.dtype(torch::kFloat32));
    const long long hn = (long long)H * N * N;
    if (hn > 0) {
      const long long groups = (hn + 7) / 8;
      dim3 grid((unsigned)((groups + 255) / 256), (unsigned)Bb);
      attention_dbias_reduce_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __half*>(ds.data_ptr()), dbias.data_ptr<float>(),
                                                              (int)B, (int)R, (int)H, (long long)N * N, Bb > 1 ? 1 : 0, (hn % 8 == 0) ? 1 : 0);
      C10_CUDA_KERNEL_LAUNCH_CHECK();
    }
  } else {
    dbias = torch::empty({0}, bf.dtype(torch::kFloat32));
  }
  return {dq, dk, dv, dbias};
}

}  // namespace df3
