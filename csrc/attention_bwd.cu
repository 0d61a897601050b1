// Causal softmax attention backward on tcgen05, in two kernels that never use atomics:
//   k_attn_bwd_dq   one CTA per 128-row query block, loops over 64-key blocks:
//                   S = Q K^T, dP = dO V^T (tensor memory) -> dS = P o (dP - delta) * scale (bf16, written
//                   back over dP) -> dQ += dS K
//   k_attn_bwd_dkv  one CTA per 128-key block, loops over 64-row query blocks:
//                   S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T (bf16 in tensor memory) -> dV += P^T dO,
//                   dK += dS^T Q
// P is recomputed from the saved log-sum-exp; delta = rowsum(O o dO) comes from a small pre-pass.
// The second operand of the accumulating products is the same shared-memory tile that fed the
// first product, read through an MN-major descriptor, so every tile is loaded once.
// Same masking as the forward (causal, optional sliding window); sinks only change the saved
// log-sum-exp.  Head dims (Dqk, Dv): (192,128), (128,128), (64,64).
//
// Replaces FlashMLA's sm100 backward (nmoe/attention/mla.py:93-147) and the Triton SWA backward
// (nmoe/triton/swa.py:290-571) of the reference.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common/ptx.cuh"
#include "common/tensormap.h"

namespace nmoe {

constexpr int kBwdThreads = 320;           // warp 0: TMA, warp 1: MMA, warps 2-9: softmax / epilogue (two column halves x four lane quadrants)
constexpr int BWD_STAGES = 3;              // streamed-tile stages: a load is issued one full iteration before it is needed
constexpr int BWD_BIG = 128;               // rows of the resident block
constexpr int BWD_SMALL = 64;              // rows of the streamed block
constexpr uint64_t kBwdWaitNs = 2000000000ull;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnBwdParams {
  int B, S, Hq, Hkv, window;
  // operand addressing exactly as in the forward (column of head h inside a row of the 2-D view):
  // K chunk c (64 columns) comes from source 1 while c < k1_chunks, from source 2 afterwards.
  int q_hs, k1_hs, k1_off, k1_chunks, k2_hs, k2_off, v_hs, v_off, do_hs;
  float scale, scale_log2;
  const float* lse;                        // [B, Hq, S] natural log
  const float* delta;                      // [B, Hq, S]
  // optional token-level sparsity, as in the forward: mask[(b*S + q)*mask_words + k/32] bit k%32, and its
  // transpose mask_t[(b*S + k)*mask_words + q/32] bit q%32 (the dK/dV kernel owns a key per thread)
  const uint32_t* mask;
  const uint32_t* mask_t;
  int mask_words;
  // outputs: one slot per QUERY head (the caller sums a GQA group or a shared rotary key);
  // *_row = row length in elements, *_hs = per-query-head stride, *_off = first column.
  __nv_bfloat16* dQ;  int dq_row, dq_hs;
  __nv_bfloat16* dK1; int dk1_row, dk1_hs, dk1_off;     // gradient of the K chunks that came from source 1
  __nv_bfloat16* dK2; int dk2_row, dk2_hs, dk2_off;     // ... from source 2
  __nv_bfloat16* dV;  int dv_row, dv_hs, dv_off;
  StatusRecord* status;
};

NMOE_DEVICE uint64_t bwd_timer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
NMOE_DEVICE bool bwd_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = bwd_timer();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 255u) == 0) {
      if (*abort_flag) return false;
      if (bwd_timer() - t0 > kBwdWaitNs) return false;
    }
  }
  return true;
}
NMOE_DEVICE void bwd_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
NMOE_DEVICE void bwd_tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
NMOE_DEVICE float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
NMOE_DEVICE bool masked(int q, int k, int S, int window) {
  return k > q || k >= S || (window > 0 && k <= q - window);
}
// store 32 fp32 accumulator values (scaled) as bf16 to a row in global memory
NMOE_DEVICE void store_row32(__nv_bfloat16* dst, const uint32_t* r, float s) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    int4 v;
    v.x = pack_bf16x2(__uint_as_float(r[8 * t]) * s, __uint_as_float(r[8 * t + 1]) * s);
    v.y = pack_bf16x2(__uint_as_float(r[8 * t + 2]) * s, __uint_as_float(r[8 * t + 3]) * s);
    v.z = pack_bf16x2(__uint_as_float(r[8 * t + 4]) * s, __uint_as_float(r[8 * t + 5]) * s);
    v.w = pack_bf16x2(__uint_as_float(r[8 * t + 6]) * s, __uint_as_float(r[8 * t + 7]) * s);
    reinterpret_cast<int4*>(dst)[t] = v;
  }
}

// delta[b,h,s] = sum_d O[b,s,h,d] * dO[b,s,h,d]   (Dv/8 lanes per (row, head), 16 bytes each)
__global__ void __launch_bounds__(256)
k_attn_delta(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
             int B, int S, int H, int Dv) {
  const int lpr = Dv >> 3;                                     // lanes per row: 8 or 16
  const long long tid = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const long long idx = tid / lpr;
  const int sub = static_cast<int>(tid % lpr);
  const bool live = idx < static_cast<long long>(B) * S * H;
  float acc = 0.f;
  if (live) {
    const int4 a = ld_nc_v4(o + idx * Dv + sub * 8), b = ld_nc_v4(d_o + idx * Dv + sub * 8);
    const float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
    acc = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
  }
  for (int off = lpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (live && sub == 0) {
    const int h = static_cast<int>(idx % H);
    const long long bs = idx / H;
    const int b = static_cast<int>(bs / S), sq = static_cast<int>(bs % S);
    delta[(static_cast<long long>(b) * H + h) * S + sq] = acc;
  }
}

template <int DQK, int DV>
struct BwdSmem {
  static constexpr int kBigQK = BWD_BIG * DQK * 2;      // resident [128, DQK] tile (Q or K)
  static constexpr int kBigV = BWD_BIG * DV * 2;        // resident [128, DV] tile (dO or V)
  static constexpr int kSmallQK = BWD_SMALL * DQK * 2;  // streamed [64, DQK] tile
  static constexpr int kSmallV = BWD_SMALL * DV * 2;
  static constexpr int kBytes = kBigQK + kBigV + BWD_STAGES * (kSmallQK + kSmallV) + 1024 + 256 + 1536;  // align, barriers, row statistics
};

// ---------------------------------------------------------------------------------------------
// dQ: CTA = (128-row query block, head, batch); streams 64-key blocks through BWD_STAGES stages.
// Tensor memory columns: S[2] at 0/64, dP[2] at 128/192, dQ accumulator at 256.  The eight
// softmax warps split a block's 64 columns in two halves; each half writes its dS as bf16 over
// the first 16 columns of the dP columns it has just read (columns 0-15 and 32-47 of the buffer).
// ---------------------------------------------------------------------------------------------
template <int DQK, int DV>
__global__ void __launch_bounds__(kBwdThreads, 1)
k_attn_bwd_dq(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmK2, const __grid_constant__ CUtensorMap tmV,
              const __grid_constant__ CUtensorMap tmdO, const AttnBwdParams p) {
  using SM = BwdSmem<DQK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + SM::kBigQK;
  uint8_t* sK = sdO + SM::kBigV;
  uint8_t* sV = sK + BWD_STAGES * SM::kSmallQK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + BWD_STAGES * SM::kSmallV);
  uint64_t* qdo_full = bars;          // [1]
  uint64_t* kv_full = bars + 1;       // [3]
  uint64_t* kv_empty = bars + 4;      // [3]
  uint64_t* sdp_full = bars + 7;      // [2]  S and dP of a block are in tensor memory
  uint64_t* ds_full = bars + 9;       // [2]  dS written by the eight softmax warps
  uint64_t* dq_done = bars + 11;      // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_blk = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // heavy blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = q_blk * BWD_BIG;
  const int hkv = h / (p.Hq / p.Hkv);
  const int hi = min((q0 + BWD_BIG + BWD_SMALL - 1) / BWD_SMALL, (p.S + BWD_SMALL - 1) / BWD_SMALL);
  const int lo = p.window > 0 ? max(0, (q0 - p.window + 1) / BWD_SMALL) : 0;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < BWD_STAGES; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sdp_full[i], 1); mbar_init(&ds_full[i], 8); }
    mbar_init(dq_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColdP = 128, kColdQ = 256;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmK2); tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmdO);
      const int row_q = b * p.S + q0;
      mbar_expect_tx(qdo_full, SM::kBigQK + SM::kBigV);
#pragma unroll
      for (int c = 0; c < DQK / 64; ++c) tma_load_2d(sQ + c * (BWD_BIG * 128), &tmQ, qdo_full, h * p.q_hs + c * 64, row_q);
#pragma unroll
      for (int c = 0; c < DV / 64; ++c) tma_load_2d(sdO + c * (BWD_BIG * 128), &tmdO, qdo_full, h * p.do_hs + c * 64, row_q);
      int st = 0; uint32_t ph = 0;
      for (int i = lo; i < hi; ++i) {
        const int row_k = b * p.S + i * BWD_SMALL;
        if (!bwd_wait(&kv_empty[st], ph ^ 1, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 800, i, 0); *abort_flag = 1; break; }
        mbar_expect_tx(&kv_full[st], SM::kSmallQK + SM::kSmallV);
#pragma unroll
        for (int c = 0; c < DQK / 64; ++c) {
          if (c < p.k1_chunks)
            tma_load_2d(sK + st * SM::kSmallQK + c * (BWD_SMALL * 128), &tmK, &kv_full[st], hkv * p.k1_hs + p.k1_off + c * 64, row_k);
          else
            tma_load_2d(sK + st * SM::kSmallQK + c * (BWD_SMALL * 128), &tmK2, &kv_full[st],
                        hkv * p.k2_hs + p.k2_off + (c - p.k1_chunks) * 64, row_k);
        }
#pragma unroll
        for (int c = 0; c < DV / 64; ++c)
          tma_load_2d(sV + st * SM::kSmallV + c * (BWD_SMALL * 128), &tmV, &kv_full[st], hkv * p.v_hs + p.v_off + c * 64, row_k);
        if (++st == BWD_STAGES) { st = 0; ph ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BWD_BIG, BWD_SMALL, 0, 0);
      constexpr uint32_t idesc_dq = make_idesc_bf16(BWD_BIG, DQK, 0, 1);
      bool ok = hi > lo && bwd_wait(qdo_full, 0, abort_flag);
      const uint32_t qa = smem_u32(sQ), doa = smem_u32(sdO);
      int st_s = 0; uint32_t ph_s = 0;       // stage / phase of the next block whose S, dP get issued
      auto issue_sdp = [&](int i) -> bool {
        const int bf = (i - lo) & 1;
        if (!bwd_wait(&kv_full[st_s], ph_s, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 810, i, 0); *abort_flag = 1; return false; }
        tc_fence_after_sync();
        const uint32_t ka = smem_u32(sK + st_s * SM::kSmallQK), va = smem_u32(sV + st_s * SM::kSmallV);
#pragma unroll
        for (int j = 0; j < DQK / 16; ++j)
          mma_f16_ss(tmem_base + kColS + bf * BWD_SMALL,
                     make_smem_desc(qa + (j >> 2) * (BWD_BIG * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B),
                     make_smem_desc(ka + (j >> 2) * (BWD_SMALL * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B), idesc_s,
                     j != 0 ? 1u : 0u);
#pragma unroll
        for (int j = 0; j < DV / 16; ++j)
          mma_f16_ss(tmem_base + kColdP + bf * BWD_SMALL,
                     make_smem_desc(doa + (j >> 2) * (BWD_BIG * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B),
                     make_smem_desc(va + (j >> 2) * (BWD_SMALL * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B), idesc_s,
                     j != 0 ? 1u : 0u);
        mma_commit(&sdp_full[bf]);
        if (++st_s == BWD_STAGES) { st_s = 0; ph_s ^= 1; }
        return true;
      };
      if (ok) ok = issue_sdp(lo);
      int st = 0;
      for (int i = lo; ok && i < hi; ++i) {
        const int gi = i - lo, bf = gi & 1;
        if (i + 1 < hi) { ok = issue_sdp(i + 1); if (!ok) break; }
        if (!bwd_wait(&ds_full[bf], (gi >> 1) & 1, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 811, i, 0); *abort_flag = 1; ok = false; break; }
        tc_fence_after_sync();
        const uint32_t ka = smem_u32(sK + st * SM::kSmallQK);
        const uint32_t a_t = tmem_base + kColdP + bf * BWD_SMALL;
#pragma unroll
        for (int j = 0; j < BWD_SMALL / 16; ++j)
          bwd_mma_ts(tmem_base + kColdQ, a_t + (j >> 1) * 32 + (j & 1) * 8,
                     make_smem_desc(ka + j * 2048, BWD_SMALL * 128, 1024, kSwizzle128B), idesc_dq, (gi | j) != 0 ? 1u : 0u);
        mma_commit(&kv_empty[st]);
        if (++st == BWD_STAGES) st = 0;
      }
      if (ok) mma_commit(dq_done);
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = q0 + q * 32 + lane;
    const bool row_ok = row < p.S;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const size_t stat_idx = (static_cast<size_t>(b) * p.Hq + h) * p.S + (row_ok ? row : 0);
    const float lse2 = row_ok ? p.lse[stat_idx] * kLog2e : 1e30f;    // rows past the sequence: P = 0
    const float dl = row_ok ? p.delta[stat_idx] : 0.f;
    bool ok = true;
    for (int i = lo; i < hi; ++i) {
      const int gi = i - lo, bf = gi & 1;
      ok = bwd_wait(&sdp_full[bf], (gi >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 820, i, 0); *abort_flag = 1; break; }
      tc_fence_after_sync();
      const int k0 = i * BWD_SMALL + half * 32;
      const bool need_mask = (k0 + 31 > q0) || (p.window > 0 && k0 <= q0 + BWD_BIG - 1 - p.window) || (k0 + 32 > p.S);
      const uint32_t s_addr = tmem_base + lane_addr + kColS + bf * BWD_SMALL + half * 32;
      const uint32_t dp_addr = tmem_base + lane_addr + kColdP + bf * BWD_SMALL + half * 32;
      uint32_t s[32], dp[32], pk[16];
      tmem_ld_32x32b_x32(s_addr, s);
      tmem_ld_32x32b_x32(dp_addr, dp);
      uint32_t mw = 0xffffffffu;
      if (p.mask != nullptr)
        mw = row_ok ? __ldg(p.mask + (static_cast<size_t>(b) * p.S + row) * p.mask_words + (k0 >> 5)) : 0u;
      tmem_ld_wait();
#pragma unroll
      for (int t = 0; t < 32; t += 2) {
        float p0 = bwd_exp2(fmaf(__uint_as_float(s[t]), p.scale_log2, -lse2));
        float p1 = bwd_exp2(fmaf(__uint_as_float(s[t + 1]), p.scale_log2, -lse2));
        if (need_mask) {
          if (masked(row, k0 + t, p.S, p.window)) p0 = 0.f;
          if (masked(row, k0 + t + 1, p.S, p.window)) p1 = 0.f;
        }
        if (!((mw >> t) & 1u)) p0 = 0.f;
        if (!((mw >> (t + 1)) & 1u)) p1 = 0.f;
        const float d0 = p0 * (__uint_as_float(dp[t]) - dl) * p.scale;
        const float d1 = p1 * (__uint_as_float(dp[t + 1]) - dl) * p.scale;
        pk[t >> 1] = pack_bf16x2(d0, d1);
      }
      bwd_tmem_st_x16(dp_addr, pk);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[bf]);
    }
    if (ok && hi > lo) {
      ok = bwd_wait(dq_done, 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 821, 0, 0); *abort_flag = 1; }
    }
    if (ok) {
      tc_fence_after_sync();
      __nv_bfloat16* drow = p.dQ + (static_cast<size_t>(b) * p.S + (row_ok ? row : 0)) * p.dq_row + static_cast<size_t>(h) * p.dq_hs;
#pragma unroll 1
      for (int c = half; c < DQK / 32; c += 2) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColdQ + c * 32, o);
        tmem_ld_wait();
        if (row_ok) store_row32(drow + c * 32, o, 1.f);
      }
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// dK, dV: CTA = (128-key block, query head, batch); streams 64-row query blocks.
// Tensor memory columns: S^T[2] at 0/64, dP^T at 128, dV accumulator at 192, dK accumulator at
// 192+DV.  Each half of the eight softmax warps owns 32 of a block's 64 columns and writes P^T /
// dS^T as bf16 over the first 16 of the columns it has just read (0-15 and 32-47).
// ---------------------------------------------------------------------------------------------
template <int DQK, int DV>
__global__ void __launch_bounds__(kBwdThreads, 1)
k_attn_bwd_dkv(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmK2, const __grid_constant__ CUtensorMap tmV,
               const __grid_constant__ CUtensorMap tmdO, const AttnBwdParams p) {
  using SM = BwdSmem<DQK, DV>;
  static_assert(192 + DV + DQK <= 512, "tensor memory budget");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + SM::kBigQK;
  uint8_t* sQ = sV + SM::kBigV;
  uint8_t* sdO = sQ + BWD_STAGES * SM::kSmallQK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdO + BWD_STAGES * SM::kSmallV);
  uint64_t* kv_full = bars;           // [1]
  uint64_t* q_full = bars + 1;        // [3]  Q, dO tiles (TMA) and the row statistics (warp 0) of a block
  uint64_t* q_empty = bars + 4;       // [3]
  uint64_t* s_full = bars + 7;        // [2]
  uint64_t* dp_full = bars + 9;       // [1]
  uint64_t* pds_full = bars + 10;     // [1]  P^T and dS^T written by the eight softmax warps
  uint64_t* acc_done = bars + 11;     // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* s_lse = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 256);   // [stage][64], log2 units
  float* s_delta = s_lse + BWD_STAGES * BWD_SMALL;                                   // [stage][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int k0 = kb * BWD_BIG;
  const int hkv = h / (p.Hq / p.Hkv);
  const int n_qb = (p.S + BWD_SMALL - 1) / BWD_SMALL;
  const int lo = k0 / BWD_SMALL;
  const int hi = p.window > 0 ? min(n_qb, (k0 + BWD_BIG - 1 + p.window - 1) / BWD_SMALL + 1) : n_qb;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < BWD_STAGES; ++i) { mbar_init(&q_full[i], 2); mbar_init(&q_empty[i], 1); }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColdP = 128, kColdV = 192, kColdK = 192 + DV;

  if (warp == 0) {
    // whole warp: one elected lane issues the TMA copies, all lanes stage lse / delta of the block
    const bool leader = elect_one();
    if (leader) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmK2); tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmdO);
      const int row_k = b * p.S + k0;
      mbar_expect_tx(kv_full, SM::kBigQK + SM::kBigV);
#pragma unroll
      for (int c = 0; c < DQK / 64; ++c) {
        if (c < p.k1_chunks)
          tma_load_2d(sK + c * (BWD_BIG * 128), &tmK, kv_full, hkv * p.k1_hs + p.k1_off + c * 64, row_k);
        else
          tma_load_2d(sK + c * (BWD_BIG * 128), &tmK2, kv_full, hkv * p.k2_hs + p.k2_off + (c - p.k1_chunks) * 64, row_k);
      }
#pragma unroll
      for (int c = 0; c < DV / 64; ++c)
        tma_load_2d(sV + c * (BWD_BIG * 128), &tmV, kv_full, hkv * p.v_hs + p.v_off + c * 64, row_k);
    }
    const size_t stat_base = (static_cast<size_t>(b) * p.Hq + h) * p.S;
    int st = 0; uint32_t ph = 0;
    for (int i = lo; i < hi; ++i) {
      bool ok = bwd_wait(&q_empty[st], ph ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 830, i, 0); *abort_flag = 1; break; }
      if (leader) {
        const int row_q = b * p.S + i * BWD_SMALL;
        mbar_expect_tx(&q_full[st], SM::kSmallQK + SM::kSmallV);
#pragma unroll
        for (int c = 0; c < DQK / 64; ++c)
          tma_load_2d(sQ + st * SM::kSmallQK + c * (BWD_SMALL * 128), &tmQ, &q_full[st], h * p.q_hs + c * 64, row_q);
#pragma unroll
        for (int c = 0; c < DV / 64; ++c)
          tma_load_2d(sdO + st * SM::kSmallV + c * (BWD_SMALL * 128), &tmdO, &q_full[st], h * p.do_hs + c * 64, row_q);
      }
#pragma unroll
      for (int t = lane; t < BWD_SMALL; t += 32) {
        const int r = i * BWD_SMALL + t;
        // rows past the sequence get an "infinite" log-sum-exp so that their P is exactly zero
        s_lse[st * BWD_SMALL + t] = r < p.S ? p.lse[stat_base + r] * kLog2e : 1e30f;
        s_delta[st * BWD_SMALL + t] = r < p.S ? p.delta[stat_base + r] : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full[st]);
      if (++st == BWD_STAGES) { st = 0; ph ^= 1; }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BWD_BIG, BWD_SMALL, 0, 0);
      constexpr uint32_t idesc_dv = make_idesc_bf16(BWD_BIG, DV, 0, 1);
      constexpr uint32_t idesc_dk = make_idesc_bf16(BWD_BIG, DQK, 0, 1);
      bool ok = hi > lo && bwd_wait(kv_full, 0, abort_flag);
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      int st_s = 0; uint32_t ph_s = 0;       // stage / phase of the next block whose S^T gets issued
      auto issue_s = [&](int i) -> bool {
        const int bf = (i - lo) & 1;
        if (!bwd_wait(&q_full[st_s], ph_s, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 840, i, 0); *abort_flag = 1; return false; }
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(sQ + st_s * SM::kSmallQK);
#pragma unroll
        for (int j = 0; j < DQK / 16; ++j)
          mma_f16_ss(tmem_base + kColS + bf * BWD_SMALL,
                     make_smem_desc(ka + (j >> 2) * (BWD_BIG * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B),
                     make_smem_desc(qa + (j >> 2) * (BWD_SMALL * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B), idesc_s,
                     j != 0 ? 1u : 0u);
        mma_commit(&s_full[bf]);
        if (++st_s == BWD_STAGES) { st_s = 0; ph_s ^= 1; }
        return true;
      };
      auto issue_dp = [&](int st) {
        const uint32_t doa = smem_u32(sdO + st * SM::kSmallV);
#pragma unroll
        for (int j = 0; j < DV / 16; ++j)
          mma_f16_ss(tmem_base + kColdP,
                     make_smem_desc(va + (j >> 2) * (BWD_BIG * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B),
                     make_smem_desc(doa + (j >> 2) * (BWD_SMALL * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B), idesc_s,
                     j != 0 ? 1u : 0u);
        mma_commit(dp_full);
      };
      if (ok) { ok = issue_s(lo); if (ok) issue_dp(0); }
      int st = 0;
      for (int i = lo; ok && i < hi; ++i) {
        const int gi = i - lo, bf = gi & 1;
        const int st_next = st + 1 == BWD_STAGES ? 0 : st + 1;
        if (i + 1 < hi) { ok = issue_s(i + 1); if (!ok) break; }
        if (!bwd_wait(pds_full, gi & 1, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 841, i, 0); *abort_flag = 1; ok = false; break; }
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(sQ + st * SM::kSmallQK), doa = smem_u32(sdO + st * SM::kSmallV);
        const uint32_t p_t = tmem_base + kColS + bf * BWD_SMALL, ds_t = tmem_base + kColdP;
        // dK first: it frees the dP^T columns, so the next block's dP^T (which the softmax warps
        // wait for) is issued before dV
#pragma unroll
        for (int j = 0; j < BWD_SMALL / 16; ++j)
          bwd_mma_ts(tmem_base + kColdK, ds_t + (j >> 1) * 32 + (j & 1) * 8,
                     make_smem_desc(qa + j * 2048, BWD_SMALL * 128, 1024, kSwizzle128B), idesc_dk, (gi | j) != 0 ? 1u : 0u);
        if (i + 1 < hi) issue_dp(st_next);
#pragma unroll
        for (int j = 0; j < BWD_SMALL / 16; ++j)
          bwd_mma_ts(tmem_base + kColdV, p_t + (j >> 1) * 32 + (j & 1) * 8,
                     make_smem_desc(doa + j * 2048, BWD_SMALL * 128, 1024, kSwizzle128B), idesc_dv, (gi | j) != 0 ? 1u : 0u);
        mma_commit(&q_empty[st]);
        st = st_next;
      }
      if (ok) mma_commit(acc_done);
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int key = k0 + q * 32 + lane;
    const bool key_ok = key < p.S;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    int st = 0; uint32_t ph = 0;
    for (int i = lo; i < hi; ++i) {
      const int gi = i - lo, bf = gi & 1;
      ok = bwd_wait(&q_full[st], ph, abort_flag) && bwd_wait(&s_full[bf], (gi >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 850, i, 0); *abort_flag = 1; break; }
      tc_fence_after_sync();
      const int r0 = i * BWD_SMALL + half * 32;
      const bool need_mask = (r0 < k0 + BWD_BIG - 1) || (p.window > 0 && r0 + 31 - p.window >= k0) || (k0 + BWD_BIG > p.S);
      const uint32_t s_addr = tmem_base + lane_addr + kColS + bf * BWD_SMALL + half * 32;
      const uint32_t dp_addr = tmem_base + lane_addr + kColdP + half * 32;
      const float4* lse4 = reinterpret_cast<const float4*>(s_lse + st * BWD_SMALL + half * 32);
      const float4* dl4 = reinterpret_cast<const float4*>(s_delta + st * BWD_SMALL + half * 32);
      float pf[32];
      {
        uint32_t s[32], pk[16];
        tmem_ld_32x32b_x32(s_addr, s);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          const float4 l4 = lse4[t >> 2];
          pf[t] = bwd_exp2(fmaf(__uint_as_float(s[t]), p.scale_log2, -l4.x));
          pf[t + 1] = bwd_exp2(fmaf(__uint_as_float(s[t + 1]), p.scale_log2, -l4.y));
          pf[t + 2] = bwd_exp2(fmaf(__uint_as_float(s[t + 2]), p.scale_log2, -l4.z));
          pf[t + 3] = bwd_exp2(fmaf(__uint_as_float(s[t + 3]), p.scale_log2, -l4.w));
        }
        if (need_mask) {
#pragma unroll
          for (int t = 0; t < 32; ++t)
            if (masked(r0 + t, key, p.S, p.window)) pf[t] = 0.f;
        }
        if (p.mask_t != nullptr) {
          const uint32_t mw = key < p.S ? __ldg(p.mask_t + (static_cast<size_t>(b) * p.S + key) * p.mask_words + (r0 >> 5)) : 0u;
#pragma unroll
          for (int t = 0; t < 32; ++t)
            if (!((mw >> t) & 1u)) pf[t] = 0.f;
        }
#pragma unroll
        for (int t = 0; t < 32; t += 2) pk[t >> 1] = pack_bf16x2(pf[t], pf[t + 1]);
        bwd_tmem_st_x16(s_addr, pk);
      }
      ok = bwd_wait(dp_full, gi & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 851, i, 0); *abort_flag = 1; break; }
      tc_fence_after_sync();
      {
        uint32_t dp[32], dk[16];
        tmem_ld_32x32b_x32(dp_addr, dp);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          const float4 d4 = dl4[t >> 2];
          dk[t >> 1] = pack_bf16x2(pf[t] * (__uint_as_float(dp[t]) - d4.x) * p.scale,
                                   pf[t + 1] * (__uint_as_float(dp[t + 1]) - d4.y) * p.scale);
          dk[(t >> 1) + 1] = pack_bf16x2(pf[t + 2] * (__uint_as_float(dp[t + 2]) - d4.z) * p.scale,
                                         pf[t + 3] * (__uint_as_float(dp[t + 3]) - d4.w) * p.scale);
        }
        bwd_tmem_st_x16(dp_addr, dk);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (++st == BWD_STAGES) { st = 0; ph ^= 1; }
    }
    if (ok && hi > lo) {
      ok = bwd_wait(acc_done, 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 852, 0, 0); *abort_flag = 1; }
    }
    if (ok) {
      tc_fence_after_sync();
      const size_t grow = static_cast<size_t>(b) * p.S + (key_ok ? key : 0);
      __nv_bfloat16* dv_row = p.dV + grow * p.dv_row + static_cast<size_t>(h) * p.dv_hs + p.dv_off;
#pragma unroll 1
      for (int c = half; c < DV / 32; c += 2) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColdV + c * 32, o);
        tmem_ld_wait();
        if (key_ok) store_row32(dv_row + c * 32, o, 1.f);
      }
#pragma unroll 1
      for (int c = half; c < DQK / 32; c += 2) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + kColdK + c * 32, o);
        tmem_ld_wait();
        const int chunk = c >> 1;
        __nv_bfloat16* dst = chunk < p.k1_chunks
            ? p.dK1 + grow * p.dk1_row + static_cast<size_t>(h) * p.dk1_hs + p.dk1_off + c * 32
            : p.dK2 + grow * p.dk2_row + static_cast<size_t>(h) * p.dk2_hs + p.dk2_off + (c - 2 * p.k1_chunks) * 32;
        if (key_ok) store_row32(dst, o, 1.f);
      }
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

static int bwd_map(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint32_t box_rows) {
  using Key = std::tuple<const void*, uint64_t, uint64_t, uint32_t>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  Key k{base, inner, outer, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(k);
  if (it != cache.end()) { *out = it->second; return 0; }
  int rc = make_tensor_map_2d(out, base, kTmaBf16, inner, outer, inner * 2, 64, box_rows, kTmaSwizzle128);
  if (rc != 0) return rc;
  if (cache.size() > 1024) cache.clear();
  cache[k] = *out;
  return 0;
}

struct BwdOperands {
  const void *q, *k1, *k2, *v, *d_o;
  int q_row, k1_row, k2_row, v_row, do_row;
};

template <int DQK, int DV>
static int attn_bwd_launch(const BwdOperands& a, const AttnBwdParams& p, cudaStream_t st) {
  auto kq = k_attn_bwd_dq<DQK, DV>;
  auto kkv = k_attn_bwd_dkv<DQK, DV>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<DQK, DV>::kBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem<DQK, DV>::kBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const uint64_t rows = static_cast<uint64_t>(p.B) * p.S;
  const void* k2 = a.k2 ? a.k2 : a.k1;
  const int k2_row = a.k2 ? a.k2_row : a.k1_row;
  CUtensorMap tq, tk, tk2, tv, tdo;
  int rc;
  // dK, dV: K / V resident (128-row boxes), Q / dO streamed (64-row boxes)
  if ((rc = bwd_map(&tq, a.q, a.q_row, rows, BWD_SMALL))) return rc;
  if ((rc = bwd_map(&tk, a.k1, a.k1_row, rows, BWD_BIG))) return rc;
  if ((rc = bwd_map(&tk2, k2, k2_row, rows, BWD_BIG))) return rc;
  if ((rc = bwd_map(&tv, a.v, a.v_row, rows, BWD_BIG))) return rc;
  if ((rc = bwd_map(&tdo, a.d_o, a.do_row, rows, BWD_SMALL))) return rc;
  dim3 grid((p.S + BWD_BIG - 1) / BWD_BIG, p.Hq, p.B);
  kkv<<<grid, kBwdThreads, BwdSmem<DQK, DV>::kBytes, st>>>(tq, tk, tk2, tv, tdo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  // dQ: Q / dO resident, K / V streamed
  if ((rc = bwd_map(&tq, a.q, a.q_row, rows, BWD_BIG))) return rc;
  if ((rc = bwd_map(&tk, a.k1, a.k1_row, rows, BWD_SMALL))) return rc;
  if ((rc = bwd_map(&tk2, k2, k2_row, rows, BWD_SMALL))) return rc;
  if ((rc = bwd_map(&tv, a.v, a.v_row, rows, BWD_SMALL))) return rc;
  if ((rc = bwd_map(&tdo, a.d_o, a.do_row, rows, BWD_BIG))) return rc;
  kq<<<grid, kBwdThreads, BwdSmem<DQK, DV>::kBytes, st>>>(tq, tk, tk2, tv, tdo, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace nmoe

using namespace nmoe;

// Backward of nmoe_attn_fwd_ex with the same operand addressing.  o, d_o: [B,S,Hq,Dv] contiguous bf16;
// lse [B,Hq,S] from the forward; delta [B,Hq,S] fp32 scratch that this call fills (and leaves
// for the caller: the sink gradient is -sum exp(sink - lse) * delta).  Gradients are written per
// QUERY head: dq [rows, dq_row] at h*dq_hs; dk1 / dk2 / dv likewise with a first-column offset.
// args: 17 ints of output addressing packed as an array to keep the signature readable:
//   {dq_row, dq_hs, dk1_row, dk1_hs, dk1_off, dk2_row, dk2_hs, dk2_off, dv_row, dv_hs, dv_off}
// mask / mask_t: optional bit rows [B, S, 2*ceil(S/64)] (query-major and key-major), as in the forward.
extern "C" int nmoe_attn_bwd_masked(const void* q, int q_row, int q_hs, const void* k1, int k1_row, int k1_hs, int k1_off,
                                    int k1_chunks, const void* k2, int k2_row, int k2_hs, int k2_off, const void* v,
                                    int v_row, int v_hs, int v_off, const void* o, const void* d_o, const float* lse,
                                    float* delta, void* dq, void* dk1, void* dk2, void* dv, const int* out_addr,
                                    const void* mask, const void* mask_t, int B, int S, int Hq, int Hkv, int Dqk, int Dv,
                                    int window, float scale, void* status, cudaStream_t st);

extern "C" int nmoe_attn_bwd_ex(const void* q, int q_row, int q_hs, const void* k1, int k1_row, int k1_hs, int k1_off,
                                int k1_chunks, const void* k2, int k2_row, int k2_hs, int k2_off, const void* v,
                                int v_row, int v_hs, int v_off, const void* o, const void* d_o, const float* lse,
                                float* delta, void* dq, void* dk1, void* dk2, void* dv, const int* out_addr, int B,
                                int S, int Hq, int Hkv, int Dqk, int Dv, int window, float scale, void* status,
                                cudaStream_t st) {
  return nmoe_attn_bwd_masked(q, q_row, q_hs, k1, k1_row, k1_hs, k1_off, k1_chunks, k2, k2_row, k2_hs, k2_off, v, v_row,
                              v_hs, v_off, o, d_o, lse, delta, dq, dk1, dk2, dv, out_addr, nullptr, nullptr, B, S, Hq,
                              Hkv, Dqk, Dv, window, scale, status, st);
}

extern "C" int nmoe_attn_bwd_masked(const void* q, int q_row, int q_hs, const void* k1, int k1_row, int k1_hs, int k1_off,
                                    int k1_chunks, const void* k2, int k2_row, int k2_hs, int k2_off, const void* v,
                                    int v_row, int v_hs, int v_off, const void* o, const void* d_o, const float* lse,
                                    float* delta, void* dq, void* dk1, void* dk2, void* dv, const int* out_addr,
                                    const void* mask, const void* mask_t, int B, int S, int Hq, int Hkv, int Dqk, int Dv,
                                    int window, float scale, void* status, cudaStream_t st) {
  if (B == 0 || S == 0) return 0;
  if ((mask == nullptr) != (mask_t == nullptr)) return -4;
  if (Hq % Hkv != 0) return -1;
  if ((q_row | k1_row | k2_row | v_row) % 8 != 0) return -3;
  for (int i = 0; i < 11; ++i)
    if (out_addr[i] % 8 != 0) return -3;
  AttnBwdParams p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.window = window;
  p.q_hs = q_hs; p.k1_hs = k1_hs; p.k1_off = k1_off; p.k1_chunks = k1_chunks; p.k2_hs = k2_hs; p.k2_off = k2_off;
  p.v_hs = v_hs; p.v_off = v_off; p.do_hs = Dv;
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  p.lse = lse; p.delta = delta;
  p.mask = static_cast<const uint32_t*>(mask); p.mask_t = static_cast<const uint32_t*>(mask_t);
  p.mask_words = 2 * ((S + 63) / 64);
  p.dQ = static_cast<__nv_bfloat16*>(dq); p.dq_row = out_addr[0]; p.dq_hs = out_addr[1];
  p.dK1 = static_cast<__nv_bfloat16*>(dk1); p.dk1_row = out_addr[2]; p.dk1_hs = out_addr[3]; p.dk1_off = out_addr[4];
  p.dK2 = static_cast<__nv_bfloat16*>(dk2 ? dk2 : dk1); p.dk2_row = out_addr[5]; p.dk2_hs = out_addr[6]; p.dk2_off = out_addr[7];
  p.dV = static_cast<__nv_bfloat16*>(dv); p.dv_row = out_addr[8]; p.dv_hs = out_addr[9]; p.dv_off = out_addr[10];
  p.status = static_cast<StatusRecord*>(status);
  const long long n_rows = static_cast<long long>(B) * S * Hq;
  const long long n_thr = n_rows * (Dv / 8);
  k_attn_delta<<<static_cast<unsigned>((n_thr + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, B, S, Hq, Dv);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  BwdOperands a{q, k1, k2, v, d_o, q_row, k1_row, k2_row, v_row, Hq * Dv};
  if (Dqk == 192 && Dv == 128) return attn_bwd_launch<192, 128>(a, p, st);
  if (Dqk == 128 && Dv == 128) return attn_bwd_launch<128, 128>(a, p, st);
  if (Dqk == 64 && Dv == 64) return attn_bwd_launch<64, 64>(a, p, st);
  return -2;
}
