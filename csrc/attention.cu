// Causal softmax attention forward on tcgen05: S = Q K^T and O += P V both run on the tensor
// cores with accumulators in tensor memory; P never touches shared memory (the softmax warps
// write it back into the S columns as bf16 and the second MMA reads its A operand from tensor
// memory).  Covers MLA (d_qk 192, d_v 128), sliding-window attention (band mask), learned
// per-head sinks (a logit that only enters the denominator) and grouped-query heads, and
// returns the log-sum-exp per row for the backward.
//
// One CTA = one 128-row query tile of one (batch, head).  Warp 0 feeds K/V tiles with TMA
// (2 stages each), warp 1 issues the MMAs (S for block i+1 is issued before P V of block i so the
// tensor core works while the softmax warps exponentiate), warps 2-5 own one 32-row quadrant
// each.  The running maximum is only raised when it grows by more than 2^8 (then O is rescaled in
// tensor memory); otherwise the stale maximum is kept, which is exact after the final division.
//
// Replaces FlashAttention-4's forward (nmoe/attention/mla.py:71-91) and the Triton SWA forward
// (nmoe/triton/swa.py:24-121) of the reference.
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

constexpr int kAttnThreads = 320;   // warp 0: TMA, warp 1: MMA, warps 2-9: softmax (two query tiles x four quadrants)
constexpr int ATT_BM = 128;         // query rows per tile
constexpr int ATT_TILES = 2;        // query tiles per CTA, sharing every K/V block that is loaded
constexpr int ATT_BN = 64;          // keys per block
constexpr uint64_t kAttnWaitNs = 2000000000ull;
constexpr float kRescaleThreshold = 8.f;   // log2 units

struct AttnParams {
  int B, S, Hq, Hkv, Dqk, Dv, window;
  // column (element) addressing of the operands inside their 2-D [B*S, row_elems] views:
  // head h of Q starts at h*q_hs; K chunk c (64 columns) comes from source 1 while c < k1_chunks
  // (column hkv*k1_hs + k1_off + c*64) and from source 2 afterwards (hkv*k2_hs + k2_off + (c-k1_chunks)*64);
  // V starts at hkv*v_hs + v_off.  This lets MLA read k_nope and v straight out of the fused kv
  // projection and the shared rotary key from its own tensor without materialising K or V.
  int q_hs, k1_hs, k1_off, k1_chunks, k2_hs, k2_off, v_hs, v_off;
  float scale_log2;
  const float* sinks;
  // optional token-level sparsity: bit k of word row (b*S + q)*mask_words + k/32 set = query q may attend key k
  // (ANDed with the causal / window rule); shared by all heads.  mask_words = 2 * ceil(S / 64).
  const uint32_t* mask;
  int mask_words;
  __nv_bfloat16* O;
  float* lse;
  StatusRecord* status;
};

NMOE_DEVICE uint64_t attn_timer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
NMOE_DEVICE bool attn_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = attn_timer();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 255u) == 0) {
      if (*abort_flag) return false;
      if (attn_timer() - t0 > kAttnWaitNs) return false;
    }
  }
  return true;
}
// D[tmem] (+)= A[tmem] * B[smem desc]
NMOE_DEVICE void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
NMOE_DEVICE void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
NMOE_DEVICE float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DQK, int DV>
struct AttnSmem {
  static constexpr int kQTile = ATT_BM * DQK * 2;
  static constexpr int kQ = ATT_TILES * kQTile;
  static constexpr int kK = ATT_BN * DQK * 2;
  static constexpr int kV = ATT_BN * DV * 2;
  static constexpr int kBytes = kQ + 2 * kK + 2 * kV + 1024 + 256;
};

struct TileRange { int q0, kb_start, kb_end; };

NMOE_DEVICE TileRange tile_range(const AttnParams& p, int q0) {
  TileRange r;
  r.q0 = q0;
  if (q0 >= p.S) { r.kb_start = 0; r.kb_end = 0; return r; }
  r.kb_end = min((q0 + ATT_BM + ATT_BN - 1) / ATT_BN, (p.S + ATT_BN - 1) / ATT_BN);
  r.kb_start = p.window > 0 ? max(0, (q0 - p.window + 1) / ATT_BN) : 0;
  return r;
}

template <int DQK, int DV>
__global__ void __launch_bounds__(kAttnThreads, 1)
k_attn_fwd(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmK2, const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using SM = AttnSmem<DQK, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + SM::kQ;
  uint8_t* sV = sK + 2 * SM::kK;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + 2 * SM::kV);
  uint64_t* q_full = bars;            // [1]
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* k_empty = bars + 3;       // [2]
  uint64_t* v_full = bars + 5;        // [2]
  uint64_t* v_empty = bars + 7;       // [2]
  uint64_t* s_full = bars + 9;        // [tile][buf]
  uint64_t* p_full = bars + 13;       // [tile][buf]
  uint64_t* pv_done = bars + 17;      // [tile]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first: better tail behaviour under the causal mask
  const int q_blk = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int q0 = q_blk * ATT_BM * ATT_TILES;
  const int hkv = h / (p.Hq / p.Hkv);
  const TileRange tr0 = tile_range(p, q0), tr1 = tile_range(p, q0 + ATT_BM);
  const int lo = tr0.kb_start;                      // tile 0 starts no later and ends no later than tile 1
  const int hi = max(tr0.kb_end, tr1.kb_end);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 4; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); }
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA loads
    if (elect_one()) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmK2); tma_prefetch_desc(&tmV);
      const int row_q = b * p.S + q0;
      mbar_expect_tx(q_full, SM::kQ);
#pragma unroll
      for (int t = 0; t < ATT_TILES; ++t)
#pragma unroll
        for (int c = 0; c < DQK / 64; ++c)
          tma_load_2d(sQ + t * SM::kQTile + c * (ATT_BM * 128), &tmQ, q_full, h * p.q_hs + c * 64, row_q + t * ATT_BM);
      for (int i = lo; i < hi; ++i) {
        const int gi = i - lo, st = gi & 1;
        const uint32_t ph = (gi >> 1) & 1;
        const int row_k = b * p.S + i * ATT_BN;
        if (!attn_wait(&k_empty[st], ph ^ 1, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 700, i, 0); *abort_flag = 1; break; }
        mbar_expect_tx(&k_full[st], SM::kK);
#pragma unroll
        for (int c = 0; c < DQK / 64; ++c) {
          if (c < p.k1_chunks)
            tma_load_2d(sK + st * SM::kK + c * (ATT_BN * 128), &tmK, &k_full[st], hkv * p.k1_hs + p.k1_off + c * 64, row_k);
          else
            tma_load_2d(sK + st * SM::kK + c * (ATT_BN * 128), &tmK2, &k_full[st],
                        hkv * p.k2_hs + p.k2_off + (c - p.k1_chunks) * 64, row_k);
        }
        if (!attn_wait(&v_empty[st], ph ^ 1, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 701, i, 0); *abort_flag = 1; break; }
        mbar_expect_tx(&v_full[st], SM::kV);
#pragma unroll
        for (int c = 0; c < DV / 64; ++c)
          tma_load_2d(sV + st * SM::kV + c * (ATT_BN * 128), &tmV, &v_full[st], hkv * p.v_hs + p.v_off + c * 64, row_k);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issue
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(ATT_BM, DV, 0, 1);
      const TileRange trs[2] = {tr0, tr1};
      bool ok = hi > lo && attn_wait(q_full, 0, abort_flag);
      // S = Q_t K_i^T for both tiles that see block i; releases the K stage afterwards
      auto issue_s = [&](int i) -> bool {
        const int gi = i - lo, st = gi & 1;
        if (!attn_wait(&k_full[st], (gi >> 1) & 1, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 710, i, 0); *abort_flag = 1; return false; }
        tc_fence_after_sync();
        const uint32_t ka = smem_u32(sK + st * SM::kK);
#pragma unroll
        for (int t = 0; t < ATT_TILES; ++t) {
          if (i < trs[t].kb_start || i >= trs[t].kb_end) continue;
          const int li = i - trs[t].kb_start;
          const uint32_t qa = smem_u32(sQ + t * SM::kQTile);
          const uint32_t d = tmem_base + t * 128 + (li & 1) * ATT_BN;
#pragma unroll
          for (int j = 0; j < DQK / 16; ++j)
            mma_f16_ss(d, make_smem_desc(qa + (j >> 2) * (ATT_BM * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B),
                       make_smem_desc(ka + (j >> 2) * (ATT_BN * 128) + (j & 3) * 32, 0, 1024, kSwizzle128B), idesc_s,
                       j != 0 ? 1u : 0u);
          mma_commit(&s_full[t * 2 + (li & 1)]);
        }
        mma_commit(&k_empty[st]);
        return true;
      };
      if (ok) ok = issue_s(lo);
      for (int i = lo; ok && i < hi; ++i) {
        const int gi = i - lo, st = gi & 1;
        if (i + 1 < hi) { ok = issue_s(i + 1); if (!ok) break; }
        if (!attn_wait(&v_full[st], (gi >> 1) & 1, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 712, i, 0); *abort_flag = 1; break; }
        const uint32_t va = smem_u32(sV + st * SM::kV);
#pragma unroll
        for (int t = 0; t < ATT_TILES; ++t) {
          if (i < trs[t].kb_start || i >= trs[t].kb_end) continue;
          const int li = i - trs[t].kb_start;
          if (!attn_wait(&p_full[t * 2 + (li & 1)], (li >> 1) & 1, abort_flag)) { report_status(p.status, kStatusWaitTimeout, 711, i, t); *abort_flag = 1; ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_t = tmem_base + t * 128 + (li & 1) * ATT_BN;
#pragma unroll
          for (int j = 0; j < ATT_BN / 16; ++j)
            mma_f16_ts(tmem_base + 256 + t * 128, a_t + j * 8, make_smem_desc(va + j * 2048, ATT_BN * 128, 1024, kSwizzle128B),
                       idesc_pv, (li | j) != 0 ? 1u : 0u);
          mma_commit(&pv_done[t]);
        }
        mma_commit(&v_empty[st]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax + epilogue: warp -> (tile, 32-row quadrant)
    const int tile = (warp - 2) >> 2;
    const int q = warp & 3;
    const TileRange tr = tile ? tr1 : tr0;
    const int n_blocks = tr.kb_end - tr.kb_start;
    const int row = tr.q0 + q * 32 + lane;           // query position inside the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t tmem_o = tmem_base + 256 + tile * 128;
    float m = -1e30f, l = 0.f;
    if (p.sinks != nullptr) { m = p.sinks[h] * 1.4426950408889634f; l = 1.f; }
    bool ok = true;
    for (int i = 0; i < n_blocks; ++i) {
      const int bf = i & 1;
      const uint32_t s_addr = tmem_base + lane_addr + tile * 128 + bf * ATT_BN;
      ok = attn_wait(&s_full[tile * 2 + bf], (i >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 720, i, tile); *abort_flag = 1; break; }
      tc_fence_after_sync();
      const int k0 = (tr.kb_start + i) * ATT_BN;
      const bool need_mask = (k0 + ATT_BN - 1 > tr.q0) || (p.window > 0 && k0 <= tr.q0 + ATT_BM - 1 - p.window) || (k0 + ATT_BN > p.S);
      uint32_t r[ATT_BN];
      tmem_ld_32x32b_x32(s_addr, r);
      tmem_ld_32x32b_x32(s_addr + 32, r + 32);
      uint32_t mw0 = 0xffffffffu, mw1 = 0xffffffffu;
      if (p.mask != nullptr) {
        if (row < p.S) {
          const uint32_t* mr = p.mask + (static_cast<size_t>(b) * p.S + row) * p.mask_words + (k0 >> 5);
          mw0 = __ldg(mr); mw1 = __ldg(mr + 1);
        } else {
          mw0 = mw1 = 0u;
        }
      }
      tmem_ld_wait();
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int t = 0; t < ATT_BN; ++t) {
          const int j = k0 + t;
          if (j > row || j >= p.S || (p.window > 0 && j <= row - p.window)) r[t] = 0xff800000u;   // -inf
        }
      }
      if (p.mask != nullptr) {
#pragma unroll
        for (int t = 0; t < ATT_BN; ++t)
          if (!(((t < 32 ? mw0 : mw1) >> (t & 31)) & 1u)) r[t] = 0xff800000u;
      }
#pragma unroll
      for (int t = 0; t < ATT_BN; ++t) mx = fmaxf(mx, __uint_as_float(r[t]));
      const float m_cand = fmaxf(m, mx * p.scale_log2);
      bool grow = (m_cand - m > kRescaleThreshold);
      if (i == 0) { grow = false; if (m_cand > m) { l *= fast_exp2(m - m_cand); m = m_cand; } }
      if (__any_sync(0xffffffffu, grow)) {
        // O must be final for block i-1 before it is rescaled
        ok = attn_wait(&pv_done[tile], (i - 1) & 1, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 721, i, tile); *abort_flag = 1; break; }
        tc_fence_after_sync();
        float alpha = 1.f;
        if (grow) { alpha = fast_exp2(m - m_cand); m = m_cand; l *= alpha; }
#pragma unroll 1
        for (int c = 0; c < DV / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_o + lane_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t) o[t] = __float_as_uint(__uint_as_float(o[t]) * alpha);
          tmem_st_32x32b_x32(tmem_o + lane_addr + c * 32, o);
        }
        tmem_st_wait();
      }
      // P = 2^(s*scale - m) as bf16 pairs, written over the first 32 columns of this S buffer
      float rs = 0.f;
      uint32_t pk[ATT_BN / 2];
#pragma unroll
      for (int t = 0; t < ATT_BN; t += 2) {
        const float p0 = fast_exp2(fmaf(__uint_as_float(r[t]), p.scale_log2, -m));
        const float p1 = fast_exp2(fmaf(__uint_as_float(r[t + 1]), p.scale_log2, -m));
        rs += p0 + p1;
        pk[t >> 1] = pack_bf16x2(p0, p1);
      }
      l += rs;
      tmem_st_32x32b_x16(s_addr, pk);
      tmem_st_32x32b_x16(s_addr + 16, pk + 16);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[tile * 2 + bf]);
    }
    // epilogue
    if (ok && n_blocks > 0) {
      ok = attn_wait(&pv_done[tile], (n_blocks - 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) { if (lane == 0) report_status(p.status, kStatusWaitTimeout, 722, 0, tile); *abort_flag = 1; }
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = row < p.S;
      __nv_bfloat16* orow = p.O + (static_cast<size_t>(b) * p.S + row) * (static_cast<size_t>(p.Hq) * DV) + static_cast<size_t>(h) * DV;
#pragma unroll 1
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t o[32];
        if (n_blocks > 0) {
          tmem_ld_32x32b_x32(tmem_o + lane_addr + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) o[t] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            int4 v;
            v.x = pack_bf16x2(__uint_as_float(o[8 * t]) * inv_l, __uint_as_float(o[8 * t + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(o[8 * t + 2]) * inv_l, __uint_as_float(o[8 * t + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(o[8 * t + 4]) * inv_l, __uint_as_float(o[8 * t + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(o[8 * t + 6]) * inv_l, __uint_as_float(o[8 * t + 7]) * inv_l);
            reinterpret_cast<int4*>(orow + c * 32)[t] = v;
          }
        }
      }
      if (row_ok && p.lse != nullptr)
        p.lse[(static_cast<size_t>(b) * p.Hq + h) * p.S + row] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
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

static int attn_map(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
                    uint32_t box_rows) {
  using Key = std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  Key k{base, inner, outer, pitch_bytes, box_rows};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(k);
  if (it != cache.end()) { *out = it->second; return 0; }
  int rc = make_tensor_map_2d(out, base, kTmaBf16, inner, outer, pitch_bytes, 64, box_rows, kTmaSwizzle128);
  if (rc != 0) return rc;
  if (cache.size() > 1024) cache.clear();
  cache[k] = *out;
  return 0;
}

template <int DQK, int DV>
static int attn_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tk2, const CUtensorMap& tv,
                       const AttnParams& p, cudaStream_t st) {
  auto kern = k_attn_fwd<DQK, DV>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<DQK, DV>::kBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid((p.S + ATT_BM * ATT_TILES - 1) / (ATT_BM * ATT_TILES), p.Hq, p.B);
  kern<<<grid, kAttnThreads, AttnSmem<DQK, DV>::kBytes, st>>>(tq, tk, tk2, tv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace nmoe

using namespace nmoe;

// General form.  Every operand is a bf16 matrix with B*S rows; *_row is its row length in elements
// (a multiple of 8) and the *_hs / *_off arguments place a head's columns inside a row (see AttnParams).
// o [B,S,Hq,Dv] contiguous; lse [B,Hq,S] fp32 (optional); sinks [Hq] fp32 raw logits (optional);
// window 0 = full causal.  Supported head dims (Dqk, Dv): (192,128), (128,128), (64,64).
// mask: optional [B, S, 2*ceil(S/64)] uint32 bit rows (see AttnParams), shared by all heads.
extern "C" int nmoe_attn_fwd_masked(const void* q, int q_row, int q_hs, const void* k1, int k1_row, int k1_hs, int k1_off,
                                    int k1_chunks, const void* k2, int k2_row, int k2_hs, int k2_off, const void* v,
                                    int v_row, int v_hs, int v_off, void* o, float* lse, const float* sinks,
                                    const void* mask, int B, int S, int Hq, int Hkv, int Dqk, int Dv, int window,
                                    float scale, void* status, cudaStream_t st);

extern "C" int nmoe_attn_fwd_ex(const void* q, int q_row, int q_hs, const void* k1, int k1_row, int k1_hs, int k1_off,
                                int k1_chunks, const void* k2, int k2_row, int k2_hs, int k2_off, const void* v,
                                int v_row, int v_hs, int v_off, void* o, float* lse, const float* sinks, int B, int S,
                                int Hq, int Hkv, int Dqk, int Dv, int window, float scale, void* status,
                                cudaStream_t st) {
  return nmoe_attn_fwd_masked(q, q_row, q_hs, k1, k1_row, k1_hs, k1_off, k1_chunks, k2, k2_row, k2_hs, k2_off, v, v_row,
                              v_hs, v_off, o, lse, sinks, nullptr, B, S, Hq, Hkv, Dqk, Dv, window, scale, status, st);
}

extern "C" int nmoe_attn_fwd_masked(const void* q, int q_row, int q_hs, const void* k1, int k1_row, int k1_hs, int k1_off,
                                    int k1_chunks, const void* k2, int k2_row, int k2_hs, int k2_off, const void* v,
                                    int v_row, int v_hs, int v_off, void* o, float* lse, const float* sinks,
                                    const void* mask, int B, int S, int Hq, int Hkv, int Dqk, int Dv, int window,
                                    float scale, void* status, cudaStream_t st) {
  if (B == 0 || S == 0) return 0;
  if (Hq % Hkv != 0) return -1;
  if ((q_row | k1_row | k2_row | v_row) % 8 != 0) return -3;
  AttnParams p;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.Dqk = Dqk; p.Dv = Dv; p.window = window;
  p.q_hs = q_hs; p.k1_hs = k1_hs; p.k1_off = k1_off; p.k1_chunks = k1_chunks; p.k2_hs = k2_hs; p.k2_off = k2_off;
  p.v_hs = v_hs; p.v_off = v_off;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.sinks = sinks; p.O = static_cast<__nv_bfloat16*>(o); p.lse = lse; p.status = static_cast<StatusRecord*>(status);
  p.mask = static_cast<const uint32_t*>(mask); p.mask_words = 2 * ((S + 63) / 64);
  CUtensorMap tq, tk, tk2, tv;
  const uint64_t rows = static_cast<uint64_t>(B) * S;
  int rc = attn_map(&tq, q, q_row, rows, static_cast<uint64_t>(q_row) * 2, ATT_BM);
  if (rc) return rc;
  rc = attn_map(&tk, k1, k1_row, rows, static_cast<uint64_t>(k1_row) * 2, ATT_BN);
  if (rc) return rc;
  rc = attn_map(&tk2, k2 ? k2 : k1, k2 ? k2_row : k1_row, rows, static_cast<uint64_t>(k2 ? k2_row : k1_row) * 2, ATT_BN);
  if (rc) return rc;
  rc = attn_map(&tv, v, v_row, rows, static_cast<uint64_t>(v_row) * 2, ATT_BN);
  if (rc) return rc;
  if (Dqk == 192 && Dv == 128) return attn_launch<192, 128>(tq, tk, tk2, tv, p, st);
  if (Dqk == 128 && Dv == 128) return attn_launch<128, 128>(tq, tk, tk2, tv, p, st);
  if (Dqk == 64 && Dv == 64) return attn_launch<64, 64>(tq, tk, tk2, tv, p, st);
  return -2;
}

// q [B,S,Hq,Dqk], k [B,S,Hkv,Dqk], v [B,S,Hkv,Dv] contiguous.
extern "C" int nmoe_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const float* sinks,
                             int B, int S, int Hq, int Hkv, int Dqk, int Dv, int window, float scale, void* status,
                             cudaStream_t st) {
  return nmoe_attn_fwd_ex(q, Hq * Dqk, Dqk, k, Hkv * Dqk, Dqk, 0, Dqk / 64, nullptr, 0, 0, 0, v, Hkv * Dv, Dv, 0, o, lse,
                          sinks, B, S, Hq, Hkv, Dqk, Dv, window, scale, status, st);
}
