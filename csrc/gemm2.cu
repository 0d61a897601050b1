// Two-SM variant of the bf16 tcgen05 GEMM: a pair of CTAs (a 2-CTA cluster on neighbouring SMs)
// computes one 256 x 256 output tile with `tcgen05.mma.cta_group::2`.  Each CTA loads only ITS
// 128 rows of A and ITS 128 columns of B per K step (32 KB instead of the 48 KB a lone CTA needs
// for a 128 x 256 tile), so shared-memory fill per FLOP drops by a third and six pipeline stages
// fit.  The even CTA of the pair issues every MMA; both CTAs own the 128 accumulator rows that
// live in their tensor memory and run their own epilogue.  Loads are plain per-CTA TMA copies
// (nothing is broadcast across the cluster); the odd CTA's copies complete on the even CTA's
// mbarrier, pipeline slots are released to both CTAs by the MMA commit.
//
// Same modes and operand majors as gemm.cu.  Mode 1 (ragged rows per expert) needs 256-row-aligned
// segments, because the two CTAs of a pair share one B operand.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common/epilogue.cuh"
#include "common/ptx.cuh"
#include "common/tensormap.h"

namespace nmoe {

constexpr int G2_BM = 128;             // rows per CTA (256 per pair)
constexpr int G2_BK = 64;
constexpr int G2_BN = 256;             // columns per pair; each CTA loads G2_BN / 2 of B
constexpr int kG2Threads = 192;
constexpr int kG2Stages = 6;
constexpr int kG2GroupM = 8;           // 256-row tiles per rasterisation group
constexpr uint64_t kG2WaitNs = 2000000000ull;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;   // clears the CTA-rank bit of a shared::cluster address

struct Gemm2Params {
  int M, N, K, E;
  const int* tile_expert;
  const int* n_m_tiles;        // mode 1: number of valid 128-row tiles (even)
  const int* offs;
  void* C;
  long long ldc;
  int out_fp32, accumulate;
  long long b_rows_per_expert;
  StatusRecord* status;
  // fused RDEP return (mode 1, bf16): see GemmParams in gemm.cu
  const int* push_runs;        // [3][E][world] return-run tables from nmoe_rdep_plan (non-null selects the fused return)
  __nv_bfloat16* peer_ret[8];
  float* peer_retg[8];
  const float* rowval;
  int push_world, push_pairs;  // ranks in the run tables; rows of a source's return buffer (bound)
  int push_bulk;               // 1: the fused return hands 256-byte row segments to the bulk-copy unit
  SwigluBwdEpi sb;             // mode 1: SwiGLU backward in the epilogue (sb.h13 != nullptr); C is not written
};

NMOE_DEVICE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
NMOE_DEVICE uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
NMOE_DEVICE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
NMOE_DEVICE void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Per-CTA tiled copy whose completion bytes are credited to the barrier of the pair's even CTA.
NMOE_DEVICE void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t leader_bar, int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
NMOE_DEVICE void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of `mask` once the MMAs issued so far are done.
NMOE_DEVICE void mma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}
NMOE_DEVICE void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
NMOE_DEVICE void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
NMOE_DEVICE void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
NMOE_DEVICE uint64_t g2_timer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
NMOE_DEVICE bool g2_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = g2_timer();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 255u) == 0) {
      if (*abort_flag) return false;
      if (g2_timer() - t0 > kG2WaitNs) return false;
    }
  }
  return true;
}

struct Tile2 { int m_blk, n_blk, expert, kb_begin, kb_count; };

template <int MODE>
NMOE_DEVICE bool decode_tile2(const Gemm2Params& p, int t, int m_tiles, int n_tiles, Tile2& tc) {
  if (MODE == 2) {
    const int per_e = m_tiles * n_tiles;
    const int e = t / per_e;
    if (e >= p.E) return false;
    const int r = t - e * per_e;
    tc.expert = e;
    tc.m_blk = r % m_tiles;
    tc.n_blk = r / m_tiles;
    const int r0 = p.offs[e], r1 = p.offs[e + 1];
    tc.kb_begin = r0 / G2_BK;
    tc.kb_count = (r1 - r0) / G2_BK;
    return true;
  }
  if (t >= m_tiles * n_tiles) return false;
  const int per_group = kG2GroupM * n_tiles;
  const int g = t / per_group;
  const int first_m = g * kG2GroupM;
  const int gm = min(kG2GroupM, m_tiles - first_m);
  const int r = t - g * per_group;
  tc.m_blk = first_m + r % gm;
  tc.n_blk = r / gm;
  tc.expert = (MODE == 1) ? p.tile_expert[2 * tc.m_blk] : 0;
  tc.kb_begin = 0;
  tc.kb_count = (p.K + G2_BK - 1) / G2_BK;
  return true;
}

constexpr int kG2StageA = G2_BM * G2_BK * 2;
constexpr int kG2StageB = (G2_BN / 2) * G2_BK * 2;
// staging of the fused-return epilogue: bulk copies of 256-byte row segments (or the 4 KB transposing store)
constexpr int kG2EpiWarp = EpiBulk<256>::kWarpBytes > kEpiStageBytesPerWarp ? EpiBulk<256>::kWarpBytes : kEpiStageBytesPerWarp;
constexpr int kG2EpiStage = 4 * kG2EpiWarp;
constexpr int kG2SmemBytes = kG2Stages * (kG2StageA + kG2StageB) + kG2EpiStage + 1024 + 256;
static_assert(kG2SmemBytes <= 232448, "shared memory budget");

template <bool A_MN, bool B_MN, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kG2Threads, 1)
k_gemm_bf16_pair(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kG2Stages * kG2StageA;
  uint8_t* epi_stage = smem + kG2Stages * (kG2StageA + kG2StageB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + kG2EpiStage);
  uint64_t* full = bars;
  uint64_t* empty = bars + kG2Stages;
  uint64_t* tmem_full = bars + 2 * kG2Stages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

  int m_tiles;
  if (MODE == 1) m_tiles = min(*p.n_m_tiles / 2, (p.M + 2 * G2_BM - 1) / (2 * G2_BM));
  else m_tiles = (p.M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int n_tiles = (p.N + G2_BN - 1) / G2_BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kG2Stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 8); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();                 // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      Tile2 tc;
      bool ok = true;
      for (int t = cluster_id; ok && decode_tile2<MODE>(p, t, m_tiles, n_tiles, tc); t += n_clusters) {
        const int m0 = tc.m_blk * 2 * G2_BM + static_cast<int>(rank) * G2_BM;
        const int n0 = tc.n_blk * G2_BN + static_cast<int>(rank) * (G2_BN / 2);
        for (int kb = 0; kb < tc.kb_count; ++kb) {
          if (!g2_wait(&empty[stage], phase ^ 1, abort_flag)) {
            report_status(p.status, kStatusWaitTimeout, 800, stage, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t lbar = smem_u32(&full[stage]) & kPeerBitMask;
          if (leader) mbar_expect_tx(&full[stage], 2 * (kG2StageA + kG2StageB));
          const int k0 = (tc.kb_begin + kb) * G2_BK;
          uint8_t* a_dst = sA + stage * kG2StageA;
          uint8_t* b_dst = sB + stage * kG2StageB;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < G2_BM / 64; ++c) tma_load_2d_pair(a_dst + c * (G2_BK * 128), &tmA, lbar, m0 + c * 64, k0);
          } else {
            tma_load_2d_pair(a_dst, &tmA, lbar, k0, m0);
          }
          if (B_MN) {
            const int krow = (MODE == 1) ? static_cast<int>(tc.expert * p.b_rows_per_expert) + k0 : k0;
#pragma unroll
            for (int c = 0; c < G2_BN / 2 / 64; ++c) tma_load_2d_pair(b_dst + c * (G2_BK * 128), &tmB, lbar, n0 + c * 64, krow);
          } else {
            const int nrow = (MODE == 1) ? static_cast<int>(tc.expert * p.b_rows_per_expert) + n0 : n0;
            tma_load_2d_pair(b_dst, &tmB, lbar, k0, nrow);
          }
          if (++stage == kG2Stages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (leader && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * G2_BM, G2_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      Tile2 tc;
      bool ok = true;
      for (int t = cluster_id; ok && decode_tile2<MODE>(p, t, m_tiles, n_tiles, tc); t += n_clusters) {
        if (tc.kb_count == 0) continue;
        if (!g2_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          report_status(p.status, kStatusWaitTimeout, 810, acc, t);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * G2_BN;
        for (int kb = 0; kb < tc.kb_count; ++kb) {
          if (!g2_wait(&full[stage], phase, abort_flag)) {
            report_status(p.status, kStatusWaitTimeout, 811, stage, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * kG2StageA);
          const uint32_t b_addr = smem_u32(sB + stage * kG2StageB);
#pragma unroll
          for (int j = 0; j < G2_BK / 16; ++j) {
            const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + j * 2048, G2_BK * 128, 1024, kSwizzle128B)
                                         : make_smem_desc(a_addr + j * 32, 0, 1024, kSwizzle128B);
            const uint64_t b_desc = B_MN ? make_smem_desc(b_addr + j * 2048, G2_BK * 128, 1024, kSwizzle128B)
                                         : make_smem_desc(b_addr + j * 32, 0, 1024, kSwizzle128B);
            mma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0 ? 1u : 0u);
          }
          mma_commit_pair(&empty[stage], 3);
          if (++stage == kG2Stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit_pair(&tmem_full[acc], 3);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    Tile2 tc;
    const int m_limit = (MODE == 1) ? m_tiles * 2 * G2_BM : p.M;
    const uint32_t leader_empty0 = mapa_shared(smem_u32(&tmem_empty[0]), 0);
    bool used_bulk = false;
    for (int t = cluster_id; decode_tile2<MODE>(p, t, m_tiles, n_tiles, tc); t += n_clusters) {
      const int row = tc.m_blk * 2 * G2_BM + static_cast<int>(rank) * G2_BM + q * 32 + lane;
      const int n0 = tc.n_blk * G2_BN;
      bool row_ok = row < m_limit;
      const long long crow = (MODE == 2) ? static_cast<long long>(tc.expert) * p.M + row : row;
      const bool have_acc = tc.kb_count > 0;
      __nv_bfloat16* push_dst = nullptr;
      float push_gate = 1.f;
      if (MODE == 1 && p.push_runs != nullptr && row_ok) {
        int src = 0, drow = 0;
        row_ok = run_lookup(p.push_runs, p.E, p.push_world, tc.expert, row, src, drow) && drow >= 0 && drow < p.push_pairs &&
                 p.peer_ret[src & 7] != nullptr;
        if (row_ok) {
          push_dst = p.peer_ret[src] + static_cast<long long>(drow) * p.ldc;
          if (tc.n_blk == 0 && p.rowval != nullptr) p.peer_retg[src][drow] = p.rowval[row];
        }
      }
      if (have_acc) {
        bool ok = g2_wait(&tmem_full[acc], acc_phase, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report_status(p.status, kStatusWaitTimeout, 820, acc, t);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
      }
      if (MODE == 1 && p.sb.h13 != nullptr && have_acc) {
        // SwiGLU backward in the epilogue: the accumulator is dA; dh13 and the scaled activation leave, dA does not
        const float sc = (row_ok && p.sb.row_scale != nullptr) ? p.sb.row_scale[row] : 1.f;
        const long long row0 = static_cast<long long>(row - lane);           // first row of this warp's 32-row slab
        const int rows_ok = max(0, min(32, m_limit - static_cast<int>(row0)));
        uint8_t* t0 = epi_stage + (warp - 2) * kG2EpiWarp;
        uint8_t* t1 = t0 + 4096;
        float dot = 0.f;
        int4 g[8];
        if (n0 < p.N) {
          sb_issue_loads(g, p.sb.h13, row0, rows_ok, 2LL * p.N, n0, lane);
          sb_stage_h(t0, g, lane);
          __syncwarp();
        }
#pragma unroll 1
        for (int c = 0; c < G2_BN / 32; ++c) {
          const int col = n0 + c * 32;
          if (col >= p.N) break;               // uniform over the warp
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * G2_BN + c * 32, r);
          const bool more = col + 32 < p.N && c + 1 < G2_BN / 32;
          if (more) sb_issue_loads(g, p.sb.h13, row0, rows_ok, 2LL * p.N, col + 32, lane);   // in flight during this chunk
          tmem_ld_wait();
          swiglu_bwd_cols32(r, t0, t1, p.sb.dh13, p.sb.a_out, row0, rows_ok, p.N, col, sc, dot, lane);
          if (more) {
            sb_stage_h(t0, g, lane);
            __syncwarp();
          }
        }
        if (row_ok && p.sb.rowdot_parts != nullptr) p.sb.rowdot_parts[static_cast<long long>(tc.n_blk) * p.sb.rows_cap + row] = dot;
      } else
      if (MODE == 1 && p.push_runs != nullptr && have_acc && p.push_bulk && (p.N & 127) == 0 && (p.ldc & 7) == 0) {
        // fused return through the copy unit: 128 columns (256 bytes) of this lane's row per bulk copy
        uint8_t* srow = EpiBulk<256>::row(epi_stage + (warp - 2) * kG2EpiWarp, lane);
        __nv_bfloat16* dst0 = (row_ok && push_dst != nullptr) ? push_dst : nullptr;
#pragma unroll 1
        for (int c = 0; c < G2_BN / 64; ++c) {
          const int col = n0 + c * 64;
          if (col >= p.N) break;
          uint32_t r[64];
          const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * G2_BN + c * 64;
          tmem_ld_32x32b_x32(ta, r);
          tmem_ld_32x32b_x32(ta + 32, r + 32);
          if ((c & 1) == 0) epi_bulk_wait_read();
          tmem_ld_wait();
          stage_64cols(srow, (c & 1) * 128, r, push_gate);
          if (c & 1) {
            epi_bulk_fence();
            epi_bulk_store(dst0 ? dst0 + (col - 64) : nullptr, srow, 256);
          }
        }
        used_bulk = true;
      } else if (MODE == 1 && p.push_runs != nullptr && have_acc) {
        // fused return, coalesced: 64 columns (128 bytes) of 4 rows per store instruction
        uint8_t* stage = epi_stage + (warp - 2) * kG2EpiWarp;
#pragma unroll 1
        for (int c = 0; c < G2_BN / 64; ++c) {
          const int col = n0 + c * 64;
          if (col >= p.N) break;
          uint32_t r[64];
          const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * G2_BN + c * 64;
          tmem_ld_32x32b_x32(ta, r);
          tmem_ld_32x32b_x32(ta + 32, r + 32);
          tmem_ld_wait();
          warp_store_rows_64cols(stage, r, push_gate, (row_ok && push_dst != nullptr) ? push_dst + col : nullptr, lane);
        }
      } else
#pragma unroll 1
      for (int c = 0; c < G2_BN / 32; ++c) {
        uint32_t r[32];
        if (have_acc) {
          tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * G2_BN + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        const int col = n0 + c * 32;
        if (row_ok && col < p.N) {
          if (p.out_fp32) {
            float* dst = static_cast<float*>(p.C) + crow * p.ldc + col;
            if (col + 32 <= p.N) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                       __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
                if (p.accumulate) {
                  float4 o = reinterpret_cast<float4*>(dst)[i];
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                reinterpret_cast<float4*>(dst)[i] = v;
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i) dst[i] = __uint_as_float(r[i]) + (p.accumulate ? dst[i] : 0.f);
            }
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.C) + crow * p.ldc + col;
            if (col + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * i + j]);
                if (p.accumulate) {
                  int4 o = reinterpret_cast<int4*>(dst)[i];
                  float2 o0 = unpack_bf16x2(o.x), o1 = unpack_bf16x2(o.y), o2 = unpack_bf16x2(o.z), o3 = unpack_bf16x2(o.w);
                  f[0] += o0.x; f[1] += o0.y; f[2] += o1.x; f[3] += o1.y;
                  f[4] += o2.x; f[5] += o2.y; f[6] += o3.x; f[7] += o3.y;
                }
                int4 v;
                v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
                v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
                reinterpret_cast<int4*>(dst)[i] = v;
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i) {
                float f = __uint_as_float(r[i]);
                if (p.accumulate) f += __bfloat162float(dst[i]);
                dst[i] = __float2bfloat16(f);
              }
            }
          }
        }
      }
      if (have_acc) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_empty0 + acc * 8);     // the even CTA's tmem_empty[acc]
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    if (used_bulk) epi_bulk_drain();         // this lane's row copies have been written before the kernel ends
  }

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (MODE == 1 && p.push_runs != nullptr) __threadfence_system();
  tc_fence_before_sync();
  cluster_sync_all();                 // neither CTA may free tensor memory or exit while its partner still uses the pair
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

static int g2_map(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
                  uint32_t box_inner, uint32_t box_outer) {
  using Key = std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  Key k{base, inner, outer, pitch_bytes, box_inner, box_outer};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(k);
  if (it != cache.end()) { *out = it->second; return 0; }
  int rc = make_tensor_map_2d(out, base, kTmaBf16, inner, outer, pitch_bytes, box_inner, box_outer, kTmaSwizzle128);
  if (rc != 0) return rc;
  if (cache.size() > 4096) cache.clear();
  cache[k] = *out;
  return 0;
}

template <bool A_MN, bool B_MN, int MODE>
static int g2_launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Gemm2Params& p, int max_tiles, cudaStream_t st) {
  auto kern = k_gemm_bf16_pair<A_MN, B_MN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kG2SmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int pairs = sms / 2;
  if (max_tiles < pairs) pairs = max_tiles;
  if (pairs < 1) return 0;
  kern<<<2 * pairs, kG2Threads, kG2SmemBytes, st>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace nmoe

using namespace nmoe;

// Same contract as nmoe_gemm_bf16 including the fused RDEP return (push_runs / peer_ret / peer_retg / rowval);
// N tile is fixed at 256 and grouped row segments must be 256-aligned.
static int g2_go(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                        long long ldb, long long ldc, int a_mn, int b_mn, int mode, int E,
                                        const int* tile_expert, const int* n_m_tiles, const int* offs, long long a_rows,
                                        long long b_rows, int out_fp32, int accumulate, void* status, const void* push_runs,
                                        void* const* peer_ret, void* const* peer_retg, const float* rowval,
                                        int push_pairs, int world, const SwigluBwdEpi* sb, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (push_runs && (mode != 1 || out_fp32 || world > 8 || (N & 63) != 0 || (ldc & 7) != 0)) return -6;
  if (mode != 2 && K <= 0) return -1;
  if ((lda % 8) || (ldb % 8)) return -2;
  if (mode == 2 && !(a_mn && b_mn)) return -3;
  if (mode == 1 && (K % G2_BK) != 0) return -4;
  Gemm2Params p;
  p.M = M; p.N = N; p.K = K; p.E = E; p.tile_expert = tile_expert; p.n_m_tiles = n_m_tiles; p.offs = offs;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.b_rows_per_expert = (mode == 1) ? (b_mn ? K : N) : 0;
  p.status = static_cast<StatusRecord*>(status);
  p.push_runs = static_cast<const int*>(push_runs); p.rowval = rowval; p.push_pairs = push_pairs; p.push_world = world;
  p.push_bulk = epi_push_bulk_enabled();
  p.sb = SwigluBwdEpi{nullptr, nullptr, nullptr, nullptr, nullptr, 0};
  if (sb != nullptr) {
    if (mode != 1 || push_runs != nullptr || (N % 32) != 0) return -7;
    p.sb = *sb;
  }
  for (int r = 0; r < 8; ++r) {
    p.peer_ret[r] = (push_runs && peer_ret && r < world) ? static_cast<__nv_bfloat16*>(peer_ret[r]) : nullptr;
    p.peer_retg[r] = (push_runs && peer_retg && r < world) ? static_cast<float*>(peer_retg[r]) : nullptr;
  }
  CUtensorMap tmA, tmB;
  int rc;
  if (a_mn) rc = g2_map(&tmA, A, static_cast<uint64_t>(M), static_cast<uint64_t>(a_rows), lda * 2, 64, G2_BK);
  else rc = g2_map(&tmA, A, static_cast<uint64_t>(K), static_cast<uint64_t>(a_rows), lda * 2, G2_BK, G2_BM);
  if (rc != 0) return rc;
  if (b_mn) rc = g2_map(&tmB, B, static_cast<uint64_t>(N), static_cast<uint64_t>(b_rows), ldb * 2, 64, G2_BK);
  else rc = g2_map(&tmB, B, static_cast<uint64_t>(K), static_cast<uint64_t>(b_rows), ldb * 2, G2_BK, G2_BN / 2);
  if (rc != 0) return rc;
  const int m_tiles = (M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int n_tiles = (N + G2_BN - 1) / G2_BN;
  const int max_tiles = (mode == 2) ? E * m_tiles * n_tiles : m_tiles * n_tiles;
#define G2_GO(MODE_)                                                                          \
  ((!a_mn && !b_mn)  ? g2_launch<false, false, MODE_>(tmA, tmB, p, max_tiles, st)             \
   : (!a_mn && b_mn) ? g2_launch<false, true, MODE_>(tmA, tmB, p, max_tiles, st)              \
   : (a_mn && b_mn)  ? g2_launch<true, true, MODE_>(tmA, tmB, p, max_tiles, st)               \
                     : g2_launch<true, false, MODE_>(tmA, tmB, p, max_tiles, st))
  if (mode == 0) return G2_GO(0);
  if (mode == 1) return G2_GO(1);
  return g2_launch<true, true, 2>(tmA, tmB, p, max_tiles, st);
#undef G2_GO
}

extern "C" int nmoe_gemm_bf16_pair_push(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                        long long ldb, long long ldc, int a_mn, int b_mn, int mode, int E,
                                        const int* tile_expert, const int* n_m_tiles, const int* offs, long long a_rows,
                                        long long b_rows, int out_fp32, int accumulate, void* status, const void* push_runs,
                                        void* const* peer_ret, void* const* peer_retg, const float* rowval,
                                        int push_pairs, int world, cudaStream_t st) {
  return g2_go(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, E, tile_expert, n_m_tiles, offs, a_rows, b_rows, out_fp32, accumulate, status, push_runs, peer_ret, peer_retg, rowval, push_pairs, world, nullptr, st);
}

// Grouped dA = dY W2^T on CTA pairs whose epilogue is the SwiGLU backward (see SwigluBwdEpi): reads h13 [M, 2N], writes
// dh13 [M, 2N], a_out [M, N] (optional) and rowdot_parts [ceil(N/256), rows_cap] (optional).  N % 32 == 0.
extern "C" int nmoe_gemm_bf16_pair_swiglu_bwd(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                              int b_mn, int E, const int* tile_expert, const int* n_m_tiles, long long a_rows,
                                              long long b_rows, const void* h13, void* dh13, void* a_out,
                                              const float* row_scale, float* rowdot_parts, long long rows_cap, void* status,
                                              cudaStream_t st) {
  if (h13 == nullptr || dh13 == nullptr) return -7;
  SwigluBwdEpi sb{static_cast<const __nv_bfloat16*>(h13), static_cast<__nv_bfloat16*>(dh13), static_cast<__nv_bfloat16*>(a_out),
                  row_scale, rowdot_parts, rows_cap};
  return g2_go(A, B, dh13, M, N, K, lda, ldb, N, 0, b_mn, 1, E, tile_expert, n_m_tiles, nullptr, a_rows, b_rows, 0, 0, status,
               nullptr, nullptr, nullptr, nullptr, 0, 0, &sb, st);
}

// Without the fused-return arguments.
extern "C" int nmoe_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                   long long ldb, long long ldc, int a_mn, int b_mn, int mode, int E,
                                   const int* tile_expert, const int* n_m_tiles, const int* offs, long long a_rows,
                                   long long b_rows, int out_fp32, int accumulate, void* status, cudaStream_t st) {
  return nmoe_gemm_bf16_pair_push(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, E, tile_expert, n_m_tiles, offs, a_rows,
                                  b_rows, out_fp32, accumulate, status, nullptr, nullptr, nullptr, nullptr, 0, 0, st);
}
