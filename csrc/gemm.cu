// bf16 GEMM family on the 5th-generation tensor cores: TMA-fed, tcgen05.mma with the
// accumulator in tensor memory, persistent over output tiles, warp-specialised
// (1 TMA warp, 1 MMA warp, 4 epilogue warps), double-buffered accumulators so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// One kernel template covers everything the trainer needs:
//   mode 0  dense      C[M,N]   = op(A) op(B)         linears, lm_head, dgrad, wgrad
//   mode 1  grouped-M  rows of A/C are 128-aligned per-expert segments, B is per expert
//                      (expert up/gate/down projections and their dgrads)
//   mode 2  grouped-K  C[e]     = A_e^T B_e over the rows of expert e (expert wgrad),
//                      empty experts produce zeros
// Each operand may be K-major or MN-major (transposed in memory); the tensor core reads
// either straight from 128-byte-swizzled shared memory, so no transposes are materialised.
//
// Replaces cuBLAS nn.Linear, torch._grouped_mm (nmoe/moe.py:24-49) and the per-expert
// cuBLASLt wgrad loops (nmoe/csrc/gemm.cu:253-337) of the reference.
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

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = one 128-byte swizzle span
constexpr int kGemmThreads = 192;      // warp 0: TMA, warp 1: MMA, warps 2-5: epilogue
constexpr int kGroupM = 16;            // row tiles per rasterisation group (L2 reuse of B)
constexpr uint64_t kWaitBudgetNs = 2000000000ull;   // every wait gives up after 2 s

struct GemmParams {
  int M, N, K;
  int E;
  const int* tile_expert;      // mode 1: expert id of each 128-row tile
  const int* n_m_tiles;        // mode 1: device scalar, number of valid row tiles
  const int* offs;             // mode 2: [E+1] row offsets (multiples of 128)
  void* C;
  long long ldc;
  int out_fp32;
  int accumulate;              // C += result instead of C = result
  long long b_rows_per_expert; // mode 1: rows of B's 2-D view per expert
  StatusRecord* status;
  // Fused RDEP return (mode 1, bf16 output): when push_runs != nullptr the epilogue does not write C; it stores
  // row r into the SOURCE rank's return buffer peer_ret[src] at the row the run tables give (rows of one source are
  // contiguous in the segment and at the destination, so a tile's rows stream to consecutive remote rows), and
  // forwards the optional per-row scalar rowval[r] to peer_retg[src] at the same row.  Gates are applied by the
  // source when it sums its slots.
  const int* push_runs;        // [3][E][world] return-run tables from nmoe_rdep_plan (non-null selects the fused return)
  __nv_bfloat16* peer_ret[8];
  float* peer_retg[8];
  const float* rowval;
  int push_world, push_pairs;  // ranks in the run tables; rows of a source's return buffer (bound)
  int push_bulk;               // 1: the fused return hands 256-byte row segments to the bulk-copy unit
  // Mode 3 (sparse-attention indexer): rows of A are keys, columns of B are (query, head) pairs; the epilogue
  // writes C[query][key] = sum_head idx_w[query*heads + head] * relu(acc), -inf above the diagonal when causal.
  const float* idx_w;
  int idx_heads;
  int idx_causal;
  SwigluBwdEpi sb;             // mode 1: SwiGLU backward in the epilogue (sb.h13 != nullptr); C is not written
};

NMOE_DEVICE uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Wait on an mbarrier phase with a wall-clock bound.  Returns false on timeout or when
// another role of this CTA has already given up.
NMOE_DEVICE bool mbar_wait_timed(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 255u) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitBudgetNs) return false;
    }
  }
  return true;
}

struct TileCoord {
  int m_blk, n_blk, expert;
  int kb_begin, kb_count;    // K range in units of BK
};

template <int BN, int MODE>
NMOE_DEVICE bool decode_tile(const GemmParams& p, int t, int m_tiles, int n_tiles, TileCoord& tc) {
  if (MODE == 2) {
    const int per_e = m_tiles * n_tiles;
    const int e = t / per_e;
    if (e >= p.E) return false;
    const int r = t - e * per_e;
    tc.expert = e;
    tc.m_blk = r % m_tiles;
    tc.n_blk = r / m_tiles;
    const int r0 = p.offs[e], r1 = p.offs[e + 1];
    tc.kb_begin = r0 / BK;
    tc.kb_count = (r1 - r0) / BK;
    return true;
  }
  if (t >= m_tiles * n_tiles) return false;
  const int per_group = kGroupM * n_tiles;
  const int g = t / per_group;
  const int first_m = g * kGroupM;
  const int gm = min(kGroupM, m_tiles - first_m);
  const int r = t - g * per_group;
  tc.m_blk = first_m + r % gm;
  tc.n_blk = r / gm;
  tc.expert = (MODE == 1) ? p.tile_expert[tc.m_blk] : 0;
  tc.kb_begin = 0;
  tc.kb_count = (p.K + BK - 1) / BK;
  if (MODE == 3 && p.idx_causal) {
    // every key of the tile lies after every query of the tile: nothing to multiply
    const int last_query = (min((tc.n_blk + 1) * BN, p.N) - 1) / p.idx_heads;
    if (tc.m_blk * BM > last_query) tc.kb_count = 0;
  }
  return true;
}

template <int BN>
struct GemmSmem {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  // staging of the fused-return epilogue: bulk copies of 256-byte row segments (or the 4 KB transposing store)
  static constexpr int kEpiWarp = EpiBulk<256>::kWarpBytes > kEpiStageBytesPerWarp ? EpiBulk<256>::kWarpBytes : kEpiStageBytesPerWarp;
  static constexpr int kEpiStage = 4 * kEpiWarp;
  static constexpr int kBytes = kStages * (kStageA + kStageB) + kEpiStage + 1024 /*align*/ + 256 /*barriers*/;
};

// Indexer epilogue (mode 3), 64 accumulator columns of one key: relu, head weight (handed out by shuffles from the
// two coalesced loads w_lo / w_hi), sum over the heads of a query, one store per finished query.  HEADS > 0 fixes the
// head count at compile time (col is a multiple of 64, so the query boundaries are static); 0 uses hmask / hshift.
template <int HEADS>
NMOE_DEVICE void indexer_cols64(const uint32_t (&r)[64], float w_lo, float w_hi, int col, int N, int hmask, int hshift,
                                bool row_ok, int row, int causal, long long ldc, float* outp, float& accum) {
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    const float wv = __shfl_sync(0xffffffffu, i < 32 ? w_lo : w_hi, i & 31);   // zero past the last column
    accum = fmaf(fmaxf(__uint_as_float(r[i]), 0.f), wv, accum);
    const int cc = col + i;
    const bool last = HEADS > 0 ? ((i & (HEADS - 1)) == HEADS - 1) : ((cc & hmask) == hmask);
    if (last && cc < N) {
      const int tq = HEADS > 0 ? cc / HEADS : (cc >> hshift);
      if (row_ok) outp[static_cast<long long>(tq) * ldc + row] = (causal && row > tq) ? -INFINITY : accum;
      accum = 0.f;
    }
  }
}

template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(kGemmThreads, 1)
k_gemm_bf16(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using S = GemmSmem<BN>;
  constexpr int kStages = S::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * S::kStageA;
  uint8_t* epi_stage = smem + kStages * (S::kStageA + S::kStageB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + S::kEpiStage);
  uint64_t* full = bars;                    // [kStages]
  uint64_t* empty = bars + kStages;         // [kStages]
  uint64_t* tmem_full = bars + 2 * kStages; // [2]
  uint64_t* tmem_empty = tmem_full + 2;     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  int m_tiles, n_tiles;
  if (MODE == 1) m_tiles = min(*p.n_m_tiles, (p.M + BM - 1) / BM);
  else m_tiles = (p.M + BM - 1) / BM;
  n_tiles = (p.N + BN - 1) / BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      TileCoord tc;
      bool ok = true;
      for (int t = blockIdx.x; ok && decode_tile<BN, MODE>(p, t, m_tiles, n_tiles, tc); t += gridDim.x) {
        const int m0 = tc.m_blk * BM, n0 = tc.n_blk * BN;
        for (int kb = 0; kb < tc.kb_count; ++kb) {
          if (!mbar_wait_timed(&empty[stage], phase ^ 1, abort_flag)) {
            report_status(p.status, kStatusWaitTimeout, 100, stage, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          mbar_expect_tx(&full[stage], S::kStageA + S::kStageB);
          const int k0 = (tc.kb_begin + kb) * BK;
          uint8_t* a_dst = sA + stage * S::kStageA;
          uint8_t* b_dst = sB + stage * S::kStageB;
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(a_dst + c * (BK * 128), &tmA, &full[stage], m0 + c * 64, k0);
          } else {
            tma_load_2d(a_dst, &tmA, &full[stage], k0, m0);
          }
          if (B_MN) {
            const int krow = (MODE == 1) ? static_cast<int>(tc.expert * p.b_rows_per_expert) + k0 : k0;
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * (BK * 128), &tmB, &full[stage], n0 + c * 64, krow);
          } else {
            const int nrow = (MODE == 1) ? static_cast<int>(tc.expert * p.b_rows_per_expert) + n0 : n0;
            tma_load_2d(b_dst, &tmB, &full[stage], k0, nrow);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      TileCoord tc;
      bool ok = true;
      for (int t = blockIdx.x; ok && decode_tile<BN, MODE>(p, t, m_tiles, n_tiles, tc); t += gridDim.x) {
        if (tc.kb_count == 0) continue;
        if (!mbar_wait_timed(&tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          report_status(p.status, kStatusWaitTimeout, 200, acc, t);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < tc.kb_count; ++kb) {
          if (!mbar_wait_timed(&full[stage], phase, abort_flag)) {
            report_status(p.status, kStatusWaitTimeout, 201, stage, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kStageA);
          const uint32_t b_addr = smem_u32(sB + stage * S::kStageB);
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            const uint64_t a_desc = A_MN ? make_smem_desc(a_addr + j * 2048, BK * 128, 1024, kSwizzle128B)
                                         : make_smem_desc(a_addr + j * 32, 0, 1024, kSwizzle128B);
            const uint64_t b_desc = B_MN ? make_smem_desc(b_addr + j * 2048, BK * 128, 1024, kSwizzle128B)
                                         : make_smem_desc(b_addr + j * 32, 0, 1024, kSwizzle128B);
            mma_f16_ss(d_tmem, a_desc, b_desc, idesc, (kb | j) != 0 ? 1u : 0u);
          }
          mma_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&tmem_full[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue: TMEM -> registers -> global
    const int q = warp & 3;                  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool used_bulk = false;
    TileCoord tc;
    const int m_limit = (MODE == 1) ? m_tiles * BM : p.M;
    for (int t = blockIdx.x; decode_tile<BN, MODE>(p, t, m_tiles, n_tiles, tc); t += gridDim.x) {
      const int row = tc.m_blk * BM + q * 32 + lane;
      const int n0 = tc.n_blk * BN;
      bool row_ok = row < m_limit;
      __nv_bfloat16* push_dst = nullptr;
      float push_gate = 1.f;
      if (MODE == 1 && p.push_runs != nullptr && row_ok) {
        // rows of one source are contiguous in an expert's segment and land contiguously at that source:
        // consecutive rows of this tile go to consecutive destination rows
        int src = 0, drow = 0;
        row_ok = run_lookup(p.push_runs, p.E, p.push_world, tc.expert, row, src, drow) && drow >= 0 && drow < p.push_pairs &&
                 p.peer_ret[src & 7] != nullptr;
        if (row_ok) {
          push_dst = p.peer_ret[src] + static_cast<long long>(drow) * p.ldc;
          if (tc.n_blk == 0 && p.rowval != nullptr) p.peer_retg[src][drow] = p.rowval[row];
        }
      }
      const long long crow = (MODE == 2) ? static_cast<long long>(tc.expert) * p.M + row : row;
      const bool have_acc = tc.kb_count > 0;
      if (have_acc) {
        bool ok = mbar_wait_timed(&tmem_full[acc], acc_phase, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report_status(p.status, kStatusWaitTimeout, 300, acc, t);
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
        uint8_t* t0 = epi_stage + (warp - 2) * S::kEpiWarp;
        uint8_t* t1 = t0 + 4096;
        float dot = 0.f;
        int4 g[8];
        if (n0 < p.N) {
          sb_issue_loads(g, p.sb.h13, row0, rows_ok, 2LL * p.N, n0, lane);
          sb_stage_h(t0, g, lane);
          __syncwarp();
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = n0 + c * 32;
          if (col >= p.N) break;               // uniform over the warp
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32, r);
          const bool more = col + 32 < p.N && c + 1 < BN / 32;
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
        uint8_t* srow = EpiBulk<256>::row(epi_stage + (warp - 2) * S::kEpiWarp, lane);
        __nv_bfloat16* dst0 = (row_ok && push_dst != nullptr) ? push_dst : nullptr;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = n0 + c * 64;
          if (col >= p.N) break;               // uniform over the warp
          uint32_t r[64];
          const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 64;
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
      } else if (MODE == 1 && p.push_runs != nullptr && have_acc && (p.N & 63) == 0 && (p.ldc & 7) == 0) {
        // fused return, coalesced: 64 columns (128 bytes) of 4 rows per store instruction
        uint8_t* stage = epi_stage + (warp - 2) * S::kEpiWarp;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = n0 + c * 64;
          if (col >= p.N) break;               // uniform over the warp
          uint32_t r[64];
          const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 64;
          tmem_ld_32x32b_x32(ta, r);
          tmem_ld_32x32b_x32(ta + 32, r + 32);
          tmem_ld_wait();
          warp_store_rows_64cols(stage, r, push_gate, (row_ok && push_dst != nullptr) ? push_dst + col : nullptr, lane);
        }
      } else if (MODE == 3) {
        // indexer scores: this thread owns one key; each group of idx_heads columns is one query
        float* outp = static_cast<float*>(p.C);
        const int hmask = p.idx_heads - 1;       // heads is a power of two that divides BN
        const int hshift = 31 - __clz(p.idx_heads);
        float accum = 0.f;
        if (!have_acc) {
          // tile skipped by the causal test in decode_tile: every key comes after every query
          const int q_end = min(n0 + BN, p.N) >> hshift;
          if (row_ok)
            for (int tq = n0 >> hshift; tq < q_end; ++tq) outp[static_cast<long long>(tq) * p.ldc + row] = -INFINITY;
        } else
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = n0 + c * 64;
          if (col >= p.N) break;                 // uniform over the warp
          // head weights of these 64 columns: two coalesced loads, handed out by shuffles below
          const float w_lo = (col + lane < p.N) ? __ldg(p.idx_w + col + lane) : 0.f;
          const float w_hi = (col + 32 + lane < p.N) ? __ldg(p.idx_w + col + 32 + lane) : 0.f;
          uint32_t r[64];
          if (have_acc) {
            const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 64;
            tmem_ld_32x32b_x32(ta, r);
            tmem_ld_32x32b_x32(ta + 32, r + 32);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 64; ++i) r[i] = 0u;
          }
#define NMOE_IDX_CASE(H_) \
  case H_: indexer_cols64<H_>(r, w_lo, w_hi, col, p.N, hmask, hshift, row_ok, row, p.idx_causal, p.ldc, outp, accum); break
          switch (p.idx_heads) {
            NMOE_IDX_CASE(1); NMOE_IDX_CASE(2); NMOE_IDX_CASE(4); NMOE_IDX_CASE(8);
            NMOE_IDX_CASE(16); NMOE_IDX_CASE(32); NMOE_IDX_CASE(64);
            default: indexer_cols64<0>(r, w_lo, w_hi, col, p.N, hmask, hshift, row_ok, row, p.idx_causal, p.ldc, outp, accum);
          }
#undef NMOE_IDX_CASE
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        if (have_acc) {
          tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32, r);
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
              for (int i = 0; i < 32 && col + i < p.N; ++i)
                dst[i] = __uint_as_float(r[i]) + (p.accumulate ? dst[i] : 0.f);
            }
          } else if (MODE == 1 && push_dst != nullptr) {
            __nv_bfloat16* dst = push_dst + col;
            if (col + 32 <= p.N && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                int4 v;
                v.x = pack_bf16x2(__uint_as_float(r[8 * i]) * push_gate, __uint_as_float(r[8 * i + 1]) * push_gate);
                v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * push_gate, __uint_as_float(r[8 * i + 3]) * push_gate);
                v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * push_gate, __uint_as_float(r[8 * i + 5]) * push_gate);
                v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * push_gate, __uint_as_float(r[8 * i + 7]) * push_gate);
                st_relaxed_sys_v4(reinterpret_cast<int4*>(dst) + i, v);
              }
            } else {
              for (int i = 0; i < 32 && col + i < p.N; ++i) dst[i] = __float2bfloat16(__uint_as_float(r[i]) * push_gate);
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
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
    if (used_bulk) epi_bulk_drain();         // this lane's row copies have been written before the kernel ends
  }

  // Teardown.  After a timeout, give copies in flight a moment to land before the CTA's
  // shared memory and tensor memory are released.
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (MODE == 1 && p.push_runs != nullptr) __threadfence_system();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------ host side
struct MapKey {
  const void* base; int dtype; uint64_t inner, outer, pitch; uint32_t bi, bo; int sw;
  bool operator<(const MapKey& o) const {
    return std::tie(base, dtype, inner, outer, pitch, bi, bo, sw) <
           std::tie(o.base, o.dtype, o.inner, o.outer, o.pitch, o.bi, o.bo, o.sw);
  }
};

static int cached_map(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch_bytes,
                      uint32_t box_inner, uint32_t box_outer) {
  static std::map<MapKey, CUtensorMap> cache;
  static std::mutex mu;
  MapKey k{base, kTmaBf16, inner, outer, pitch_bytes, box_inner, box_outer, kTmaSwizzle128};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(k);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  int rc = make_tensor_map_2d(out, base, kTmaBf16, inner, outer, pitch_bytes, box_inner, box_outer, kTmaSwizzle128);
  if (rc != 0) return rc;
  if (cache.size() > 4096) cache.clear();
  cache[k] = *out;
  return 0;
}

static int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, bool A_MN, bool B_MN, int MODE>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int max_tiles, cudaStream_t st) {
  auto kern = k_gemm_bf16<BN, A_MN, B_MN, MODE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::kBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int grid = max_tiles < num_sms() ? max_tiles : num_sms();
  if (grid < 1) return 0;
  kern<<<grid, kGemmThreads, GemmSmem<BN>::kBytes, st>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

template <int BN, int MODE>
static int dispatch_major(int a_mn, int b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p,
                          int max_tiles, cudaStream_t st) {
  if (!a_mn && !b_mn) return launch<BN, false, false, MODE>(tmA, tmB, p, max_tiles, st);
  if (!a_mn && b_mn) return launch<BN, false, true, MODE>(tmA, tmB, p, max_tiles, st);
  if (a_mn && b_mn) return launch<BN, true, true, MODE>(tmA, tmB, p, max_tiles, st);
  return launch<BN, true, false, MODE>(tmA, tmB, p, max_tiles, st);
}

}  // namespace nmoe

using namespace nmoe;

extern "C" {

// C = op(A) op(B) in bf16 with fp32 accumulation.
//   mode 0: A is [M,K] (a_mn=0, lda >= K) or [K,M] (a_mn=1, lda >= M); B is [N,K] (b_mn=0) or [K,N] (b_mn=1).
//   mode 1: M = capacity in rows (multiple of 128); tile_expert / n_m_tiles describe the valid
//           128-row tiles; B holds E stacked matrices ([E*N,K] or [E*K,N]).
//   mode 2: A is [R,M] and B is [R,N] (both MN-major, rows = contraction), offs[E+1] gives each
//           expert's row range; C holds E stacked [M,N] outputs.
// bn selects the N tile (64, 128 or 256; 0 = choose).  status may be null.
static int gemm_bf16_go(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                        long long ldc, int a_mn, int b_mn, int mode, int E, const int* tile_expert, const int* n_m_tiles,
                        const int* offs, long long a_rows, long long b_rows, int out_fp32, int accumulate, int bn,
                        void* status, const void* push_runs, void* const* peer_ret, void* const* peer_retg,
                        const float* rowval, int push_pairs, int world, const SwigluBwdEpi* sb, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (mode != 2 && K <= 0) return -1;
  if ((lda % 8) || (ldb % 8)) return -2;
  if (mode == 2 && !(a_mn && b_mn)) return -3;
  if (mode != 0 && (K % BK) != 0 && mode == 1) return -4;
  if (bn == 0) bn = (N >= 256 && (N % 256 == 0 || N > 1024)) ? 256 : (N > 64 ? 128 : 64);
  if (bn != 64 && bn != 128 && bn != 256) return -5;

  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.E = E;
  p.tile_expert = tile_expert; p.n_m_tiles = n_m_tiles; p.offs = offs;
  p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.b_rows_per_expert = (mode == 1) ? (b_mn ? K : N) : 0;
  p.status = static_cast<StatusRecord*>(status);
  p.push_runs = static_cast<const int*>(push_runs);
  p.rowval = rowval;
  p.push_pairs = push_pairs; p.push_world = world;
  p.push_bulk = epi_push_bulk_enabled();
  p.idx_w = nullptr; p.idx_heads = 1; p.idx_causal = 0;
  p.sb = SwigluBwdEpi{nullptr, nullptr, nullptr, nullptr, nullptr, 0};
  if (sb != nullptr) {
    if (mode != 1 || push_runs != nullptr || (N % 32) != 0) return -7;
    p.sb = *sb;
  }
  for (int r = 0; r < 8; ++r) {
    p.peer_ret[r] = (push_runs && peer_ret && r < world) ? static_cast<__nv_bfloat16*>(peer_ret[r]) : nullptr;
    p.peer_retg[r] = (push_runs && peer_retg && r < world) ? static_cast<float*>(peer_retg[r]) : nullptr;
  }
  if (push_runs && (mode != 1 || out_fp32 || world > 8)) return -6;

  // Tensor maps.  a_rows / b_rows are the outer extents of the 2-D views (rows in memory).
  CUtensorMap tmA, tmB;
  int rc;
  if (a_mn) rc = cached_map(&tmA, A, static_cast<uint64_t>(M), static_cast<uint64_t>(a_rows), lda * 2, 64, BK);
  else rc = cached_map(&tmA, A, static_cast<uint64_t>(K), static_cast<uint64_t>(a_rows), lda * 2, BK, BM);
  if (rc != 0) return rc;
  if (b_mn) rc = cached_map(&tmB, B, static_cast<uint64_t>(N), static_cast<uint64_t>(b_rows), ldb * 2, 64, BK);
  else rc = cached_map(&tmB, B, static_cast<uint64_t>(K), static_cast<uint64_t>(b_rows), ldb * 2, BK, bn);
  if (rc != 0) return rc;

  const int m_tiles = (M + BM - 1) / BM;
  const int n_tiles = (N + bn - 1) / bn;
  const int max_tiles = (mode == 2) ? E * m_tiles * n_tiles : m_tiles * n_tiles;

#define GO(BN_)                                                                                   \
  (mode == 0   ? dispatch_major<BN_, 0>(a_mn, b_mn, tmA, tmB, p, max_tiles, st)                   \
   : mode == 1 ? dispatch_major<BN_, 1>(a_mn, b_mn, tmA, tmB, p, max_tiles, st)                   \
               : launch<BN_, true, true, 2>(tmA, tmB, p, max_tiles, st))
  if (bn == 256) return GO(256);
  if (bn == 128) return GO(128);
  return GO(64);
#undef GO
}

int nmoe_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                   long long ldc, int a_mn, int b_mn, int mode, int E, const int* tile_expert, const int* n_m_tiles,
                   const int* offs, long long a_rows, long long b_rows, int out_fp32, int accumulate, int bn,
                   void* status, const void* push_runs, void* const* peer_ret, void* const* peer_retg,
                   const float* rowval, int push_pairs, int world, cudaStream_t st) {
  return gemm_bf16_go(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, mode, E, tile_expert, n_m_tiles, offs, a_rows, b_rows,
                      out_fp32, accumulate, bn, status, push_runs, peer_ret, peer_retg, rowval, push_pairs, world, nullptr, st);
}

// Grouped dA = dY W2^T (mode 1) whose epilogue is the SwiGLU backward: reads h13 [M, 2N], writes dh13 [M, 2N], the
// scaled activation a_out [M, N] (optional) and per-column-tile partial row dots rowdot_parts [ceil(N/256), rows_cap]
// (optional).  dA is not written.  N % 32 == 0.  The column tile is 256.
int nmoe_gemm_bf16_swiglu_bwd(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, int b_mn,
                              int E, const int* tile_expert, const int* n_m_tiles, long long a_rows, long long b_rows,
                              const void* h13, void* dh13, void* a_out, const float* row_scale, float* rowdot_parts,
                              long long rows_cap, void* status, cudaStream_t st) {
  SwigluBwdEpi sb{static_cast<const __nv_bfloat16*>(h13), static_cast<__nv_bfloat16*>(dh13), static_cast<__nv_bfloat16*>(a_out),
                  row_scale, rowdot_parts, rows_cap};
  if (h13 == nullptr || dh13 == nullptr) return -7;
  return gemm_bf16_go(A, B, dh13, M, N, K, lda, ldb, N, 0, b_mn, 1, E, tile_expert, n_m_tiles, nullptr, a_rows, b_rows,
                      0, 0, 256, status, nullptr, nullptr, nullptr, nullptr, 0, 0, &sb, st);
}

// Lightning-indexer scores of sparse attention, one batch element per call:
//   out[t][s] = sum_h w[t*heads + h] * relu(q[t*heads + h, :] . k[s, :]),  -inf where s > t if causal.
// k is [S, D] (row stride ldk), q is [T*heads, D] (row stride ldq), w is fp32 [T*heads], out is fp32 [T, ldo].
// heads must be a power of two <= 128; D a multiple of 8.
int nmoe_dsa_indexer_scores(const void* k, const void* q, const float* w, float* out, int S, int T, int heads, int D,
                            long long ldk, long long ldq, long long ldo, int causal, void* status, cudaStream_t st) {
  if (S <= 0 || T <= 0) return 0;
  if (heads <= 0 || heads > 128 || (heads & (heads - 1)) != 0) return -1;
  if (D <= 0 || (D % 8) || (ldk % 8) || (ldq % 8)) return -2;
  constexpr int kBn = 128;
  GemmParams p;
  p.M = S; p.N = T * heads; p.K = D; p.E = 1;
  p.tile_expert = nullptr; p.n_m_tiles = nullptr; p.offs = nullptr;
  p.C = out; p.ldc = ldo; p.out_fp32 = 1; p.accumulate = 0;
  p.b_rows_per_expert = 0;
  p.status = static_cast<StatusRecord*>(status);
  p.push_runs = nullptr; p.rowval = nullptr; p.push_pairs = 0; p.push_world = 0; p.push_bulk = 0;
  for (int r = 0; r < 8; ++r) { p.peer_ret[r] = nullptr; p.peer_retg[r] = nullptr; }
  p.idx_w = w; p.idx_heads = heads; p.idx_causal = causal;
  p.sb = SwigluBwdEpi{nullptr, nullptr, nullptr, nullptr, nullptr, 0};
  CUtensorMap tmA, tmB;
  int rc = cached_map(&tmA, k, static_cast<uint64_t>(D), static_cast<uint64_t>(S), ldk * 2, BK, BM);
  if (rc != 0) return rc;
  rc = cached_map(&tmB, q, static_cast<uint64_t>(D), static_cast<uint64_t>(p.N), ldq * 2, BK, kBn);
  if (rc != 0) return rc;
  const int m_tiles = (S + BM - 1) / BM, n_tiles = (p.N + kBn - 1) / kBn;
  return launch<kBn, false, false, 3>(tmA, tmB, p, m_tiles * n_tiles, st);
}

}  // extern "C"
