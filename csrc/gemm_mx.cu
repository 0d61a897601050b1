// Block-scaled FP8 GEMM (MXFP8: E4M3 values, one E8M0 scale per 32 elements of K) on tcgen05:
// C[M,N] (bf16) = A[M,K] * B[N,K]^T with both operands K-major.  Same structure as the bf16
// kernel (TMA producer warp, single-thread MMA issuer, 4 epilogue warps, persistent tiles,
// accumulators in tensor memory); in addition each pipeline stage carries the 512-byte scale
// atoms of its A and B tiles, which the MMA thread moves from shared to tensor memory with
// tcgen05.cp right before the four K=32 `kind::mxf8f6f4.block_scale` instructions of the stage.
//
// mode 0: dense.  mode 1: rows of A/C are 128-aligned per-expert segments (tile -> expert table,
// valid tile count on the device), B and its scales are stacked per expert.  The epilogue can
// push rows straight into the source ranks' RDEP return buffers (see gemm.cu).
// Requirements: K % 32 == 0 (FP8; a tail shorter than a stage is zero-filled by TMA); scales in the atom layout of common/sf_layout.cuh.
//
// FMT = 1 is the same kernel for MXFP4 operands (E2M1 nibbles, two per byte, E8M0 per 32):
// a stage is still 128 bytes of K per row (256 elements, two scale atoms per 128 rows) and issues
// four K=64 `kind::mxf4nvf4.block_scale.scale_vec::2X` instructions; K % 128 == 0.
// FMT = 2 is NVFP4: E2M1 nibbles with one UE4M3 scale per 16 elements (`scale_vec::4X`, four atoms per stage,
// one per instruction) and a per-tensor fp32 scale pair folded into the epilogue (alpha); K % 64 == 0.
//
// Replaces the reference's CuTe-DSL grouped block-scaled kernel (nmoe/blockscaled/grouped.py:545-2093).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common/epilogue.cuh"
#include "common/ptx.cuh"
#include "common/quant_dev.cuh"
#include "common/tensormap.h"

namespace nmoe {

constexpr int MX_BM = 128;
constexpr int MX_BK = 128;               // bytes == elements for fp8; one 128-byte swizzle span
constexpr int kMxThreads = 192;
constexpr int kMxGroupM = 16;
constexpr uint64_t kMxWaitBudgetNs = 2000000000ull;

struct MxParams {
  int M, N, K, E;
  const int* tile_expert;
  const int* n_m_tiles;
  __nv_bfloat16* C;
  long long ldc;
  const uint8_t* sfa;          // A scales, atoms [M/128][K/128]
  const uint8_t* sfb;          // B scales, atoms [(E*N)/128][K/128]
  StatusRecord* status;
  const int* push_runs;        // [3][E][world] return-run tables from nmoe_rdep_plan (non-null selects the fused return)
  __nv_bfloat16* peer_ret[8];
  int push_world, push_pairs;  // ranks in the run tables; rows of a source's return buffer (bound)
  int push_bulk;               // 1: the fused return hands 128-byte row segments to the bulk-copy unit
  float alpha;                 // multiplies every output (NVFP4: product of the two per-tensor scales)
  const float* alpha_dev;      // optional second factor read from device memory (a scale that only the device knows)
  // fused SwiGLU + quantise epilogue (act_q != nullptr): instead of C [rows, N], write the quantised
  // activation [rows, N/2] (E4M3 bytes, or E2M1 nibbles when act_fp4) and its E8M0 scale atoms
  uint8_t* act_q;
  uint8_t* act_sf;
  int act_sf_cols;
  int act_fp4;
};

NMOE_DEVICE uint64_t mx_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
NMOE_DEVICE bool mx_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = mx_timer_ns();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++it & 255u) == 0) {
      if (*abort_flag) return false;
      if (mx_timer_ns() - t0 > kMxWaitBudgetNs) return false;
    }
  }
  return true;
}
// Untiled bulk copy global -> shared completing on an mbarrier (16-byte aligned, size % 16 == 0).
NMOE_DEVICE void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// FMT: 0 = MXFP8 (E4M3, E8M0 per 32), 1 = MXFP4 (E2M1, E8M0 per 32), 2 = NVFP4 (E2M1, UE4M3 per 16)
template <int BN, int FMT>
struct MxSmem {
  static constexpr int kKA = FMT == 0 ? 1 : (FMT == 1 ? 2 : 4);   // scale atoms (4 scale bytes per row each) per stage
  static constexpr int kStageK = FMT == 0 ? 128 : 256;            // elements of K per stage (always 128 bytes per row)
  static constexpr int kAtomK = FMT == 2 ? 64 : 128;              // elements of K covered by one scale atom
  static constexpr int kStageA = MX_BM * MX_BK;
  static constexpr int kStageB = BN * MX_BK;
  static constexpr int kStageSF = kKA * (512 + (BN / 128) * 512);
  static constexpr int kStages = (BN == 256) ? (FMT == 2 ? 3 : 4) : (FMT == 2 ? 5 : 6);
  // staging of the fused-return epilogue: bulk copies of 128-byte row segments (or the 4 KB transposing store)
  static constexpr int kEpiWarp = EpiBulk<128>::kWarpBytes > kEpiStageBytesPerWarp ? EpiBulk<128>::kWarpBytes : kEpiStageBytesPerWarp;
  static_assert(kStages * (MX_BM * MX_BK + BN * MX_BK + kKA * (512 + (BN / 128) * 512)) + 4 * kEpiWarp + 1280 <= 232448,
                "shared memory budget");
  static constexpr int kAcc = (BN == 256) ? 1 : 2;
  static constexpr int kEpiStage = 4 * kEpiWarp;
  static constexpr int kBytes = kStages * (kStageA + kStageB + kStageSF) + kEpiStage + 1024 + 256;
};

template <int BN, int MODE>
NMOE_DEVICE bool mx_decode(const MxParams& p, int t, int m_tiles, int n_tiles, int& m_blk, int& n_blk, int& expert) {
  if (t >= m_tiles * n_tiles) return false;
  const int per_group = kMxGroupM * n_tiles;
  const int g = t / per_group;
  const int first_m = g * kMxGroupM;
  const int gm = min(kMxGroupM, m_tiles - first_m);
  const int r = t - g * per_group;
  m_blk = first_m + r % gm;
  n_blk = r / gm;
  expert = (MODE == 1) ? p.tile_expert[m_blk] : 0;
  return true;
}

template <int BN, int MODE, int FMT>
__global__ void __launch_bounds__(kMxThreads, 1)
k_gemm_mx(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const MxParams p) {
  using S = MxSmem<BN, FMT>;
  constexpr bool FP4 = FMT != 0;
  constexpr int kStages = S::kStages;
  constexpr int kAcc = S::kAcc;
  constexpr int KA = S::kKA;
  constexpr uint32_t kSfaCol = kAcc * BN;
  constexpr uint32_t kSfbCol = kSfaCol + 4 * KA;
  static_assert(kSfbCol + 4 * KA * (BN / 128) <= 512, "tensor memory budget");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + kStages * S::kStageA;
  uint8_t* sSF = sB + kStages * S::kStageB;
  uint8_t* epi_stage = sSF + kStages * S::kStageSF;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + S::kEpiStage);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tmem_full = bars + 2 * kStages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (MODE == 1) ? min(*p.n_m_tiles, (p.M + MX_BM - 1) / MX_BM) : (p.M + MX_BM - 1) / MX_BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int k_blocks = (p.K + S::kStageK - 1) / S::kStageK;     // a stage covers 128 bytes of K per row
  // 4-bit formats with a K tail shorter than a stage: the last stage loads only the scale atoms that
  // exist and issues only their instructions (the tile loads past K are zero-filled by TMA)
  const int tail_atoms = (FP4 && (p.K % S::kStageK) != 0) ? ((p.K % S::kStageK) + S::kAtomK - 1) / S::kAtomK : KA;
  const int sf_k_atoms = (p.K + S::kAtomK - 1) / S::kAtomK;     // atom columns along K (the last one may be partial)

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 4); }
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
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      int m_blk, n_blk, expert;
      bool ok = true;
      for (int t = blockIdx.x; ok && mx_decode<BN, MODE>(p, t, m_tiles, n_tiles, m_blk, n_blk, expert); t += gridDim.x) {
        const int m0 = m_blk * MX_BM, n0 = n_blk * BN;
        const long long brow = (MODE == 1 ? static_cast<long long>(expert) * p.N : 0) + n0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mx_wait(&empty[stage], phase ^ 1, abort_flag)) {
            report_status(p.status, kStatusWaitTimeout, 600, stage, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const int n_atoms = (kb == k_blocks - 1) ? tail_atoms : KA;
          mbar_expect_tx(&full[stage], S::kStageA + S::kStageB + n_atoms * (512 + (BN / 128) * 512));
          tma_load_2d(sA + stage * S::kStageA, &tmA, &full[stage], kb * MX_BK, m0);
          tma_load_2d(sB + stage * S::kStageB, &tmB, &full[stage], kb * MX_BK, static_cast<int>(brow));
          uint8_t* sf_dst = sSF + stage * S::kStageSF;
#pragma unroll
          for (int ka = 0; ka < KA; ++ka) {
            if (ka >= n_atoms) break;
            bulk_load(sf_dst + 512 * ka, p.sfa + (static_cast<size_t>(m_blk) * sf_k_atoms + kb * KA + ka) * 512, 512,
                      &full[stage]);
#pragma unroll
            for (int a = 0; a < BN / 128; ++a)
              bulk_load(sf_dst + 512 * (KA + ka * (BN / 128) + a),
                        p.sfb + (static_cast<size_t>(brow / 128 + a) * sf_k_atoms + kb * KA + ka) * 512, 512, &full[stage]);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      int m_blk, n_blk, expert;
      bool ok = true;
      for (int t = blockIdx.x; ok && mx_decode<BN, MODE>(p, t, m_tiles, n_tiles, m_blk, n_blk, expert); t += gridDim.x) {
        if (!mx_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag)) {
          report_status(p.status, kStatusWaitTimeout, 610, acc, t);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mx_wait(&full[stage], phase, abort_flag)) {
            report_status(p.status, kStatusWaitTimeout, 611, stage, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(sA + stage * S::kStageA);
          const uint32_t b_addr = smem_u32(sB + stage * S::kStageB);
          const uint32_t sf_addr = smem_u32(sSF + stage * S::kStageSF);
          // scale atoms: 32 rows x 16 bytes, no swizzle, 8-row groups 128 bytes apart
          const int n_atoms = (kb == k_blocks - 1) ? tail_atoms : KA;
#pragma unroll
          for (int ka = 0; ka < KA; ++ka) {
            if (ka >= n_atoms) break;
            tmem_cp_32x128b_warpx4(tmem_base + kSfaCol + 4 * ka, make_smem_desc(sf_addr + 512 * ka, 0, 128, kSwizzleNone));
#pragma unroll
            for (int a = 0; a < BN / 128; ++a)
              tmem_cp_32x128b_warpx4(tmem_base + kSfbCol + 4 * (ka * (BN / 128) + a),
                                     make_smem_desc(sf_addr + 512 * (KA + ka * (BN / 128) + a), 0, 128, kSwizzleNone));
          }
#pragma unroll
          for (int j = 0; j < MX_BK / 32; ++j) {
            const uint64_t a_desc = make_smem_desc(a_addr + j * 32, 0, 1024, kSwizzle128B);
            const uint64_t b_desc = make_smem_desc(b_addr + j * 32, 0, 1024, kSwizzle128B);
            if (FMT == 2) {
              // NVFP4: K=64 per instruction, four UE4M3 scale bytes per row = one whole atom per instruction
              if (j >= n_atoms) break;
              const uint32_t idesc = make_idesc_mx(MX_BM, BN, 1, 1, 0, 0, 0);
              mma_nvf4_block16_ss(d_tmem, a_desc, b_desc, idesc, tmem_base + kSfaCol + 4 * j,
                                  tmem_base + kSfbCol + 4 * (BN / 128) * j, (kb | j) != 0 ? 1u : 0u);
              continue;
            }
            if (FP4 && (j >> 1) >= n_atoms) break;
            if (FP4) {
              // K=64 per instruction: two scale bytes per row, picked by id 0 / 2 inside atom j/2
              const uint32_t id = static_cast<uint32_t>(j & 1) * 2;
              const uint32_t idesc = make_idesc_mx(MX_BM, BN, 1, 1, 1, id, id);
              mma_mxf4_block32_ss(d_tmem, a_desc, b_desc, idesc, tmem_base + kSfaCol + 4 * (j >> 1),
                                  tmem_base + kSfbCol + 4 * (BN / 128) * (j >> 1), (kb | j) != 0 ? 1u : 0u);
            } else {
              const uint32_t idesc = make_idesc_mx(MX_BM, BN, 0, 0, 1, static_cast<uint32_t>(j), static_cast<uint32_t>(j));
              mma_mxf8f6f4_ss(d_tmem, a_desc, b_desc, idesc, tmem_base + kSfaCol, tmem_base + kSfbCol,
                              (kb | j) != 0 ? 1u : 0u);
            }
          }
          mma_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mma_commit(&tmem_full[acc]);
        if (++acc == kAcc) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool used_bulk = false;
    int m_blk, n_blk, expert;
    const int m_limit = (MODE == 1) ? m_tiles * MX_BM : p.M;
    for (int t = blockIdx.x; mx_decode<BN, MODE>(p, t, m_tiles, n_tiles, m_blk, n_blk, expert); t += gridDim.x) {
      const int row = m_blk * MX_BM + q * 32 + lane;
      const int n0 = n_blk * BN;
      bool row_ok = row < m_limit;
      __nv_bfloat16* dst_row = row_ok ? p.C + static_cast<long long>(row) * p.ldc : nullptr;
      float gate = p.alpha * (p.alpha_dev != nullptr ? __ldg(p.alpha_dev) : 1.f);
      if (MODE == 1 && p.push_runs != nullptr && row_ok) {
        int src = 0, drow = 0;
        row_ok = run_lookup(p.push_runs, p.E, p.push_world, expert, row, src, drow) && drow >= 0 && drow < p.push_pairs &&
                 p.peer_ret[src & 7] != nullptr;
        if (row_ok) dst_row = p.peer_ret[src] + static_cast<long long>(drow) * p.ldc;
      }
      bool ok = mx_wait(&tmem_full[acc], acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report_status(p.status, kStatusWaitTimeout, 620, acc, t);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      if (MODE == 1 && p.push_runs != nullptr && p.push_bulk && (p.N & 63) == 0 && (p.ldc & 7) == 0) {
        // fused return through the copy unit: 64 columns (128 bytes) of this lane's row per bulk copy
        uint8_t* srow = EpiBulk<128>::row(epi_stage + (warp - 2) * S::kEpiWarp, lane);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = n0 + c * 64;
          if (col >= p.N) break;
          uint32_t r[64];
          const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 64;
          tmem_ld_32x32b_x32(ta, r);
          tmem_ld_32x32b_x32(ta + 32, r + 32);
          epi_bulk_wait_read();
          tmem_ld_wait();
          stage_64cols(srow, 0, r, gate);
          epi_bulk_fence();
          epi_bulk_store(row_ok ? dst_row + col : nullptr, srow, 128);
        }
        used_bulk = true;
      } else if (MODE == 1 && p.push_runs != nullptr && (p.N & 63) == 0 && (p.ldc & 7) == 0) {
        // fused return, coalesced: 64 columns (128 bytes) of 4 rows per store instruction
        uint8_t* stage = epi_stage + (warp - 2) * S::kEpiWarp;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = n0 + c * 64;
          if (col >= p.N) break;
          uint32_t r[64];
          const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 64;
          tmem_ld_32x32b_x32(ta, r);
          tmem_ld_32x32b_x32(ta + 32, r + 32);
          tmem_ld_wait();
          warp_store_rows_64cols(stage, r, gate, row_ok ? dst_row + col : nullptr, lane);
        }
      } else if (p.act_q != nullptr) {
        // fused SwiGLU + quantise (up/gate projection, columns interleaved gate even / up odd): 64 accumulator
        // columns of a row give 32 activations = one scale block, owned by one thread, so no shuffles are
        // needed; h13 itself is never written
        const int F = p.N >> 1;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = n0 + c * 64;
          if (col >= p.N) break;
          uint32_t r[64];
          const uint32_t ta = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 64;
          tmem_ld_32x32b_x32(ta, r);
          tmem_ld_32x32b_x32(ta + 32, r + 32);
          tmem_ld_wait();
          if (!row_ok) continue;
          if (p.C != nullptr) {
            // the backward wants H13 itself: store the 64 bf16 values next to the quantised activation (one pass
            // over the accumulator instead of a GEMM that writes H13 and a second kernel that reads it back)
            int4* hrow = reinterpret_cast<int4*>(p.C + static_cast<long long>(row) * p.ldc + col);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              int4 h;
              h.x = pack_bf16x2(__uint_as_float(r[8 * j]) * p.alpha, __uint_as_float(r[8 * j + 1]) * p.alpha);
              h.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * p.alpha, __uint_as_float(r[8 * j + 3]) * p.alpha);
              h.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * p.alpha, __uint_as_float(r[8 * j + 5]) * p.alpha);
              h.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * p.alpha, __uint_as_float(r[8 * j + 7]) * p.alpha);
              hrow[j] = h;
            }
          }
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            // round through bf16 twice like the unfused path (h13 stored as bf16, activation stored as bf16)
            const float g = __bfloat162float(__float2bfloat16(__uint_as_float(r[2 * i]) * p.alpha));
            const float u = __bfloat162float(__float2bfloat16(__uint_as_float(r[2 * i + 1]) * p.alpha));
            v[i] = __bfloat162float(__float2bfloat16(g / (1.f + __expf(-g)) * u));
          }
          const int b = col >> 6;                              // 32-element block index along F
          uint32_t w[8];
          uint8_t s;
          if (p.act_fp4) {
            s = quant_block_e2m1_regs(v, w);
            *reinterpret_cast<int4*>(p.act_q + static_cast<long long>(row) * (F >> 1) + b * 16) = make_int4(w[0], w[1], w[2], w[3]);
          } else {
            s = quant_block_e4m3_regs(v, w);
            int4* dq = reinterpret_cast<int4*>(p.act_q + static_cast<long long>(row) * F + b * 32);
            dq[0] = make_int4(w[0], w[1], w[2], w[3]);
            dq[1] = make_int4(w[4], w[5], w[6], w[7]);
          }
          p.act_sf[sf_mma_offset(row, b, p.act_sf_cols)] = s;
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (row_ok && col < p.N) {
          __nv_bfloat16* dst = dst_row + col;
          if (col + 32 <= p.N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              int4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * i]) * gate, __uint_as_float(r[8 * i + 1]) * gate);
              v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]) * gate, __uint_as_float(r[8 * i + 3]) * gate);
              v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]) * gate, __uint_as_float(r[8 * i + 5]) * gate);
              v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]) * gate, __uint_as_float(r[8 * i + 7]) * gate);
              st_relaxed_sys_v4(reinterpret_cast<int4*>(dst) + i, v);
            }
          } else {
            for (int i = 0; i < 32 && col + i < p.N; ++i) dst[i] = __float2bfloat16(__uint_as_float(r[i]) * gate);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (++acc == kAcc) { acc = 0; acc_phase ^= 1; }
    }
    if (used_bulk) epi_bulk_drain();         // this lane's row copies have been written before the kernel ends
  }

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  if (MODE == 1 && p.push_runs != nullptr) __threadfence_system();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

static int mx_cached_map(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t pitch,
                         uint32_t box_inner, uint32_t box_outer) {
  using Key = std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t>;
  static std::map<Key, CUtensorMap> cache;
  static std::mutex mu;
  Key k{base, inner, outer, pitch, box_inner, box_outer};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(k);
  if (it != cache.end()) { *out = it->second; return 0; }
  int rc = make_tensor_map_2d(out, base, kTmaU8, inner, outer, pitch, box_inner, box_outer, kTmaSwizzle128);
  if (rc != 0) return rc;
  if (cache.size() > 4096) cache.clear();
  cache[k] = *out;
  return 0;
}

template <int BN, int MODE, int FMT = 0>
static int mx_launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const MxParams& p, int max_tiles, cudaStream_t st) {
  auto kern = k_gemm_mx<BN, MODE, FMT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MxSmem<BN, FMT>::kBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = max_tiles < sms ? max_tiles : sms;
  if (grid < 1) return 0;
  kern<<<grid, kMxThreads, MxSmem<BN, FMT>::kBytes, st>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace nmoe

using namespace nmoe;

// A: [a_rows, K] e4m3 bytes, sfa: its scales; B: [b_rows, K] e4m3 (b_rows = N, or E*N for mode 1), sfb likewise.
// C: bf16 [*, ldc].  mode 1 additionally takes the tile table; push_runs/peer_ret select the fused RDEP return (see gemm.cu).
extern "C" int nmoe_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N,
                               int K, long long ldc, int mode, int E, const int* tile_expert, const int* n_m_tiles,
                               long long a_rows, long long b_rows, int bn, void* status, const void* push_runs,
                               void* const* peer_ret, int push_pairs, int world, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 32) != 0) return -1;         // a K tail shorter than 128 is zero-filled by TMA; its scale bytes are padding (127)
  if (mode == 1 && (N % 128) != 0) return -2;
  if (bn == 0) bn = (N % 256 == 0) ? 256 : 128;
  if (bn != 128 && bn != 256) return -5;
  MxParams p;
  p.M = M; p.N = N; p.K = K; p.E = E; p.tile_expert = tile_expert; p.n_m_tiles = n_m_tiles;
  p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.sfa = static_cast<const uint8_t*>(sfa); p.sfb = static_cast<const uint8_t*>(sfb);
  p.status = static_cast<StatusRecord*>(status);
  p.push_runs = static_cast<const int*>(push_runs); p.push_pairs = push_pairs; p.push_world = world;
  p.push_bulk = epi_push_bulk_enabled(true); p.alpha = 1.f; p.alpha_dev = nullptr; p.act_q = nullptr; p.act_sf = nullptr; p.act_sf_cols = 0; p.act_fp4 = 0;
  for (int r = 0; r < 8; ++r)
    p.peer_ret[r] = (push_runs && peer_ret && r < world) ? static_cast<__nv_bfloat16*>(peer_ret[r]) : nullptr;
  if (push_runs && (mode != 1 || world > 8)) return -6;
  CUtensorMap tmA, tmB;
  int rc = mx_cached_map(&tmA, A, K, a_rows, K, MX_BK, MX_BM);
  if (rc != 0) return rc;
  rc = mx_cached_map(&tmB, B, K, b_rows, K, MX_BK, bn);
  if (rc != 0) return rc;
  const int max_tiles = ((M + MX_BM - 1) / MX_BM) * ((N + bn - 1) / bn);
  if (bn == 256) return mode == 1 ? mx_launch<256, 1>(tmA, tmB, p, max_tiles, st) : mx_launch<256, 0>(tmA, tmB, p, max_tiles, st);
  return mode == 1 ? mx_launch<128, 1>(tmA, tmB, p, max_tiles, st) : mx_launch<128, 0>(tmA, tmB, p, max_tiles, st);
}

// MXFP4 operands: A [a_rows, K/2] bytes (two E2M1 nibbles per byte, low nibble = even k), B likewise,
// scales as for MXFP8 (E8M0 per 32 elements, atom layout).  K counts elements; K % 128 == 0.
extern "C" int nmoe_gemm_mxfp4(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N,
                               int K, long long ldc, int mode, int E, const int* tile_expert, const int* n_m_tiles,
                               long long a_rows, long long b_rows, int bn, void* status, const void* push_runs,
                               void* const* peer_ret, int push_pairs, int world, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % MX_BK) != 0) return -1;
  if (mode == 1 && (N % 128) != 0) return -2;
  if (bn == 0) bn = (N % 256 == 0) ? 256 : 128;
  if (bn != 128 && bn != 256) return -5;
  MxParams p;
  p.M = M; p.N = N; p.K = K; p.E = E; p.tile_expert = tile_expert; p.n_m_tiles = n_m_tiles;
  p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.sfa = static_cast<const uint8_t*>(sfa); p.sfb = static_cast<const uint8_t*>(sfb);
  p.status = static_cast<StatusRecord*>(status);
  p.push_runs = static_cast<const int*>(push_runs); p.push_pairs = push_pairs; p.push_world = world;
  p.push_bulk = epi_push_bulk_enabled(true); p.alpha = 1.f; p.alpha_dev = nullptr; p.act_q = nullptr; p.act_sf = nullptr; p.act_sf_cols = 0; p.act_fp4 = 0;
  for (int r = 0; r < 8; ++r)
    p.peer_ret[r] = (push_runs && peer_ret && r < world) ? static_cast<__nv_bfloat16*>(peer_ret[r]) : nullptr;
  if (push_runs && (mode != 1 || world > 8)) return -6;
  CUtensorMap tmA, tmB;
  int rc = mx_cached_map(&tmA, A, K / 2, a_rows, K / 2, MX_BK, MX_BM);
  if (rc != 0) return rc;
  rc = mx_cached_map(&tmB, B, K / 2, b_rows, K / 2, MX_BK, bn);
  if (rc != 0) return rc;
  const int max_tiles = ((M + MX_BM - 1) / MX_BM) * ((N + bn - 1) / bn);
  if (bn == 256)
    return mode == 1 ? mx_launch<256, 1, 1>(tmA, tmB, p, max_tiles, st) : mx_launch<256, 0, 1>(tmA, tmB, p, max_tiles, st);
  return mode == 1 ? mx_launch<128, 1, 1>(tmA, tmB, p, max_tiles, st) : mx_launch<128, 0, 1>(tmA, tmB, p, max_tiles, st);
}

// NVFP4 operands: packed E2M1 as for MXFP4; scales are UE4M3 bytes, one per 16 elements, in the same
// 128-row x 4-byte atom layout (atoms [rows/128][K/64]); alpha = tensor_scale_a * tensor_scale_b.
static int gemm_nvfp4_go(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N,
                         int K, long long ldc, int mode, int E, const int* tile_expert, const int* n_m_tiles,
                         long long a_rows, long long b_rows, int bn, float alpha, const float* alpha_dev, void* status,
                         cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 64) != 0) return -1;
  if (mode == 1 && (N % 128) != 0) return -2;
  if (bn == 0) bn = (N % 256 == 0) ? 256 : 128;
  if (bn != 128 && bn != 256) return -5;
  MxParams p;
  p.M = M; p.N = N; p.K = K; p.E = E; p.tile_expert = tile_expert; p.n_m_tiles = n_m_tiles;
  p.C = static_cast<__nv_bfloat16*>(C); p.ldc = ldc;
  p.sfa = static_cast<const uint8_t*>(sfa); p.sfb = static_cast<const uint8_t*>(sfb);
  p.status = static_cast<StatusRecord*>(status);
  p.push_runs = nullptr; p.push_pairs = 0; p.push_world = 0; p.push_bulk = 0; p.alpha = alpha; p.alpha_dev = alpha_dev; p.act_q = nullptr; p.act_sf = nullptr; p.act_sf_cols = 0; p.act_fp4 = 0;
  for (int r = 0; r < 8; ++r) p.peer_ret[r] = nullptr;
  CUtensorMap tmA, tmB;
  int rc = mx_cached_map(&tmA, A, K / 2, a_rows, K / 2, MX_BK, MX_BM);
  if (rc != 0) return rc;
  rc = mx_cached_map(&tmB, B, K / 2, b_rows, K / 2, MX_BK, bn);
  if (rc != 0) return rc;
  const int max_tiles = ((M + MX_BM - 1) / MX_BM) * ((N + bn - 1) / bn);
  if (bn == 256)
    return mode == 1 ? mx_launch<256, 1, 2>(tmA, tmB, p, max_tiles, st) : mx_launch<256, 0, 2>(tmA, tmB, p, max_tiles, st);
  return mode == 1 ? mx_launch<128, 1, 2>(tmA, tmB, p, max_tiles, st) : mx_launch<128, 0, 2>(tmA, tmB, p, max_tiles, st);
}

extern "C" int nmoe_gemm_nvfp4(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N,
                               int K, long long ldc, int mode, int E, const int* tile_expert, const int* n_m_tiles,
                               long long a_rows, long long b_rows, int bn, float alpha, void* status, cudaStream_t st) {
  return gemm_nvfp4_go(A, sfa, B, sfb, C, M, N, K, ldc, mode, E, tile_expert, n_m_tiles, a_rows, b_rows, bn, alpha, nullptr,
                       status, st);
}

// The same with the product of the two tensor scales left on the device: out = alpha * (*alpha_dev) * (A B^T).
// Used by the grouped expert GEMMs, whose weight scale comes out of a device-side amax.
extern "C" int nmoe_gemm_nvfp4_dev(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N,
                                   int K, long long ldc, int mode, int E, const int* tile_expert, const int* n_m_tiles,
                                   long long a_rows, long long b_rows, int bn, float alpha, const float* alpha_dev,
                                   void* status, cudaStream_t st) {
  return gemm_nvfp4_go(A, sfa, B, sfb, C, M, N, K, ldc, mode, E, tile_expert, n_m_tiles, a_rows, b_rows, bn, alpha, alpha_dev,
                       status, st);
}

// Grouped up/gate projection with the SwiGLU and the re-quantisation fused into the epilogue: rows of A are
// 128-aligned expert segments, B = W13 [E, 2F, K] with gate / up rows interleaved; writes act_q [a_rows, F]
// (E4M3) or [a_rows, F/2] (E2M1 when fp4 != 0) and act_sf (atom layout for [a_rows, F]).  Operands are MXFP8
// (fp4 == 0) or MXFP4 (fp4 != 0).  N = 2F must be a multiple of 128.
extern "C" int nmoe_gemm_mx_swiglu_quant_h13(const void* A, const void* sfa, const void* B, const void* sfb, void* act_q,
                                             void* act_sf, void* h13, int M, int N, int K, int E, const int* tile_expert,
                                             const int* n_m_tiles, long long a_rows, long long b_rows, int fp4, int bn,
                                             void* status, cudaStream_t st);

extern "C" int nmoe_gemm_mx_swiglu_quant(const void* A, const void* sfa, const void* B, const void* sfb, void* act_q,
                                         void* act_sf, int M, int N, int K, int E, const int* tile_expert,
                                         const int* n_m_tiles, long long a_rows, long long b_rows, int fp4, int bn,
                                         void* status, cudaStream_t st) {
  return nmoe_gemm_mx_swiglu_quant_h13(A, sfa, B, sfb, act_q, act_sf, nullptr, M, N, K, E, tile_expert, n_m_tiles, a_rows,
                                       b_rows, fp4, bn, status, st);
}

// Same, and when h13 != nullptr the epilogue also writes the bf16 up/gate output H13 [a_rows, N] (for a backward that
// keeps it instead of recomputing it).
extern "C" int nmoe_gemm_mx_swiglu_quant_h13(const void* A, const void* sfa, const void* B, const void* sfb, void* act_q,
                                             void* act_sf, void* h13, int M, int N, int K, int E, const int* tile_expert,
                                             const int* n_m_tiles, long long a_rows, long long b_rows, int fp4, int bn,
                                             void* status, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % (fp4 ? 128 : 32)) != 0 || (N % 128) != 0) return -1;
  if (bn == 0) bn = (N % 256 == 0) ? 256 : 128;
  if (bn != 128 && bn != 256) return -5;
  MxParams p;
  p.M = M; p.N = N; p.K = K; p.E = E; p.tile_expert = tile_expert; p.n_m_tiles = n_m_tiles;
  p.C = static_cast<__nv_bfloat16*>(h13); p.ldc = N;
  p.sfa = static_cast<const uint8_t*>(sfa); p.sfb = static_cast<const uint8_t*>(sfb);
  p.status = static_cast<StatusRecord*>(status);
  p.push_runs = nullptr; p.push_pairs = 0; p.push_world = 0; p.push_bulk = 0; p.alpha = 1.f; p.alpha_dev = nullptr;
  for (int r = 0; r < 8; ++r) p.peer_ret[r] = nullptr;
  p.act_q = static_cast<uint8_t*>(act_q); p.act_sf = static_cast<uint8_t*>(act_sf);
  p.act_sf_cols = (((N / 2) / 32) + 3) & ~3; p.act_fp4 = fp4;
  const int kb = fp4 ? K / 2 : K;
  CUtensorMap tmA, tmB;
  int rc = mx_cached_map(&tmA, A, kb, a_rows, kb, MX_BK, MX_BM);
  if (rc != 0) return rc;
  rc = mx_cached_map(&tmB, B, kb, b_rows, kb, MX_BK, bn);
  if (rc != 0) return rc;
  const int max_tiles = ((M + MX_BM - 1) / MX_BM) * ((N + bn - 1) / bn);
  if (fp4) return bn == 256 ? mx_launch<256, 1, 1>(tmA, tmB, p, max_tiles, st) : mx_launch<128, 1, 1>(tmA, tmB, p, max_tiles, st);
  return bn == 256 ? mx_launch<256, 1, 0>(tmA, tmB, p, max_tiles, st) : mx_launch<128, 1, 0>(tmA, tmB, p, max_tiles, st);
}
