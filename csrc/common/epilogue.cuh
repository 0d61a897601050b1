// Warp-level transposing store for GEMM epilogues whose rows go to unrelated addresses (the fused
// RDEP return: every accumulator row is pushed to its own (rank, token, slot) row, most of them
// over NVLink).  After tcgen05.ld each lane holds 64 consecutive fp32 columns of ITS row, so a
// direct store instruction would touch 32 rows x 16 bytes.  Going through a 4 KB per-warp
// shared-memory tile, every store instruction instead writes 4 rows x 128 contiguous bytes,
// which is what keeps NVLink packets full.
#pragma once
#include <stdint.h>
#include <stdlib.h>

#include "ptx.cuh"

namespace nmoe {

// Host side: which form of the fused-return epilogue a launch uses.  NMOE_PUSH_BULK (bf16 GEMMs, default 1 = bulk
// copies of 256-byte row segments) and NMOE_PUSH_BULK_MX (block-scaled GEMM, default 0 = 16-byte stores: its single
// accumulator leaves the epilogue exposed, and there the 128-byte copies measured slower than the stores).
inline int epi_push_bulk_enabled(bool mx = false) {
  static int v[2] = {-1, -1};
  int& r = v[mx ? 1 : 0];
  if (r < 0) {
    const char* e = getenv(mx ? "NMOE_PUSH_BULK_MX" : "NMOE_PUSH_BULK");
    r = e != nullptr ? (e[0] != '0' ? 1 : 0) : (mx ? 0 : 1);
  }
  return r;
}

// SwiGLU backward as the epilogue of the GEMM that produces dA = dY W2^T (one accumulator row per lane).
// With h13 = [gate | up] interleaved (gate in even columns), s = sigmoid(gate), A = gate * s * up and the row's routing
// weight sc:   d(gate) = sc dA up s (1 + gate (1 - s)),   d(up) = sc dA gate s,   a_out = sc A   (operand of dW2),
// and <A, dA> summed over the row is the gradient of the routing weight.  dA itself is never written.  The accumulator
// is rounded to bf16 first, so dh13 and a_out are bit-identical to the two-kernel form (GEMM storing bf16 dA, then
// k_swiglu_bwd).  rowdot_parts[n_tile][row] holds the partial dot product of each column tile: plain stores, summed
// afterwards in a fixed order, so the result does not depend on scheduling.
// Replaces k_swiglu_bwd_bf16 / k_dgate_from_adA_bf16 of the reference (nmoe/csrc/quant.cu:781, nmoe/csrc/rdep.cu:3517).
struct SwigluBwdEpi {
  const __nv_bfloat16* h13;     // [rows, 2N]; nullptr = epilogue off
  __nv_bfloat16* dh13;          // [rows, 2N]
  __nv_bfloat16* a_out;         // [rows, N] or nullptr
  const float* row_scale;       // [rows] or nullptr (1)
  float* rowdot_parts;          // [ceil(N / tile columns), rows_cap] or nullptr
  long long rows_cap;
};

// Each lane owns one accumulator row, but rows are 2N (h13, dh13) or N (a_out) elements apart in memory, so a lane that
// touched its own row directly would make every load / store instruction hit 32 different lines, and four epilogue
// warps cannot issue enough of those.  Rows therefore go through two 4 KB shared-memory tiles per warp (16-byte chunks
// XOR-swizzled by row, conflict-free in both directions): every global instruction moves 4 rows x 128 contiguous bytes
// (h13, dh13) or 8 rows x 64 bytes (a_out).  row0 = first row of the warp's 32-row slab, rows_ok = rows of it that exist.
NMOE_DEVICE void sb_issue_loads(int4 (&g)[8], const __nv_bfloat16* h13, long long row0, int rows_ok, long long n2, int col,
                                int lane) {
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = it * 4 + (lane >> 3);
    g[it] = row < rows_ok ? ld_nc_v4(h13 + (row0 + row) * n2 + 2 * col + (lane & 7) * 8) : make_int4(0, 0, 0, 0);
  }
}
NMOE_DEVICE void sb_stage_h(uint8_t* t0, const int4 (&g)[8], int lane) {
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = it * 4 + (lane >> 3);
    *reinterpret_cast<int4*>(t0 + row * 128 + (((lane & 7) ^ (row & 7)) << 4)) = g[it];
  }
}

// r: 32 accumulator columns [col, col + 32) of this lane's row (dA).  t0 holds the warp's h13 tile for these columns
// (staged and visible); t1 is scratch.  All 32 lanes must call.
NMOE_DEVICE void swiglu_bwd_cols32(const uint32_t* r, uint8_t* t0, uint8_t* t1, __nv_bfloat16* dh13, __nv_bfloat16* a_out,
                                   long long row0, int rows_ok, long long n, int col, float sc, float& dot, int lane) {
  int4 h[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) h[j] = *reinterpret_cast<const int4*>(t0 + lane * 128 + ((j ^ (lane & 7)) << 4));
  __syncwarp();                                   // every lane has its h13 row: t0 may be overwritten
  uint32_t aw[4];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t* hw = reinterpret_cast<const uint32_t*>(&h[j]);
    uint32_t ow[4];
    float av[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 gu = unpack_bf16x2(hw[i]);                      // x = gate, y = up
      const float d = __bfloat162float(__float2bfloat16(__uint_as_float(r[4 * j + i])));
      const float s = 1.f / (1.f + __expf(-gu.x));
      const float a = gu.x * s * gu.y;
      dot += a * d;
      const float gd = d * sc;
      ow[i] = pack_bf16x2(gd * gu.y * s * (1.f + gu.x * (1.f - s)), gd * gu.x * s);
      av[i] = a * sc;
    }
    *reinterpret_cast<int4*>(t1 + lane * 128 + ((j ^ (lane & 7)) << 4)) = make_int4(ow[0], ow[1], ow[2], ow[3]);
    aw[2 * (j & 1)] = pack_bf16x2(av[0], av[1]);
    aw[2 * (j & 1) + 1] = pack_bf16x2(av[2], av[3]);
    if (j & 1)       // 8 activations = one 16-byte chunk of the 64-byte a_out row; rows 64 bytes apart, swizzled by row pair
      *reinterpret_cast<int4*>(t0 + lane * 64 + (((j >> 1) ^ ((lane >> 1) & 3)) << 4)) = make_int4(aw[0], aw[1], aw[2], aw[3]);
  }
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = it * 4 + (lane >> 3);
    const int4 v = *reinterpret_cast<const int4*>(t1 + row * 128 + (((lane & 7) ^ (row & 7)) << 4));
    if (row < rows_ok) *reinterpret_cast<int4*>(dh13 + (row0 + row) * 2 * n + 2 * col + (lane & 7) * 8) = v;
  }
  if (a_out != nullptr) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int row = it * 8 + (lane >> 2);
      const int4 v = *reinterpret_cast<const int4*>(t0 + row * 64 + (((lane & 3) ^ ((row >> 1) & 3)) << 4));
      if (row < rows_ok) *reinterpret_cast<int4*>(a_out + (row0 + row) * n + col + (lane & 3) * 8) = v;
    }
  }
  __syncwarp();                                   // both tiles are free again
}

// Return runs of the expert-parallel layer (csrc/rdep.cu): inside an expert's segment of the owner's buffer the rows of
// one source rank are contiguous, and they go back as one contiguous block of that source's return buffer.
// runs = [3][n_local][world]: first row of the run in the owner's buffer, its length, its first row at the source.
// Which source owns row r of the owner's buffer (expert le), and where the row goes in that source's return buffer.
// False for padding rows and for rows of a dropped expert.
NMOE_DEVICE bool run_lookup(const int* __restrict__ runs, int n_local, int world, int le, int r, int& src, int& drow) {
  const int nlw = n_local * world;
  const int* start = runs + le * world;
#pragma unroll 1
  for (int s = 0; s < world; ++s) {
    const int off = r - __ldg(start + s);
    if (off >= 0 && off < __ldg(start + nlw + s)) {
      src = s;
      drow = __ldg(start + 2 * nlw + s) + off;
      return true;
    }
  }
  return false;
}

constexpr int kEpiStageBytesPerWarp = 32 * 128;

// r: 64 fp32 accumulator values (as bits) of this lane's row; scale: multiplier applied before
// the bf16 conversion; row_dst: where this lane's 128-byte row segment goes (nullptr = skip the
// row; must be 16-byte aligned); stage: this warp's 4 KB staging tile.  All 32 lanes must call.
NMOE_DEVICE void warp_store_rows_64cols(uint8_t* stage, const uint32_t* r, float scale, __nv_bfloat16* row_dst, int lane) {
  int4* srow = reinterpret_cast<int4*>(stage + lane * 128);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int4 v;
    v.x = pack_bf16x2(__uint_as_float(r[8 * j]) * scale, __uint_as_float(r[8 * j + 1]) * scale);
    v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * scale, __uint_as_float(r[8 * j + 3]) * scale);
    v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * scale, __uint_as_float(r[8 * j + 5]) * scale);
    v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * scale, __uint_as_float(r[8 * j + 7]) * scale);
    srow[j ^ (lane & 7)] = v;                 // 16-byte chunks XOR-swizzled by row: conflict-free both ways
  }
  __syncwarp();
  const unsigned long long mine = reinterpret_cast<unsigned long long>(row_dst);
  const int j = lane & 7;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = it * 4 + (lane >> 3);
    const unsigned long long dst = __shfl_sync(0xffffffffu, mine, row);
    const int4 v = reinterpret_cast<const int4*>(stage + row * 128)[j ^ (row & 7)];
    if (dst != 0ull) st_relaxed_sys_v4(reinterpret_cast<int4*>(dst) + j, v);
  }
  __syncwarp();
}

// ---------------------------------------------------------------------------------------------------------------
// Copy-engine variant: the lane converts its row segment into its own shared-memory staging row and then hands the
// whole segment to the bulk-copy (TMA) unit with one `cp.async.bulk.global.shared::cta`.  The warp is free again as
// soon as the copy is issued; the bytes (most of them bound for another GPU) travel while the next accumulator
// columns are being converted, and the number of stores in flight no longer depends on how many warps the epilogue
// has.  SEG_BYTES = 256 stages 128 columns per copy, 128 stages 64 columns (for kernels short of shared memory).
//
// Staging rows are laid out so that the 32 lanes' 16-byte stores spread over all banks:
//   128-byte segments: row stride 144 bytes;  256-byte segments: rows in pairs, 528 bytes per pair.
// Every row start is 16-byte aligned, as the bulk copy requires.
template <int SEG_BYTES>
struct EpiBulk {
  static_assert(SEG_BYTES == 128 || SEG_BYTES == 256, "segment size");
  static constexpr int kWarpBytes = SEG_BYTES == 128 ? 32 * 144 : 16 * 528;
  static constexpr int kSegCols = SEG_BYTES / 2;
  static NMOE_DEVICE uint8_t* row(uint8_t* warp_stage, int lane) {
    return SEG_BYTES == 128 ? warp_stage + lane * 144 : warp_stage + (lane >> 1) * 528 + (lane & 1) * 256;
  }
};

// 64 fp32 accumulator values of this lane's row -> bf16 (times scale) at byte offset `off` of its staging row.
NMOE_DEVICE void stage_64cols(uint8_t* srow, int off, const uint32_t* r, float scale) {
  int4* d = reinterpret_cast<int4*>(srow + off);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int4 v;
    v.x = pack_bf16x2(__uint_as_float(r[8 * j]) * scale, __uint_as_float(r[8 * j + 1]) * scale);
    v.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]) * scale, __uint_as_float(r[8 * j + 3]) * scale);
    v.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]) * scale, __uint_as_float(r[8 * j + 5]) * scale);
    v.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]) * scale, __uint_as_float(r[8 * j + 7]) * scale);
    d[j] = v;
  }
}

// Issue the copy of this lane's staged segment to dst (null: the row is padding, nothing is sent) and close the
// thread's bulk group.  The caller must have made its staging writes visible to the copy unit (epi_bulk_fence).
NMOE_DEVICE void epi_bulk_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
NMOE_DEVICE void epi_bulk_store(void* dst, const uint8_t* srow, uint32_t bytes) {
  if (dst != nullptr)
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(dst), "r"(smem_u32(srow)), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Before a lane rewrites its staging row: its earlier copies have finished READING shared memory.
NMOE_DEVICE void epi_bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Before the kernel ends (and before any flag that publishes the rows): the lane's copies are complete.
NMOE_DEVICE void epi_bulk_drain() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  asm volatile("fence.proxy.async;" ::: "memory");
}

}  // namespace nmoe
