// Warp-level transposing store for GEMM epilogues whose rows go to unrelated addresses (the fused
// RDEP return: every accumulator row is pushed to its own (rank, token, slot) row, most of them
// over NVLink).  After tcgen05.ld each lane holds 64 consecutive fp32 columns of ITS row, so a
// direct store instruction would touch 32 rows x 16 bytes.  Going through a 4 KB per-warp
// shared-memory tile, every store instruction instead writes 4 rows x 128 contiguous bytes,
// which is what keeps NVLink packets full.
#pragma once
#include <stdint.h>

#include "ptx.cuh"

namespace nmoe {

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

}  // namespace nmoe
