// Host-side creation of TMA tensor maps.  The driver entry point is resolved at
// run time through the CUDA runtime, so the library does not link libcuda and
// still loads on a machine without a driver (the CPU build check).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nmoe {

enum TmaDtype { kTmaU8 = 0, kTmaBf16 = 1, kTmaF32 = 2 };
enum TmaSwizzle { kTmaSwizzleNone = 0, kTmaSwizzle32 = 1, kTmaSwizzle64 = 2, kTmaSwizzle128 = 3 };

// 2-D row-major tensor [outer, inner] with row pitch `pitch_bytes`, copied in boxes of
// [box_outer, box_inner].  Returns 0 on success, a CUresult / cudaError code otherwise.
// Requirements checked here: base 16-byte aligned, pitch multiple of 16, box_inner * elem
// multiple of 16 and (with swizzle) not wider than the swizzle span.
int make_tensor_map_2d(CUtensorMap* out, const void* base, TmaDtype dtype, uint64_t inner, uint64_t outer,
                       uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, TmaSwizzle swizzle);

}  // namespace nmoe
