#include "tensormap.h"

#include <mutex>

namespace nmoe {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn resolve_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

int make_tensor_map_2d(CUtensorMap* out, const void* base, TmaDtype dtype, uint64_t inner, uint64_t outer,
                       uint64_t pitch_bytes, uint32_t box_inner, uint32_t box_outer, TmaSwizzle swizzle) {
  EncodeFn fn = resolve_encode();
  if (fn == nullptr) return -100;
  CUtensorMapDataType dt;
  uint32_t esz;
  switch (dtype) {
    case kTmaU8: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; esz = 1; break;
    case kTmaBf16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; esz = 2; break;
    default: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; esz = 4; break;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return -101;
  if (pitch_bytes % 16 != 0) return -102;
  if ((box_inner * esz) % 16 != 0) return -103;
  if (box_inner > 256 || box_outer > 256) return -104;
  static const uint32_t span[4] = {0, 32, 64, 128};
  if (swizzle != kTmaSwizzleNone && box_inner * esz > span[swizzle]) return -105;
  CUtensorMapSwizzle sw = swizzle == kTmaSwizzle128  ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle == kTmaSwizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == kTmaSwizzle32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                     : CU_TENSOR_MAP_SWIZZLE_NONE;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -200 - static_cast<int>(r);
}

}  // namespace nmoe
