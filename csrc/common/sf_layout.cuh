// Scale-factor layout consumed by block-scaled tcgen05.mma: 128-row x 4-column atoms of 512
// bytes, tiled row-major over (row / 128, sf_col / 4).  Inside an atom the byte of (row m,
// scale column k) sits at (m % 32) * 16 + ((m / 32) % 4) * 4 + (k % 4), i.e. 32 "lanes" of 16
// bytes, which is exactly what one tcgen05.cp 32x128b.warpx4 moves into tensor memory.
// (Same contract as the reference's nmoe/csrc/swizzle.cuh:33-54.)
#pragma once
#include <stdint.h>

namespace nmoe {

__host__ __device__ __forceinline__ size_t sf_atom_index(int m, int k, int sf_cols_padded) {
  return static_cast<size_t>(m >> 7) * (sf_cols_padded >> 2) + (k >> 2);
}
__host__ __device__ __forceinline__ size_t sf_mma_offset(int m, int k, int sf_cols_padded) {
  return sf_atom_index(m, k, sf_cols_padded) * 512 + (m & 31) * 16 + ((m >> 5) & 3) * 4 + (k & 3);
}

// Smallest power of two >= amax / qmax as an E8M0 byte (value 2^(b-127)); zero block -> 127.
__host__ __device__ __forceinline__ uint8_t e8m0_from_amax(float amax, float inv_qmax) {
  const float r = amax * inv_qmax;
  if (!(r > 0.f)) return 127;
  uint32_t bits;
#ifdef __CUDA_ARCH__
  bits = __float_as_uint(r);
#else
  union { float f; uint32_t u; } cv; cv.f = r; bits = cv.u;
#endif
  uint32_t e = (bits >> 23) & 0xFF;
  const uint32_t man = bits & 0x7FFFFF;
  if (e == 0) e = man ? 1 : 0;          // subnormal ratio -> 2^-126
  else if (man) e += 1;
  return static_cast<uint8_t>(e > 254 ? 254 : e);
}
__host__ __device__ __forceinline__ float e8m0_inv_scale(uint8_t b) {
  // 2^(127-b) built directly in the exponent field (b in [1,253] covers every case reached here)
  const int e = 254 - static_cast<int>(b);
  uint32_t bits = static_cast<uint32_t>(e < 1 ? 1 : (e > 254 ? 254 : e)) << 23;
#ifdef __CUDA_ARCH__
  return __uint_as_float(bits);
#else
  union { float f; uint32_t u; } cv; cv.u = bits; return cv.f;
#endif
}

}  // namespace nmoe
