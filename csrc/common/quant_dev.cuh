// Device helpers shared by the quantising kernels: load a 32-element bf16 block, quantise it to
// E4M3 with a power-of-two (E8M0) scale, pack and store 32 bytes.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "ptx.cuh"
#include "sf_layout.cuh"

namespace nmoe {

constexpr float kInvFp8Max = 1.f / 448.f;
constexpr float kInvFp4Max = 1.f / 6.f;

NMOE_DEVICE uint32_t pack4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Quantise 32 floats; returns the scale byte and the 32 output bytes in w[8].
NMOE_DEVICE uint8_t quant_block_e4m3_regs(const float* v, uint32_t* w) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const uint8_t sf = e8m0_from_amax(amax, kInvFp8Max);
  const float inv = e8m0_inv_scale(sf);
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = pack4_e4m3(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
  return sf;
}

NMOE_DEVICE uint8_t quant_block_e4m3(const float* v, uint8_t* dst) {
  uint32_t w[8];
  const uint8_t sf = quant_block_e4m3_regs(v, w);
  reinterpret_cast<int4*>(dst)[0] = make_int4(w[0], w[1], w[2], w[3]);
  reinterpret_cast<int4*>(dst)[1] = make_int4(w[4], w[5], w[6], w[7]);
  return sf;
}

// E2M1 code (sign | 3 bits) of x: round to nearest on the grid 0,.5,1,1.5,2,3,4,6, ties to the even mantissa bit.
NMOE_DEVICE uint32_t e2m1_code(float x) {
  const float a = fabsf(x);
  uint32_t c;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.f) c = 6;
  else c = 7;
  return c | (x < 0.f ? 8u : 0u);
}

// Quantise 32 floats to E2M1 nibbles (low nibble = even element); returns the E8M0 scale byte, 16 output bytes in w[4].
NMOE_DEVICE uint8_t quant_block_e2m1_regs(const float* v, uint32_t* w) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const uint8_t sf = e8m0_from_amax(amax, kInvFp4Max);
  const float inv = e8m0_inv_scale(sf);
  w[0] = w[1] = w[2] = w[3] = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) w[i >> 3] |= e2m1_code(v[i] * inv) << ((i & 7) * 4);
  return sf;
}

NMOE_DEVICE void load_block_bf16(const __nv_bfloat16* src, float* v) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int4 p = ld_nc_v4(reinterpret_cast<const int4*>(src) + i);
    const float2 a = unpack_bf16x2(p.x), b = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
    v[8 * i] = a.x; v[8 * i + 1] = a.y; v[8 * i + 2] = b.x; v[8 * i + 3] = b.y;
    v[8 * i + 4] = c.x; v[8 * i + 5] = c.y; v[8 * i + 6] = d.x; v[8 * i + 7] = d.y;
  }
}

}  // namespace nmoe
