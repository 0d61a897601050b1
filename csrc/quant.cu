// Block-scaled quantisation: bf16 -> E4M3 with one E8M0 scale per 32 elements (MXFP8), scales
// written directly in the tensor-core atom layout (common/sf_layout.cuh); fused SwiGLU + quantise
// for the activation between the two expert GEMMs; dequantise for tests; E2M1 (4-bit) packing.
// One warp per row, each lane owns one 32-element block at a time (64-byte loads, 32-byte stores).
// Reference counterparts: nmoe/csrc/quant.cu:118-250 (quantise), :456-760 (SwiGLU+quantise),
// :51,1772 (dequantise).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/quant_dev.cuh"

namespace nmoe {

// x[M,K] bf16 -> q[M,K] e4m3, sf in atom layout with sf_cols = K/32 padded to a multiple of 4.
// rows_per_group > 0: the matrix is a stack of groups (experts) of that many rows, each with its
// own atom region (rows_per_group must be a multiple of 128).
__global__ void __launch_bounds__(256)
k_quant_mxfp8(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, long long M,
              int K, int sf_cols_padded, const int* __restrict__ n_tiles_dev) {
  if (n_tiles_dev != nullptr) M = min(M, static_cast<long long>(*n_tiles_dev) * 128);
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  const int nblk = K >> 5;
  for (int b = lane; b < nblk; b += 32) {
    float v[32];
    load_block_bf16(x + row * K + b * 32, v);
    const uint8_t s = quant_block_e4m3(v, q + row * K + b * 32);
    sf[sf_mma_offset(static_cast<int>(row), b, sf_cols_padded)] = s;
  }
}

// h13[M,2F] (gate even / up odd) -> a = silu(gate)*up quantised to e4m3 [M,F] + scales; optional bf16 copy.
__global__ void __launch_bounds__(256)
k_swiglu_quant_mxfp8(const __nv_bfloat16* __restrict__ h13, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                     long long M, int F, int sf_cols_padded, const int* __restrict__ n_tiles_dev) {
  if (n_tiles_dev != nullptr) M = min(M, static_cast<long long>(*n_tiles_dev) * 128);
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  const int nblk = F >> 5;
  for (int b = lane; b < nblk; b += 32) {
    float v[32];
    const __nv_bfloat16* src = h13 + row * 2 * F + b * 64;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int4 p = ld_nc_v4(reinterpret_cast<const int4*>(src) + i);
      const float2 a = unpack_bf16x2(p.x), bb = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
      // round through bf16 like the unfused path (swiglu writes bf16, then quantise reads it)
      v[4 * i] = __bfloat162float(__float2bfloat16(a.x / (1.f + __expf(-a.x)) * a.y));
      v[4 * i + 1] = __bfloat162float(__float2bfloat16(bb.x / (1.f + __expf(-bb.x)) * bb.y));
      v[4 * i + 2] = __bfloat162float(__float2bfloat16(c.x / (1.f + __expf(-c.x)) * c.y));
      v[4 * i + 3] = __bfloat162float(__float2bfloat16(d.x / (1.f + __expf(-d.x)) * d.y));
    }
    const uint8_t s = quant_block_e4m3(v, q + row * F + b * 32);
    sf[sf_mma_offset(static_cast<int>(row), b, sf_cols_padded)] = s;
  }
}

// Same for MXFP4 output: a = silu(gate)*up -> E2M1 nibbles [M,F/2] + scales.
__global__ void __launch_bounds__(256)
k_swiglu_quant_mxfp4(const __nv_bfloat16* __restrict__ h13, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                     long long M, int F, int sf_cols_padded, const int* __restrict__ n_tiles_dev) {
  if (n_tiles_dev != nullptr) M = min(M, static_cast<long long>(*n_tiles_dev) * 128);
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  const int nblk = F >> 5;
  for (int b = lane; b < nblk; b += 32) {
    float v[32];
    const __nv_bfloat16* src = h13 + row * 2 * F + b * 64;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int4 p = ld_nc_v4(reinterpret_cast<const int4*>(src) + i);
      const float2 a = unpack_bf16x2(p.x), bb = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
      v[4 * i] = __bfloat162float(__float2bfloat16(a.x / (1.f + __expf(-a.x)) * a.y));
      v[4 * i + 1] = __bfloat162float(__float2bfloat16(bb.x / (1.f + __expf(-bb.x)) * bb.y));
      v[4 * i + 2] = __bfloat162float(__float2bfloat16(c.x / (1.f + __expf(-c.x)) * c.y));
      v[4 * i + 3] = __bfloat162float(__float2bfloat16(d.x / (1.f + __expf(-d.x)) * d.y));
    }
    uint32_t w[4];
    const uint8_t s = quant_block_e2m1_regs(v, w);
    *reinterpret_cast<int4*>(q + row * (F >> 1) + b * 16) = make_int4(w[0], w[1], w[2], w[3]);
    sf[sf_mma_offset(static_cast<int>(row), b, sf_cols_padded)] = s;
  }
}

__global__ void k_dequant_mxfp8(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf,
                                __nv_bfloat16* __restrict__ out, long long M, int K, int sf_cols_padded) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= M * K) return;
  const long long row = i / K;
  const int col = static_cast<int>(i - row * K);
  const uint8_t s = sf[sf_mma_offset(static_cast<int>(row), col >> 5, sf_cols_padded)];
  const __half_raw h = __nv_cvt_fp8_to_halfraw(q[i], __NV_E4M3);
  const float f = __half2float(*reinterpret_cast<const __half*>(&h)) * exp2f(static_cast<float>(s) - 127.f);
  out[i] = __float2bfloat16(f);
}

// E2M1 (4-bit) with E8M0 scales per 32 elements: two values per byte, low nibble = even element.
__global__ void __launch_bounds__(256)
k_quant_mxfp4(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, long long M,
              int K, int sf_cols_padded) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  for (int b = lane; b < (K >> 5); b += 32) {
    float v[32];
    load_block_bf16(x + row * K + b * 32, v);
    uint32_t w[4];
    const uint8_t s = quant_block_e2m1_regs(v, w);
    *reinterpret_cast<int4*>(q + row * (K >> 1) + b * 16) = make_int4(w[0], w[1], w[2], w[3]);
    sf[sf_mma_offset(static_cast<int>(row), b, sf_cols_padded)] = s;
  }
}

// Expert AdamW fused with the refresh of the block-scaled weight cache: one pass over [rows, K] updates
// p / m / v (bf16 storage, fp32 math, decoupled decay first, as k_adamw_flat) and writes the quantised
// copy of the NEW weights (E4M3 or E2M1 + E8M0 atoms) that the next forward's expert GEMMs read.
// One warp per row, a lane owns one 32-element block at a time.
// Reference counterpart: expert_adamw_step emitting the fp8 / nvfp4 caches (nmoe/csrc/adamw.cu:73-489).
template <bool FP4>
__global__ void __launch_bounds__(256)
k_adamw_quant(__nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ g, __nv_bfloat16* __restrict__ m,
              __nv_bfloat16* __restrict__ v, long long rows, int K, float lr, float beta1, float beta2, float eps,
              float wd, float inv_bc1, float inv_bc2_sqrt, float grad_scale, uint8_t* __restrict__ q,
              uint8_t* __restrict__ sf, int sf_cols_padded) {
  // A thread owns 8 consecutive elements (one 16-byte vector of each tensor), so every load and store of a warp
  // covers 512 contiguous bytes; the four lanes that share a 32-element block agree on its scale with two shuffles.
  const long long nvec = rows * (K >> 3);
  const int vec_per_row = K >> 3;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int4 p4 = reinterpret_cast<const int4*>(p)[i];
    const int4 g4 = ld_nc_v4(reinterpret_cast<const int4*>(g) + i);
    const int4 m4 = reinterpret_cast<const int4*>(m)[i];
    const int4 v4 = reinterpret_cast<const int4*>(v)[i];
    const uint32_t* pw = reinterpret_cast<const uint32_t*>(&p4);
    const uint32_t* gw = reinterpret_cast<const uint32_t*>(&g4);
    const uint32_t* mw = reinterpret_cast<const uint32_t*>(&m4);
    const uint32_t* vw = reinterpret_cast<const uint32_t*>(&v4);
    float x[8];
    int4 po, mo, vo;
    uint32_t* pow_ = reinterpret_cast<uint32_t*>(&po);
    uint32_t* mow = reinterpret_cast<uint32_t*>(&mo);
    uint32_t* vow = reinterpret_cast<uint32_t*>(&vo);
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 pf = unpack_bf16x2(pw[j]), gf = unpack_bf16x2(gw[j]), mf = unpack_bf16x2(mw[j]), vf = unpack_bf16x2(vw[j]);
      // same operation order as k_adamw_flat, so the two optimisers stay bit-identical
      gf.x *= grad_scale; gf.y *= grad_scale;
      pf.x *= (1.f - lr * wd); pf.y *= (1.f - lr * wd);
      mf.x = beta1 * mf.x + (1.f - beta1) * gf.x; mf.y = beta1 * mf.y + (1.f - beta1) * gf.y;
      vf.x = beta2 * vf.x + (1.f - beta2) * gf.x * gf.x; vf.y = beta2 * vf.y + (1.f - beta2) * gf.y * gf.y;
      pf.x -= lr * inv_bc1 * mf.x / (sqrtf(vf.x) * inv_bc2_sqrt + eps);
      pf.y -= lr * inv_bc1 * mf.y / (sqrtf(vf.y) * inv_bc2_sqrt + eps);
      pow_[j] = pack_bf16x2(pf.x, pf.y); mow[j] = pack_bf16x2(mf.x, mf.y); vow[j] = pack_bf16x2(vf.x, vf.y);
      const float2 pr = unpack_bf16x2(pow_[j]);            // the cache is quantised from the stored bf16 value
      x[2 * j] = pr.x; x[2 * j + 1] = pr.y;
      amax = fmaxf(amax, fmaxf(fabsf(pr.x), fabsf(pr.y)));
    }
    reinterpret_cast<int4*>(p)[i] = po;
    reinterpret_cast<int4*>(m)[i] = mo;
    reinterpret_cast<int4*>(v)[i] = vo;
    const unsigned live = __activemask();       // the vector count is a multiple of 4: a block's four lanes leave together
    amax = fmaxf(amax, __shfl_xor_sync(live, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(live, amax, 2));
    const uint8_t sb = e8m0_from_amax(amax, FP4 ? kInvFp4Max : kInvFp8Max);
    const float inv = e8m0_inv_scale(sb);
    if (FP4) {
      uint32_t w = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) w |= e2m1_code(x[j] * inv) << (j * 4);
      reinterpret_cast<uint32_t*>(q)[i] = w;
    } else {
      int2 w;
      w.x = pack4_e4m3(x[0] * inv, x[1] * inv, x[2] * inv, x[3] * inv);
      w.y = pack4_e4m3(x[4] * inv, x[5] * inv, x[6] * inv, x[7] * inv);
      reinterpret_cast<int2*>(q)[i] = w;
    }
    if ((threadIdx.x & 3) == 0) {
      const long long row = i / vec_per_row;
      const int blk = static_cast<int>(i - row * vec_per_row) >> 2;
      sf[sf_mma_offset(static_cast<int>(row), blk, sf_cols_padded)] = sb;
    }
  }
}

// NVFP4: E2M1 values, one E4M3 scale per 16 elements (relative to the fp32 per-tensor scale *ts),
// scales in the atom layout with sf_cols = K/16 padded to a multiple of 4.  x ~= e2m1 * e4m3 * ts.
__global__ void __launch_bounds__(256)
k_quant_nvfp4(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, long long M,
              int K, int sf_cols_padded, const float* __restrict__ ts) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  const float tscale = *ts;
  for (int b = lane; b < (K >> 5); b += 32) {
    float v[32];
    load_block_bf16(x + row * K + b * 32, v);
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[16 * h + i]));
      const float want = fminf(amax / 6.f / tscale, 448.f);
      const __nv_fp8_storage_t sb = __nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3);
      const __half_raw hr = __nv_cvt_fp8_to_halfraw(sb, __NV_E4M3);
      const float denom = __half2float(*reinterpret_cast<const __half*>(&hr)) * tscale;
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int k = 16 * h + i;
        w[k >> 3] |= e2m1_code(denom > 0.f ? v[k] / denom : 0.f) << ((k & 7) * 4);
      }
      (void)inv;
      sf[sf_mma_offset(static_cast<int>(row), 2 * b + h, sf_cols_padded)] = sb;
    }
    *reinterpret_cast<int4*>(q + row * (K >> 1) + b * 16) = make_int4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace nmoe

using namespace nmoe;
#define CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return static_cast<int>(e_); } while (0)

extern "C" {

// Bytes of the scale buffer for [M,K] (M padded to 128 rows, K/32 padded to 4 columns).
long long nmoe_sf_bytes(long long M, int K) {
  const long long mt = (M + 127) / 128;
  const long long kt = ((K / 32) + 3) / 4;
  return mt * kt * 512;
}

int nmoe_quant_mxfp8(const void* x, void* q, void* sf, long long M, int K, const int* n_tiles_dev, cudaStream_t st) {
  if (M == 0) return 0;
  if (K % 32 != 0) return -1;
  const int sfc = ((K / 32) + 3) & ~3;
  k_quant_mxfp8<<<static_cast<unsigned>((M + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
      static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), M, K, sfc, n_tiles_dev);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_swiglu_quant_mxfp8(const void* h13, void* q, void* sf, long long M, int F, const int* n_tiles_dev,
                            cudaStream_t st) {
  if (M == 0) return 0;
  if (F % 32 != 0) return -1;
  const int sfc = ((F / 32) + 3) & ~3;
  k_swiglu_quant_mxfp8<<<static_cast<unsigned>((M + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h13),
      static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), M, F, sfc, n_tiles_dev);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_dequant_mxfp8(const void* q, const void* sf, void* out, long long M, int K, cudaStream_t st) {
  if (M == 0) return 0;
  const int sfc = ((K / 32) + 3) & ~3;
  const long long n = M * K;
  k_dequant_mxfp8<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(static_cast<const uint8_t*>(q),
      static_cast<const uint8_t*>(sf), static_cast<__nv_bfloat16*>(out), M, K, sfc);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_swiglu_quant_mxfp4(const void* h13, void* q, void* sf, long long M, int F, const int* n_tiles_dev,
                            cudaStream_t st) {
  if (M == 0) return 0;
  if (F % 32 != 0) return -1;
  const int sfc = ((F / 32) + 3) & ~3;
  k_swiglu_quant_mxfp4<<<static_cast<unsigned>((M + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h13),
      static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), M, F, sfc, n_tiles_dev);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_quant_mxfp4(const void* x, void* q, void* sf, long long M, int K, cudaStream_t st) {
  if (M == 0) return 0;
  if (K % 32 != 0) return -1;
  const int sfc = ((K / 32) + 3) & ~3;
  k_quant_mxfp4<<<static_cast<unsigned>((M + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
      static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), M, K, sfc);
  CHECK_LAUNCH();
  return 0;
}

// p, g, m, v: [rows, K] bf16; q: [rows, K] (E4M3) or [rows, K/2] (E2M1, fp4 != 0); sf: nmoe_sf_bytes(rows, K).
// rows must be a multiple of 128 per expert (they are: expert matrices are stacked), K % 32 == 0.
int nmoe_expert_adamw_quant(void* p, const void* g, void* m, void* v, long long rows, int K, float lr, float beta1,
                            float beta2, float eps, float wd, int step, float grad_scale, void* q, void* sf, int fp4,
                            cudaStream_t st) {
  if (rows == 0) return 0;
  if (K % 32 != 0) return -1;
  const float inv_bc1 = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  const float inv_bc2_sqrt = 1.f / sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  const int sfc = ((K / 32) + 3) & ~3;
  const long long nvec = rows * (K / 8);
  // One vector per thread (the loop in the kernel only matters beyond 2^31 blocks): with short-lived blocks the
  // hardware scheduler keeps every SM's load queues full, which a grid-stride loop whose body is ~200 instructions of
  // packing between its loads and the next ones does not (measured: 0.92 against 1.06 of the copy rate for the
  // plain AdamW kernel that is launched this way).
  long long want = (nvec + 255) / 256;
  const unsigned blocks = static_cast<unsigned>(want < 0x7fffffffLL ? want : 0x7fffffffLL);
  auto pp = static_cast<__nv_bfloat16*>(p);
  auto gg = static_cast<const __nv_bfloat16*>(g);
  auto mm = static_cast<__nv_bfloat16*>(m);
  auto vv = static_cast<__nv_bfloat16*>(v);
  if (fp4)
    k_adamw_quant<true><<<blocks, 256, 0, st>>>(pp, gg, mm, vv, rows, K, lr, beta1, beta2, eps, wd, inv_bc1, inv_bc2_sqrt,
                                                grad_scale, static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), sfc);
  else
    k_adamw_quant<false><<<blocks, 256, 0, st>>>(pp, gg, mm, vv, rows, K, lr, beta1, beta2, eps, wd, inv_bc1, inv_bc2_sqrt,
                                                 grad_scale, static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), sfc);
  CHECK_LAUNCH();
  return 0;
}

// ts: device pointer to the fp32 per-tensor scale (amax / (6 * 448)); sf buffer: nmoe_sf_bytes(M, 2 * K) bytes
// (one scale per 16 elements = twice the columns of the 32-element formats).
int nmoe_quant_nvfp4(const void* x, void* q, void* sf, long long M, int K, const float* ts, cudaStream_t st) {
  if (M == 0) return 0;
  if (K % 32 != 0) return -1;
  const int sfc = ((K / 16) + 3) & ~3;
  k_quant_nvfp4<<<static_cast<unsigned>((M + 7) / 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
      static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), M, K, sfc, ts);
  CHECK_LAUNCH();
  return 0;
}

}  // extern "C"
