// Serving-side attention over a paged KV cache (the corpus-grading engine's decode path):
//   nmoe_kv_store       scatter this step's K/V rows into cache slots (slot < 0 = skip, e.g. padding
//                       or tokens whose block came from the prefix cache)
//   nmoe_paged_decode   one query token per sequence against its block table: causal over the
//                       cached context, optional sliding window, optional learned sink, GQA
// Decode is bandwidth-bound (every cached K/V byte is read once per step), so this is a plain
// SIMT kernel: one CTA per (sequence, kv head), one warp per query head of the group (all warps
// read the same K/V lines, so they hit L1 after the first), one lane (two for D = 128) per cached
// token with a private online-softmax state that is merged across the warp at the end.
// Cache layout: [num_blocks, block_size, Hkv, D] bf16 (slot = block * block_size + offset).
//
// Replaces the Triton kernels of the reference engine (nmoe/data/model.py:145-304).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "common/ptx.cuh"

namespace nmoe {

__global__ void __launch_bounds__(256)
k_kv_store(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ k_cache,
           __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ slots, int n_tokens, int row_elems,
           long long k_stride, long long v_stride) {
  const int vec_per_row = row_elems >> 3;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(n_tokens) * vec_per_row) return;
  const int tok = static_cast<int>(idx / vec_per_row), c = static_cast<int>(idx % vec_per_row);
  const int slot = slots[tok];
  if (slot < 0) return;
  reinterpret_cast<int4*>(k_cache + static_cast<long long>(slot) * row_elems)[c] = ld_nc_v4(k + tok * k_stride + c * 8);
  reinterpret_cast<int4*>(v_cache + static_cast<long long>(slot) * row_elems)[c] = ld_nc_v4(v + tok * v_stride + c * 8);
}

// LPT lanes share one cached token (each owns D/LPT of the head dim), so that the per-lane
// state (query slice + accumulator slice) stays in registers: LPT = 1 for D = 64, 2 for D = 128.
template <int D, int LPT>
__global__ void __launch_bounds__(256)
k_paged_decode(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
               const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables,
               const int* __restrict__ context_lens, const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out,
               int Hq, int Hkv, int block_size, int max_blocks, int window, float scale_log2) {
  constexpr int DP = D / LPT;               // dims per lane
  constexpr int TPW = 32 / LPT;             // tokens per warp iteration
  const int b = blockIdx.x, hkv = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_warps = blockDim.x >> 5;
  const int group = Hq / Hkv;
  const int part = lane / TPW, tl = lane % TPW;
  const int ctx = context_lens[b];
  const int start = (window > 0 && ctx > window) ? ctx - window : 0;
  const int* bt = block_tables + static_cast<long long>(b) * max_blocks;
  const long long row = static_cast<long long>(Hkv) * D;
  for (int hg = warp; hg < group; hg += n_warps) {
    const int h = hkv * group + hg;
    float qf[DP];
    const __nv_bfloat16* qp = q + (static_cast<long long>(b) * Hq + h) * D + part * DP;
#pragma unroll
    for (int i = 0; i < DP / 8; ++i) {
      const int4 p = ld_nc_v4(qp + i * 8);
      const float2 a = unpack_bf16x2(p.x), bb = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
      qf[8 * i] = a.x; qf[8 * i + 1] = a.y; qf[8 * i + 2] = bb.x; qf[8 * i + 3] = bb.y;
      qf[8 * i + 4] = c.x; qf[8 * i + 5] = c.y; qf[8 * i + 6] = d.x; qf[8 * i + 7] = d.y;
    }
    float m = -1e30f, l = 0.f, acc[DP];
#pragma unroll
    for (int i = 0; i < DP; ++i) acc[i] = 0.f;
    // every lane of the warp runs the same number of iterations (the shuffle below needs all of them)
    for (int t0 = start; t0 < ctx; t0 += TPW) {
      const int t = t0 + tl;
      const bool live = t < ctx;
      const long long slot = live ? static_cast<long long>(bt[t / block_size]) * block_size + (t % block_size) : 0;
      const __nv_bfloat16* kp = k_cache + slot * row + hkv * D + part * DP;
      const __nv_bfloat16* vp = v_cache + slot * row + hkv * D + part * DP;
      float s = 0.f;
      if (live) {
#pragma unroll
        for (int i = 0; i < DP / 8; ++i) {
          const int4 p = *reinterpret_cast<const int4*>(kp + i * 8);
          const float2 a = unpack_bf16x2(p.x), bb = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
          s += qf[8 * i] * a.x + qf[8 * i + 1] * a.y + qf[8 * i + 2] * bb.x + qf[8 * i + 3] * bb.y +
               qf[8 * i + 4] * c.x + qf[8 * i + 5] * c.y + qf[8 * i + 6] * d.x + qf[8 * i + 7] * d.y;
        }
      }
      if (LPT == 2) s += __shfl_xor_sync(0xffffffffu, s, 16);
      if (!live) continue;
      s *= scale_log2;
      const float m_new = fmaxf(m, s);
      const float alpha = exp2f(m - m_new), p_t = exp2f(s - m_new);
      l = l * alpha + p_t;
#pragma unroll
      for (int i = 0; i < DP / 8; ++i) {
        const int4 p = *reinterpret_cast<const int4*>(vp + i * 8);
        const float2 a = unpack_bf16x2(p.x), bb = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
        acc[8 * i] = acc[8 * i] * alpha + p_t * a.x;          acc[8 * i + 1] = acc[8 * i + 1] * alpha + p_t * a.y;
        acc[8 * i + 2] = acc[8 * i + 2] * alpha + p_t * bb.x; acc[8 * i + 3] = acc[8 * i + 3] * alpha + p_t * bb.y;
        acc[8 * i + 4] = acc[8 * i + 4] * alpha + p_t * c.x;  acc[8 * i + 5] = acc[8 * i + 5] * alpha + p_t * c.y;
        acc[8 * i + 6] = acc[8 * i + 6] * alpha + p_t * d.x;  acc[8 * i + 7] = acc[8 * i + 7] * alpha + p_t * d.y;
      }
      m = m_new;
    }
    // merge the per-lane states of the TPW lanes that share a slice of the head dim
    float m_all = warp_max(m);
    const float sink2 = sinks != nullptr ? sinks[h] * 1.4426950408889634f : -1e30f;
    m_all = fmaxf(m_all, sink2);
    const float w = exp2f(m - m_all);
    float l_all = l * w;
#pragma unroll
    for (int off = TPW / 2; off > 0; off >>= 1) l_all += __shfl_xor_sync(0xffffffffu, l_all, off);
    if (sinks != nullptr) l_all += exp2f(sink2 - m_all);
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    __nv_bfloat16* op = out + (static_cast<long long>(b) * Hq + h) * D + part * DP;
#pragma unroll
    for (int i = 0; i < DP; ++i) {
      float v_i = acc[i] * w;
#pragma unroll
      for (int off = TPW / 2; off > 0; off >>= 1) v_i += __shfl_xor_sync(0xffffffffu, v_i, off);
      if (tl == (i % TPW)) op[i] = __float2bfloat16(v_i * inv);
    }
  }
}

}  // namespace nmoe

using namespace nmoe;

// k, v: [n_tokens, Hkv*D] rows (row strides in elements given separately so views of a fused qkv
// projection work); caches [num_slots, Hkv*D]; slots [n_tokens] int32.
extern "C" int nmoe_kv_store(const void* k, const void* v, void* k_cache, void* v_cache, const int* slots, int n_tokens,
                             int row_elems, long long k_stride, long long v_stride, cudaStream_t st) {
  if (n_tokens == 0) return 0;
  if ((row_elems | k_stride | v_stride) % 8 != 0) return -1;
  const long long n = static_cast<long long>(n_tokens) * (row_elems / 8);
  k_kv_store<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), static_cast<__nv_bfloat16*>(k_cache),
      static_cast<__nv_bfloat16*>(v_cache), slots, n_tokens, row_elems, k_stride, v_stride);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// q, out: [B, Hq, D] bf16; block_tables [B, max_blocks] int32; context_lens [B] int32 (tokens in the
// cache INCLUDING the current one, which must already be stored); sinks [Hq] fp32 or null.
extern "C" int nmoe_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                 const int* context_lens, const float* sinks, void* out, int B, int Hq, int Hkv, int D,
                                 int block_size, int max_blocks, int window, float scale, cudaStream_t st) {
  if (B == 0) return 0;
  if (Hq % Hkv != 0) return -1;
  dim3 grid(B, Hkv);
  const int threads = 32 * ((Hq / Hkv) < 8 ? (Hq / Hkv) : 8);
  const float sl2 = scale * 1.4426950408889634f;
  if (D == 64)
    k_paged_decode<64, 1><<<grid, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
        static_cast<const __nv_bfloat16*>(v_cache), block_tables, context_lens, sinks, static_cast<__nv_bfloat16*>(out), Hq, Hkv,
        block_size, max_blocks, window, sl2);
  else if (D == 128)
    k_paged_decode<128, 2><<<grid, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
        static_cast<const __nv_bfloat16*>(v_cache), block_tables, context_lens, sinks, static_cast<__nv_bfloat16*>(out), Hq, Hkv,
        block_size, max_blocks, window, sl2);
  else
    return -2;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
