// Memory-bound fused ops: RMSNorm fwd/bwd, rotary fwd/bwd, SwiGLU fwd/bwd, embedding
// gather with scale, flat AdamW.  One warp owns one row and moves it with 16-byte
// accesses; nothing here needs tensor cores, the target is HBM bandwidth.
//
// Replaces the reference's eager ops (nmoe/norm.py:14, nmoe/attention/rope.py:7-22,
// nmoe/model.py:48, nmoe/zero2.py:265-271) and nmoe/csrc/quant.cu:781 (SwiGLU bwd).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/ptx.cuh"

namespace nmoe {

constexpr int kWarpsPerBlock = 8;

union Pack8 {
  int4 v;
  __nv_bfloat162 h[4];
};

// ------------------------------------------------------------------ RMSNorm
// y = x * rsqrt(mean(x^2) + eps) * w ; rstd saved for backward.  H % 8 == 0.
template <int kMaxVec>   // kMaxVec 16-byte vectors per lane kept in registers (H <= kMaxVec*256)
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_rmsnorm_fwd(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
              __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int M, int H, float eps) {
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  const int4* xr = reinterpret_cast<const int4*>(x + static_cast<size_t>(row) * H);
  Pack8 xv[kMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
      xv[i].v = ld_nc_v4(xr + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(xv[i].h[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / static_cast<float>(H) + eps);
  if (lane == 0 && rstd != nullptr) rstd[row] = r;
  int4* yr = reinterpret_cast<int4*>(y + static_cast<size_t>(row) * H);
  const int4* wr = reinterpret_cast<const int4*>(w);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) {
      Pack8 wv, o;
      wv.v = __ldg(wr + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(xv[i].h[j]);
        float2 g = __bfloat1622float2(wv.h[j]);
        o.h[j] = __floats2bfloat162_rn(f.x * r * g.x, f.y * r * g.y);
      }
      yr[c] = o.v;
    }
  }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)); dw partial sums per block in fp32.
// Each block owns a contiguous range of rows and accumulates dw for them in registers,
// then the 8 warps reduce through shared memory and write one partial row.
template <int kMaxVec>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_rmsnorm_bwd(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
              const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
              __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int M, int H, int rows_per_block) {
  extern __shared__ float s_dw[];   // [kWarpsPerBlock][H]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  const int row0 = blockIdx.x * rows_per_block;
  const int row1 = min(M, row0 + rows_per_block);
  float acc[kMaxVec][8];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  Pack8 wv[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = lane + i * 32;
    if (c < nvec) wv[i].v = __ldg(reinterpret_cast<const int4*>(w) + c);
  }
  for (int row = row0 + warp; row < row1; row += kWarpsPerBlock) {
    const int4* xr = reinterpret_cast<const int4*>(x + static_cast<size_t>(row) * H);
    const int4* gr = reinterpret_cast<const int4*>(dy + static_cast<size_t>(row) * H);
    Pack8 xv[kMaxVec], gv[kMaxVec];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        xv[i].v = ld_nc_v4(xr + c);
        gv[i].v = ld_nc_v4(gr + c);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 xf = __bfloat1622float2(xv[i].h[j]);
          float2 gf = __bfloat1622float2(gv[i].h[j]);
          float2 wf = __bfloat1622float2(wv[i].h[j]);
          dot += gf.x * wf.x * xf.x + gf.y * wf.y * xf.y;
        }
      }
    }
    dot = warp_sum(dot);
    const float r = rstd[row];
    const float coef = dot * r * r * r / static_cast<float>(H);
    int4* dxr = reinterpret_cast<int4*>(dx + static_cast<size_t>(row) * H);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = lane + i * 32;
      if (c < nvec) {
        Pack8 o;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 xf = __bfloat1622float2(xv[i].h[j]);
          float2 gf = __bfloat1622float2(gv[i].h[j]);
          float2 wf = __bfloat1622float2(wv[i].h[j]);
          o.h[j] = __floats2bfloat162_rn(gf.x * wf.x * r - xf.x * coef, gf.y * wf.y * r - xf.y * coef);
          acc[i][2 * j] += gf.x * xf.x * r;
          acc[i][2 * j + 1] += gf.y * xf.y * r;
        }
        dxr[c] = o.v;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = lane + i * 32;
    if (c < nvec)
#pragma unroll
      for (int j = 0; j < 8; ++j) s_dw[warp * H + c * 8 + j] = acc[i][j];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int wv_ = 0; wv_ < kWarpsPerBlock; ++wv_) s += s_dw[wv_ * H + c];
    dw_partial[static_cast<size_t>(blockIdx.x) * H + c] = s;
  }
}

// Wide rows (H > 4096): rowdot[m] = sum_c dy*w*x, one warp per row ...
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_rmsnorm_rowdot(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                 float* __restrict__ rowdot, int M, int H) {
  const int row = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  const int4* xr = reinterpret_cast<const int4*>(x + static_cast<size_t>(row) * H);
  const int4* gr = reinterpret_cast<const int4*>(dy + static_cast<size_t>(row) * H);
  float dot = 0.f;
  for (int c = lane; c < (H >> 3); c += 32) {
    Pack8 xv, gv, wv;
    xv.v = ld_nc_v4(xr + c); gv.v = ld_nc_v4(gr + c); wv.v = __ldg(reinterpret_cast<const int4*>(w) + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = __bfloat1622float2(xv.h[j]), gf = __bfloat1622float2(gv.h[j]), wf = __bfloat1622float2(wv.h[j]);
      dot += gf.x * wf.x * xf.x + gf.y * wf.y * xf.y;
    }
  }
  dot = warp_sum(dot);
  if (lane == 0) rowdot[row] = dot;
}

// ... then a column-tiled pass: block (bx, by) owns 256 columns of a chunk of rows, one column per thread:
// dx = dy*w*r - x*coef, and the per-column sums of dy*x*r go to dw_partial[by][c].
__global__ void __launch_bounds__(256)
k_rmsnorm_bwd_wide(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const float* __restrict__ rstd, const float* __restrict__ rowdot, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int M, int H, int rows_per_block) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  const int row0 = blockIdx.y * rows_per_block;
  const int row1 = min(M, row0 + rows_per_block);
  if (c >= H) return;
  const float wf = __bfloat162float(w[c]);
  float acc = 0.f;
  for (int row = row0; row < row1; ++row) {
    const size_t i = static_cast<size_t>(row) * H + c;
    const float r = rstd[row];
    const float coef = rowdot[row] * r * r * r / static_cast<float>(H);
    const float g = __bfloat162float(dy[i]), xv = __bfloat162float(x[i]);
    dx[i] = __float2bfloat16(g * wf * r - xv * coef);
    acc += g * xv * r;
  }
  dw_partial[static_cast<size_t>(blockIdx.y) * H + c] = acc;
}

// Second pass for H <= 4096 after k_rmsnorm_rowdot: block (bx, by) owns up to 2048 columns of a chunk of rows, one
// 16-byte vector (8 columns) per thread, so a warp reads 512 contiguous bytes per row and the per-column sums
// live in eight registers.  Few registers per thread: the machine stays full, unlike the single-pass kernel whose
// 8 warps per SM (register-bound) left the copy rate at a quarter of peak.
__global__ void __launch_bounds__(256)
k_rmsnorm_bwd_cols(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const float* __restrict__ rstd, const float* __restrict__ rowdot, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int M, int H, int rows_per_block) {
  const int c = blockIdx.x * 256 + threadIdx.x;            // vector index inside the row
  const int nvec = H >> 3;
  const int row0 = blockIdx.y * rows_per_block;
  const int row1 = min(M, row0 + rows_per_block);
  if (c >= nvec) return;
  Pack8 wv;
  wv.v = __ldg(reinterpret_cast<const int4*>(w) + c);
  float wf[8], acc[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(wv.h[j]);
    wf[2 * j] = f.x; wf[2 * j + 1] = f.y;
    acc[2 * j] = 0.f; acc[2 * j + 1] = 0.f;
  }
  const float inv_h = 1.f / static_cast<float>(H);
#pragma unroll 4
  for (int row = row0; row < row1; ++row) {
    const size_t i = static_cast<size_t>(row) * nvec + c;
    Pack8 xv, gv, o;
    xv.v = ld_nc_v4(reinterpret_cast<const int4*>(x) + i);
    gv.v = ld_nc_v4(reinterpret_cast<const int4*>(dy) + i);
    const float r = rstd[row];
    const float coef = rowdot[row] * r * r * r * inv_h;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 xf = __bfloat1622float2(xv.h[j]), gf = __bfloat1622float2(gv.h[j]);
      o.h[j] = __floats2bfloat162_rn(gf.x * wf[2 * j] * r - xf.x * coef, gf.y * wf[2 * j + 1] * r - xf.y * coef);
      acc[2 * j] += gf.x * xf.x * r;
      acc[2 * j + 1] += gf.y * xf.y * r;
    }
    reinterpret_cast<int4*>(dx)[i] = o.v;
  }
  float* out = dw_partial + static_cast<size_t>(blockIdx.y) * H + c * 8;
  reinterpret_cast<float4*>(out)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  reinterpret_cast<float4*>(out)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// Same reduction with more parallelism (two-pass backward): a block owns 32 columns, its 8 warps take every 8th
// partial row (lane = column: 128-byte loads), then the warps' sums are combined in a fixed order.
__global__ void __launch_bounds__(256)
k_colsum32_to_bf16(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw, int nblocks, int H, int accumulate) {
  __shared__ float s[8][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 32 + lane;
  float acc = 0.f;
  if (c < H)
    for (int b = warp; b < nblocks; b += 8) acc += partial[static_cast<size_t>(b) * H + c];
  s[warp][lane] = acc;
  __syncthreads();
  if (warp == 0 && c < H) {
    float t = accumulate ? __bfloat162float(dw[c]) : 0.f;
#pragma unroll
    for (int w2 = 0; w2 < 8; ++w2) t += s[w2][lane];
    dw[c] = __float2bfloat16(t);
  }
}

// dw[c] = sum_b partial[b][c]  (+ existing dw when accumulate), written as bf16.
__global__ void k_colsum_to_bf16(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw, int nblocks, int H,
                                 int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = accumulate ? __bfloat162float(dw[c]) : 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[static_cast<size_t>(b) * H + c];
  dw[c] = __float2bfloat16(s);
}

// ------------------------------------------------------------------ rotary
// In place on x[row, offset : offset + D] for rows = B*S*h; position = (row / h) % S.
// Half-split convention: (x1, x2) -> (x1 c - x2 s, x2 c + x1 s); sign = -1 gives the transpose (backward).
__global__ void k_rope_inplace(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                               const float* __restrict__ sin_t, long long rows, int h, int S, long long row_stride,
                               int offset, int D, float sign) {
  const int half = D >> 1;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = rows * half;
  if (idx >= total) return;
  const long long row = idx / half;
  const int i = static_cast<int>(idx - row * half);
  const int pos = static_cast<int>((row / h) % S);
  __nv_bfloat16* p = x + row * row_stride + offset;
  const float c = cos_t[pos * half + i], s = sin_t[pos * half + i] * sign;
  const float a = __bfloat162float(p[i]), b = __bfloat162float(p[i + half]);
  p[i] = __float2bfloat16(a * c - b * s);
  p[i + half] = __float2bfloat16(b * c + a * s);
}

// ------------------------------------------------------------------ SwiGLU
// h13 is [M, 2F] with gate at even columns and up at odd columns; a[M,F] = silu(gate) * up.
__global__ void __launch_bounds__(256)
k_swiglu_fwd(const __nv_bfloat16* __restrict__ h13, __nv_bfloat16* __restrict__ a, long long M,
             int F, const int* __restrict__ n_tiles_dev) {
  if (n_tiles_dev != nullptr) M = min(M, static_cast<long long>(*n_tiles_dev) * 128);
  const long long nvec = M * (F >> 2);      // 4 outputs (8 inputs = 16 bytes) per vector
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  // grid-stride, two independent 16-byte loads in flight per thread
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < nvec; idx += 2 * stride) {
    const long long idx2 = idx + stride;
    Pack8 in[2];
    in[0].v = ld_nc_v4(reinterpret_cast<const int4*>(h13) + idx);
    if (idx2 < nvec) in[1].v = ld_nc_v4(reinterpret_cast<const int4*>(h13) + idx2);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (u == 1 && idx2 >= nvec) break;
      __nv_bfloat162 o[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float2 p0 = __bfloat1622float2(in[u].h[2 * j]);
        float2 p1 = __bfloat1622float2(in[u].h[2 * j + 1]);
        const float a0 = p0.x / (1.f + __expf(-p0.x)) * p0.y;
        const float a1 = p1.x / (1.f + __expf(-p1.x)) * p1.y;
        o[j] = __floats2bfloat162_rn(a0, a1);
      }
      reinterpret_cast<uint2*>(a)[u == 0 ? idx : idx2] = *reinterpret_cast<uint2*>(o);
    }
  }
}

// dh13 from (h13, da).  Optional per-row scale (the routing gate, applied to da) and
// optional per-row output rowdot[m] = <a[m,:], da[m,:]> (unscaled), which is the gradient
// of the routing gate by the identity dGate = <A, dA>.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_swiglu_bwd(const __nv_bfloat16* __restrict__ h13, const __nv_bfloat16* __restrict__ da,
             __nv_bfloat16* __restrict__ dh13, const float* __restrict__ row_scale, float* __restrict__ rowdot,
             __nv_bfloat16* __restrict__ a_out, long long M, int F, const int* __restrict__ n_tiles_dev) {
  if (n_tiles_dev != nullptr) M = min(M, static_cast<long long>(*n_tiles_dev) * 128);
  const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  const float sc = row_scale ? row_scale[row] : 1.f;
  const int4* hr = reinterpret_cast<const int4*>(h13 + row * 2 * F);
  const uint2* dr = reinterpret_cast<const uint2*>(da + row * F);
  int4* outr = reinterpret_cast<int4*>(dh13 + row * 2 * F);
  uint2* ar = a_out ? reinterpret_cast<uint2*>(a_out + row * F) : nullptr;
  float dot = 0.f;
  for (int c = lane; c < (F >> 2); c += 32) {
    Pack8 in, out;
    in.v = ld_nc_v4(hr + c);
    uint2 dv = dr[c];
    __nv_bfloat162 d2[2] = {*reinterpret_cast<__nv_bfloat162*>(&dv.x), *reinterpret_cast<__nv_bfloat162*>(&dv.y)};
    __nv_bfloat162 ao[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float2 d = __bfloat1622float2(d2[j]);
      float2 p0 = __bfloat1622float2(in.h[2 * j]);
      float2 p1 = __bfloat1622float2(in.h[2 * j + 1]);
      const float s0 = 1.f / (1.f + __expf(-p0.x)), s1 = 1.f / (1.f + __expf(-p1.x));
      const float a0 = p0.x * s0 * p0.y, a1 = p1.x * s1 * p1.y;
      dot += a0 * d.x + a1 * d.y;
      const float g0 = d.x * sc, g1 = d.y * sc;
      out.h[2 * j] = __floats2bfloat162_rn(g0 * p0.y * s0 * (1.f + p0.x * (1.f - s0)), g0 * p0.x * s0);
      out.h[2 * j + 1] = __floats2bfloat162_rn(g1 * p1.y * s1 * (1.f + p1.x * (1.f - s1)), g1 * p1.x * s1);
      ao[j] = __floats2bfloat162_rn(a0 * sc, a1 * sc);
    }
    outr[c] = out.v;
    if (ar) ar[c] = *reinterpret_cast<uint2*>(ao);
  }
  if (rowdot) {
    dot = warp_sum(dot);
    if (lane == 0) rowdot[row] = dot;
  }
}

// ------------------------------------------------------------------ embedding
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_embedding_fwd(const int64_t* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                __nv_bfloat16* __restrict__ out, long long T, int H, int V, float scale) {
  const long long row = static_cast<long long>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= T) return;
  const int lane = threadIdx.x & 31;
  long long tok = tokens[row];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  const int4* src = reinterpret_cast<const int4*>(table + tok * H);
  int4* dst = reinterpret_cast<int4*>(out + row * H);
  for (int c = lane; c < (H >> 3); c += 32) {
    Pack8 v;
    v.v = __ldg(src + c);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(v.h[j]);
      v.h[j] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
    }
    dst[c] = v.v;
  }
}

// ------------------------------------------------------------------ flat AdamW
// bf16 params / grads / moments, fp32 math, decoupled decay applied first.
// grad_scale multiplies the gradient (1/world for an averaged reduce, etc.).
__global__ void k_adamw_flat(__nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ g,
                             __nv_bfloat16* __restrict__ m, __nv_bfloat16* __restrict__ v, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, float inv_bc1, float inv_bc2_sqrt,
                             float grad_scale) {
  const long long i8 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i8 >= n) return;
  if (i8 + 8 <= n) {
    Pack8 pv, gv, mv, vv;
    pv.v = *reinterpret_cast<const int4*>(p + i8);
    gv.v = ld_nc_v4(g + i8);
    mv.v = *reinterpret_cast<const int4*>(m + i8);
    vv.v = *reinterpret_cast<const int4*>(v + i8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 pf = __bfloat1622float2(pv.h[j]), gf = __bfloat1622float2(gv.h[j]);
      float2 mf = __bfloat1622float2(mv.h[j]), vf = __bfloat1622float2(vv.h[j]);
      gf.x *= grad_scale; gf.y *= grad_scale;
      pf.x *= (1.f - lr * wd); pf.y *= (1.f - lr * wd);
      mf.x = beta1 * mf.x + (1.f - beta1) * gf.x; mf.y = beta1 * mf.y + (1.f - beta1) * gf.y;
      vf.x = beta2 * vf.x + (1.f - beta2) * gf.x * gf.x; vf.y = beta2 * vf.y + (1.f - beta2) * gf.y * gf.y;
      pf.x -= lr * inv_bc1 * mf.x / (sqrtf(vf.x) * inv_bc2_sqrt + eps);
      pf.y -= lr * inv_bc1 * mf.y / (sqrtf(vf.y) * inv_bc2_sqrt + eps);
      pv.h[j] = __floats2bfloat162_rn(pf.x, pf.y);
      mv.h[j] = __floats2bfloat162_rn(mf.x, mf.y);
      vv.h[j] = __floats2bfloat162_rn(vf.x, vf.y);
    }
    *reinterpret_cast<int4*>(p + i8) = pv.v;
    *reinterpret_cast<int4*>(m + i8) = mv.v;
    *reinterpret_cast<int4*>(v + i8) = vv.v;
  } else {
    for (long long i = i8; i < n; ++i) {
      float pf = __bfloat162float(p[i]), gf = __bfloat162float(g[i]) * grad_scale;
      float mf = __bfloat162float(m[i]), vf = __bfloat162float(v[i]);
      pf *= (1.f - lr * wd);
      mf = beta1 * mf + (1.f - beta1) * gf;
      vf = beta2 * vf + (1.f - beta2) * gf * gf;
      pf -= lr * inv_bc1 * mf / (sqrtf(vf) * inv_bc2_sqrt + eps);
      p[i] = __float2bfloat16(pf); m[i] = __float2bfloat16(mf); v[i] = __float2bfloat16(vf);
    }
  }
}

// sum of squares of a bf16 buffer accumulated into out[0] (fp32), for gradient-norm logging.
__global__ void k_sumsq_bf16(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ out) {
  float s = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    if (i + 8 <= n) {
      Pack8 v;
      v.v = ld_nc_v4(x + i);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(v.h[j]);
        s += f.x * f.x + f.y * f.y;
      }
    } else {
      for (long long k = i; k < n; ++k) {
        float f = __bfloat162float(x[k]);
        s += f * f;
      }
    }
  }
  s = warp_sum(s);
  __shared__ float sh[32];
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) atomicAdd(out, s);
  }
}

}  // namespace nmoe

using namespace nmoe;

#define CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return static_cast<int>(e_); } while (0)

extern "C" {

int nmoe_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int M, int H, float eps, cudaStream_t st) {
  if (M == 0) return 0;
  if (H % 8 != 0 || H > 8192) return -1;
  const int blocks = (M + kWarpsPerBlock - 1) / kWarpsPerBlock;
  auto xx = static_cast<const __nv_bfloat16*>(x);
  auto ww = static_cast<const __nv_bfloat16*>(w);
  auto yy = static_cast<__nv_bfloat16*>(y);
  if (H <= 1024) k_rmsnorm_fwd<4><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xx, ww, yy, rstd, M, H, eps);
  else if (H <= 2048) k_rmsnorm_fwd<8><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xx, ww, yy, rstd, M, H, eps);
  else if (H <= 4096) k_rmsnorm_fwd<16><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xx, ww, yy, rstd, M, H, eps);
  else k_rmsnorm_fwd<32><<<blocks, kWarpsPerBlock * 32, 0, st>>>(xx, ww, yy, rstd, M, H, eps);
  CHECK_LAUNCH();
  return 0;
}

// Number of fp32 partial rows the backward needs: scratch = nblocks * H floats.
int nmoe_rmsnorm_bwd_blocks(int M) {
  int b = (M + 23) / 24;      // ~3 rows per warp: enough blocks (<= 592 = 4 per SM) to cover the machine
  return b < 1 ? 1 : (b > 592 ? 592 : b);
}

int nmoe_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                     float* scratch, int M, int H, int accumulate, cudaStream_t st) {
  if (M == 0) return 0;
  if (H % 8 != 0 || H > 16384) return -1;
  const int nblocks = nmoe_rmsnorm_bwd_blocks(M);
  const int rpb = (M + nblocks - 1) / nblocks;
  const size_t smem = static_cast<size_t>(kWarpsPerBlock) * H * sizeof(float);
  auto a = static_cast<const __nv_bfloat16*>(dy);
  auto b = static_cast<const __nv_bfloat16*>(x);
  auto c = static_cast<const __nv_bfloat16*>(w);
  auto d = static_cast<__nv_bfloat16*>(dx);
  if (H > 4096) {
    // wide rows (DeepSeek-V2/V3 hidden sizes): row dots first, then a column-tiled pass.  The row dots live
    // in the M floats after the nblocks * H partial sums of `scratch`.
    float* rowdot = scratch + static_cast<size_t>(nblocks) * H;
    k_rmsnorm_rowdot<<<(M + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, st>>>(a, b, c, rowdot, M, H);
    CHECK_LAUNCH();
    k_rmsnorm_bwd_wide<<<dim3((H + 255) / 256, nblocks), 256, 0, st>>>(a, b, c, rstd, rowdot, d, scratch, M, H, rpb);
    CHECK_LAUNCH();
    k_colsum_to_bf16<<<(H + 255) / 256, 256, 0, st>>>(scratch, static_cast<__nv_bfloat16*>(dw), nblocks, H, accumulate);
    CHECK_LAUNCH();
    return 0;
  }
#define LAUNCH_BWD(V)                                                                                      \
  do {                                                                                                     \
    cudaFuncSetAttribute(k_rmsnorm_bwd<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    k_rmsnorm_bwd<V><<<nblocks, kWarpsPerBlock * 32, smem, st>>>(a, b, c, rstd, d, scratch, M, H, rpb);    \
  } while (0)
  if (H <= 512) LAUNCH_BWD(2);
  else if (H <= 1024) LAUNCH_BWD(4);
  else if (H <= 2048) LAUNCH_BWD(8);
  else LAUNCH_BWD(16);
#undef LAUNCH_BWD
  CHECK_LAUNCH();
  k_colsum_to_bf16<<<(H + 255) / 256, 256, 0, st>>>(scratch, static_cast<__nv_bfloat16*>(dw), nblocks, H, accumulate);
  CHECK_LAUNCH();
  return 0;
}

// Two-pass form for any H (H % 8 == 0): row dots, then a column-tiled pass with 16-byte accesses and few registers.
// scratch: nmoe_rmsnorm_bwd_blocks(M) * H + M floats.  About twice as fast as the single-pass kernel at H = 2048.
int nmoe_rmsnorm_bwd_twopass(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                             float* scratch, int M, int H, int accumulate, cudaStream_t st) {
  if (M == 0) return 0;
  if (H % 8 != 0 || H > 16384) return -1;
  const int nblocks = nmoe_rmsnorm_bwd_blocks(M);
  const int rpb = (M + nblocks - 1) / nblocks;
  auto a = static_cast<const __nv_bfloat16*>(dy);
  auto b = static_cast<const __nv_bfloat16*>(x);
  auto c = static_cast<const __nv_bfloat16*>(w);
  float* rowdot = scratch + static_cast<size_t>(nblocks) * H;
  k_rmsnorm_rowdot<<<(M + kWarpsPerBlock - 1) / kWarpsPerBlock, kWarpsPerBlock * 32, 0, st>>>(a, b, c, rowdot, M, H);
  CHECK_LAUNCH();
  const int nvec = H / 8;
  k_rmsnorm_bwd_cols<<<dim3((nvec + 255) / 256, nblocks), 256, 0, st>>>(a, b, c, rstd, rowdot, static_cast<__nv_bfloat16*>(dx),
                                                                       scratch, M, H, rpb);
  CHECK_LAUNCH();
  k_colsum32_to_bf16<<<(H + 31) / 32, 256, 0, st>>>(scratch, static_cast<__nv_bfloat16*>(dw), nblocks, H, accumulate);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_rope_inplace(void* x, const float* cos_t, const float* sin_t, long long rows, int h, int S,
                      long long row_stride, int offset, int D, int backward, cudaStream_t st) {
  const long long total = rows * (D / 2);
  if (total == 0) return 0;
  k_rope_inplace<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(
      static_cast<__nv_bfloat16*>(x), cos_t, sin_t, rows, h, S, row_stride, offset, D, backward ? -1.f : 1.f);
  CHECK_LAUNCH();
  return 0;
}

// n_tiles_dev (optional, device): only the first *n_tiles_dev * 128 rows are processed.
int nmoe_swiglu_fwd(const void* h13, void* a, long long M, int F, const int* n_tiles_dev, cudaStream_t st) {
  if (M == 0) return 0;
  if (F % 4 != 0) return -1;
  const long long nvec = M * (F / 4);
  long long blocks = (nvec + 511) / 512;
  if (blocks > 148 * 16) blocks = 148 * 16;
  k_swiglu_fwd<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(h13), static_cast<__nv_bfloat16*>(a), M, F, n_tiles_dev);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_swiglu_bwd(const void* h13, const void* da, void* dh13, const float* row_scale, float* rowdot, void* a_out,
                    long long M, int F, const int* n_tiles_dev, cudaStream_t st) {
  if (M == 0) return 0;
  if (F % 4 != 0) return -1;
  k_swiglu_bwd<<<static_cast<unsigned>((M + kWarpsPerBlock - 1) / kWarpsPerBlock), kWarpsPerBlock * 32, 0, st>>>(
      static_cast<const __nv_bfloat16*>(h13), static_cast<const __nv_bfloat16*>(da),
      static_cast<__nv_bfloat16*>(dh13), row_scale, rowdot, static_cast<__nv_bfloat16*>(a_out), M, F, n_tiles_dev);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_embedding_fwd(const int64_t* tokens, const void* table, void* out, long long T, int H, int V, float scale,
                       cudaStream_t st) {
  if (T == 0) return 0;
  if (H % 8 != 0) return -1;
  k_embedding_fwd<<<static_cast<unsigned>((T + kWarpsPerBlock - 1) / kWarpsPerBlock), kWarpsPerBlock * 32, 0, st>>>(
      tokens, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), T, H, V, scale);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_adamw_flat(void* p, const void* g, void* m, void* v, long long n, float lr, float beta1, float beta2,
                    float eps, float wd, int step, float grad_scale, cudaStream_t st) {
  if (n == 0) return 0;
  const float inv_bc1 = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  const float inv_bc2_sqrt = 1.f / sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  const long long nthreads = (n + 7) / 8;
  k_adamw_flat<<<static_cast<unsigned>((nthreads + 255) / 256), 256, 0, st>>>(
      static_cast<__nv_bfloat16*>(p), static_cast<const __nv_bfloat16*>(g), static_cast<__nv_bfloat16*>(m),
      static_cast<__nv_bfloat16*>(v), n, lr, beta1, beta2, eps, wd, inv_bc1, inv_bc2_sqrt, grad_scale);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_sumsq_bf16(const void* x, long long n, float* out, cudaStream_t st) {
  if (n == 0) return 0;
  k_sumsq_bf16<<<592, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), n, out);
  CHECK_LAUNCH();
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------ allocation-free variant
#include <atomic>

#include "noalloc.h"

namespace nmoe {
// Scratch for nmoe_rmsnorm_bwd_noalloc.  In host code this name is only a handle for
// cudaGetSymbolAddress; the kernels receive the resolved device pointer.
static __device__ __align__(256) float g_rmsnorm_bwd_scratch[NMOE_NOALLOC_RMSNORM_MAX_BLOCKS * NMOE_NOALLOC_RMSNORM_MAX_H];
constexpr int kNoallocMaxDevices = 64;
// Per-device cache of the resolved address.  Atomic: two host threads may make the first call on a device at the
// same time; both resolve the same address and both store it, which is harmless, but the accesses must not race.
static std::atomic<float*> g_rmsnorm_bwd_scratch_ptr[kNoallocMaxDevices];
}  // namespace nmoe

extern "C" int nmoe_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                        void* dw, int M, int H, int accumulate, cudaStream_t st) {
  if (M == 0) return 0;
  if (H % 8 != 0 || H > NMOE_NOALLOC_RMSNORM_MAX_H) return -1;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= nmoe::kNoallocMaxDevices) return -3;
  float* scratch = nmoe::g_rmsnorm_bwd_scratch_ptr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // once per device, with that device current
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), nmoe::g_rmsnorm_bwd_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    nmoe::g_rmsnorm_bwd_scratch_ptr[dev].store(scratch, std::memory_order_release);
  }
  // nmoe_rmsnorm_bwd_blocks(M) never exceeds NMOE_NOALLOC_RMSNORM_MAX_BLOCKS, and every partial
  // row read by the column sum is written by the backward kernel of the same call.
  return nmoe_rmsnorm_bwd(dy, x, w, rstd, dx, dw, scratch, M, H, accumulate, st);
}
