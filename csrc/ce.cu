// Fused masked cross-entropy over a chunk of logits: one block per row computes the
// log-sum-exp of (logit * scale) in a streaming pass, adds the row's loss to a global
// accumulator, and overwrites the logits in place with d(loss)/d(logit) (already divided by the
// number of unmasked targets), so the [rows, V] fp32 softmax of the eager path
// (nmoe/train.py:103-105) never exists.  Rows whose target equals ignore_id get zero gradient.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/ptx.cuh"

namespace nmoe {

constexpr int kCeThreads = 512;

union Pack8c {
  int4 v;
  __nv_bfloat162 h[4];
};

__global__ void __launch_bounds__(kCeThreads)
k_ce_fwd_bwd(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets, int V, long long ld,
             int ignore_id, float scale, const float* __restrict__ inv_count, float* __restrict__ loss_sum,
             float* __restrict__ lse_out, int write_grad) {
  __shared__ float s_m[kCeThreads / 32], s_s[kCeThreads / 32];
  __shared__ float s_lse;
  const long long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int64_t tgt = targets[row];
  const bool ignored = (tgt == ignore_id) || tgt < 0 || tgt >= V;
  const int nvec = V >> 3;
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < nvec; c += kCeThreads) {
    Pack8c p;
    p.v = *reinterpret_cast<const int4*>(lr + c * 8);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(p.h[j]);
      f[2 * j] = t.x * scale;
      f[2 * j + 1] = t.y * scale;
    }
    float cm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) cm = fmaxf(cm, f[j]);
    const float nm = fmaxf(m, cm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += kCeThreads) {
    const float f = __bfloat162float(lr[i]) * scale;
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  // block combine of (m, s)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) { s_m[threadIdx.x >> 5] = m; s_s[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x < 32) {
    m = threadIdx.x < kCeThreads / 32 ? s_m[threadIdx.x] : -INFINITY;
    s = threadIdx.x < kCeThreads / 32 ? s_s[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
      m = nm;
    }
    if (threadIdx.x == 0) {
      const float lse = m + __logf(s);
      s_lse = lse;
      if (lse_out) lse_out[row] = lse;
      if (!ignored) {
        const float zt = __bfloat162float(lr[tgt]) * scale;
        atomicAdd(loss_sum, (lse - zt) * (*inv_count));
      }
    }
  }
  __syncthreads();
  if (!write_grad) return;
  const float lse = s_lse;
  const float g = ignored ? 0.f : scale * (*inv_count);
  for (int c = threadIdx.x; c < nvec; c += kCeThreads) {
    Pack8c p;
    p.v = *reinterpret_cast<const int4*>(lr + c * 8);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = __bfloat1622float2(p.h[j]);
      float a = __expf(t.x * scale - lse), b = __expf(t.y * scale - lse);
      const int i0 = c * 8 + 2 * j;
      if (i0 == tgt) a -= 1.f;
      if (i0 + 1 == tgt) b -= 1.f;
      p.h[j] = __floats2bfloat162_rn(a * g, b * g);
    }
    *reinterpret_cast<int4*>(lr + c * 8) = p.v;
  }
  for (int i = (nvec << 3) + threadIdx.x; i < V; i += kCeThreads) {
    float a = __expf(__bfloat162float(lr[i]) * scale - lse);
    if (i == tgt) a -= 1.f;
    lr[i] = __float2bfloat16(a * g);
  }
}

}  // namespace nmoe

extern "C" int nmoe_ce_fwd_bwd(void* logits, const int64_t* targets, int rows, int V, long long ld, int ignore_id,
                               float scale, const float* inv_count, float* loss_sum, float* lse_out, int write_grad,
                               cudaStream_t st) {
  if (rows == 0) return 0;
  if ((ld % 8) != 0) return -1;
  nmoe::k_ce_fwd_bwd<<<rows, nmoe::kCeThreads, 0, st>>>(static_cast<__nv_bfloat16*>(logits), targets, V, ld, ignore_id,
                                                        scale, inv_count, loss_sum, lse_out, write_grad);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
