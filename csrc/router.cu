// Router: scores -> (optional device-limited group mask) -> bias-adjusted top-k -> renormalised
// weights of the unbiased scores, plus per-expert load counts.  One warp per token, the E scores
// of a token live in registers (E <= 512, E % 32 == 0), top-k by k rounds of warp arg-max.
//
// kind 0: score = sigmoid(scale * logit)  (aux-loss-free bias routing, nmoe/model.py:61-70)
// kind 1: score = softmax(scale * logit)
// Selection uses score + bias; ties go to the lower expert id.  With max_groups > 0 only the
// max_groups expert groups (of n_groups contiguous groups) with the largest group maximum
// of (score + bias) are eligible.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/ptx.cuh"

namespace nmoe {

constexpr int kMaxPerLane = 16;   // E <= 512

template <typename T> NMOE_DEVICE float to_f(T v);
template <> NMOE_DEVICE float to_f<float>(float v) { return v; }
template <> NMOE_DEVICE float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

NMOE_DEVICE void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// Computes scores for one token into sc[] (lane holds experts lane, lane+32, ...).  Returns softmax
// normaliser pieces through mx / denom for kind 1.
template <typename T>
NMOE_DEVICE void load_scores(const T* __restrict__ row, int E, int lane, float scale, int kind, float* sc) {
  const int per = (E + 31) >> 5;
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    if (j < per && (lane + 32 * j) < E) {
      sc[j] = to_f(row[lane + 32 * j]) * scale;
      mx = fmaxf(mx, sc[j]);
    }
  }
  if (kind == 0) {
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E) sc[j] = 1.f / (1.f + __expf(-sc[j]));
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E) { sc[j] = __expf(sc[j] - mx); sum += sc[j]; }
    sum = warp_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E) sc[j] *= inv;
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
k_router_fwd(const T* __restrict__ logits, const float* __restrict__ bias, int Tn, int E, int K, float scale,
             int kind, int n_groups, int max_groups, float* __restrict__ weights, int* __restrict__ idx,
             int* __restrict__ loads) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const int lane = threadIdx.x & 31;
  const int per = (E + 31) >> 5;
  float sc[kMaxPerLane], sel[kMaxPerLane];
  load_scores(logits + static_cast<size_t>(t) * E, E, lane, scale, kind, sc);
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j)
    if (j < per && (lane + 32 * j) < E) sel[j] = sc[j] + (bias ? bias[lane + 32 * j] : 0.f);
  if (max_groups > 0 && n_groups > 1 && max_groups < n_groups) {
    // group g owns experts [g*gs, (g+1)*gs); group maxima -> keep the top max_groups groups
    const int gs = E / n_groups;
    float gmax = -INFINITY;   // lane g (< n_groups <= 32) ends up with the maximum of group g
    for (int g = 0; g < n_groups; ++g) {
      float m = -INFINITY;
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (j < per && (lane + 32 * j) < E && (lane + 32 * j) / gs == g) m = fmaxf(m, sel[j]);
      m = warp_max(m);
      if (lane == g) gmax = m;
    }
    unsigned keep = 0;
    for (int r = 0; r < max_groups; ++r) {
      float v = (lane < n_groups && !((keep >> lane) & 1u)) ? gmax : -INFINITY;
      int i = lane;
      warp_argmax(v, i);
      keep |= 1u << i;
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E && !((keep >> ((lane + 32 * j) / gs)) & 1u)) sel[j] = -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;     // lane k keeps the k-th selected weight
  int my_i = 0;
  for (int k = 0; k < K; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E && (sel[j] > bv)) { bv = sel[j]; bi = lane + 32 * j; }
    warp_argmax(bv, bi);
    // owner lane of the winner contributes its unbiased score and retires the entry
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E && (lane + 32 * j) == bi) { s = sc[j]; sel[j] = -INFINITY; }
    s = warp_sum(s);
    wsum += s;
    if (lane == (k & 31)) { my_w = s; my_i = bi; }
    if (k >= 32 && lane == (k & 31)) { /* K <= 32 enforced on the host */ }
  }
  const float inv = 1.f / fmaxf(wsum, 1e-12f);
  if (lane < K) {
    weights[static_cast<size_t>(t) * K + lane] = my_w * inv;
    idx[static_cast<size_t>(t) * K + lane] = my_i;
    if (loads) atomicAdd(loads + my_i, 1);
  }
}

// dlogits from dweights.  Selected set and scores are recomputed from the logits.
template <typename T>
__global__ void __launch_bounds__(256)
k_router_bwd(const T* __restrict__ logits, const int* __restrict__ idx, const float* __restrict__ dweights, int Tn,
             int E, int K, float scale, int kind, T* __restrict__ dlogits) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const int lane = threadIdx.x & 31;
  const int per = (E + 31) >> 5;
  float sc[kMaxPerLane], dsc[kMaxPerLane];
  load_scores(logits + static_cast<size_t>(t) * E, E, lane, scale, kind, sc);
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) dsc[j] = 0.f;
  // lane k holds (idx_k, dw_k); S = sum of selected scores; dot = sum dw_k w_k
  const int my_i = lane < K ? idx[static_cast<size_t>(t) * K + lane] : -1;
  const float my_dw = lane < K ? dweights[static_cast<size_t>(t) * K + lane] : 0.f;
  float S = 0.f;
  for (int k = 0; k < K; ++k) {
    const int e = __shfl_sync(0xffffffffu, my_i, k);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E && (lane + 32 * j) == e) s = sc[j];
    S += warp_sum(s);
  }
  const float Sc = fmaxf(S, 1e-12f);
  float dot = 0.f;
  for (int k = 0; k < K; ++k) {
    const int e = __shfl_sync(0xffffffffu, my_i, k);
    const float dw = __shfl_sync(0xffffffffu, my_dw, k);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E && (lane + 32 * j) == e) s = sc[j];
    s = warp_sum(s);
    dot += dw * s / Sc;
  }
  for (int k = 0; k < K; ++k) {
    const int e = __shfl_sync(0xffffffffu, my_i, k);
    const float dw = __shfl_sync(0xffffffffu, my_dw, k);
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E && (lane + 32 * j) == e) dsc[j] = (S > 1e-12f) ? (dw - dot) / Sc : 0.f;
  }
  T* out = dlogits + static_cast<size_t>(t) * E;
  if (kind == 0) {
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E) {
        const float g = dsc[j] * sc[j] * (1.f - sc[j]) * scale;
        if constexpr (sizeof(T) == 2) out[lane + 32 * j] = __float2bfloat16(g);
        else out[lane + 32 * j] = g;
      }
  } else {
    float pd = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E) pd += dsc[j] * sc[j];
    pd = warp_sum(pd);
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j)
      if (j < per && (lane + 32 * j) < E) {
        const float g = scale * sc[j] * (dsc[j] - pd);
        if constexpr (sizeof(T) == 2) out[lane + 32 * j] = __float2bfloat16(g);
        else out[lane + 32 * j] = g;
      }
  }
}

// bias -= gamma * (s - mean(s)), s = sign(load_fraction - 1/E), clamp to [-16, 16]
// (nmoe/model.py:72-77).  counts are integer loads; their sum is the normaliser.
__global__ void k_router_bias_update(float* __restrict__ bias, const float* __restrict__ loads, int E, float gamma) {
  __shared__ float s_tot, s_mean;
  __shared__ float s_sign[512];
  float part = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) part += loads[e];
  part = warp_sum(part);
  if (threadIdx.x == 0) s_tot = 0.f;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) atomicAdd(&s_tot, part);
  __syncthreads();
  const float tot = fmaxf(s_tot, 1.f);
  float sp = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const float d = loads[e] / tot - 1.f / static_cast<float>(E);
    const float s = d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
    s_sign[e] = s;
    sp += s;
  }
  sp = warp_sum(sp);
  if (threadIdx.x == 0) s_mean = 0.f;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) atomicAdd(&s_mean, sp);
  __syncthreads();
  const float mean = s_mean / static_cast<float>(E);
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    bias[e] = fminf(16.f, fmaxf(-16.f, bias[e] - gamma * (s_sign[e] - mean)));
}

}  // namespace nmoe

using namespace nmoe;

extern "C" {

int nmoe_router_fwd(const void* logits, int logits_fp32, const float* bias, int T, int E, int K, float scale,
                    int kind, int n_groups, int max_groups, float* weights, int* idx, int* loads, cudaStream_t st) {
  if (T == 0) return 0;
  if (E < 1 || E > 32 * kMaxPerLane || K > 32 || K > E) return -1;
  if (max_groups > 0 && (n_groups > 32 || n_groups < 1 || E % n_groups != 0)) return -2;
  const int blocks = (T + 7) / 8;
  if (logits_fp32)
    k_router_fwd<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(logits), bias, T, E, K, scale, kind,
                                                n_groups, max_groups, weights, idx, loads);
  else
    k_router_fwd<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), bias, T, E, K,
                                                        scale, kind, n_groups, max_groups, weights, idx, loads);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

int nmoe_router_bwd(const void* logits, int logits_fp32, const int* idx, const float* dweights, int T, int E, int K,
                    float scale, int kind, void* dlogits, cudaStream_t st) {
  if (T == 0) return 0;
  if (E < 1 || E > 32 * kMaxPerLane || K > 32) return -1;
  const int blocks = (T + 7) / 8;
  if (logits_fp32)
    k_router_bwd<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(logits), idx, dweights, T, E, K, scale,
                                                kind, static_cast<float*>(dlogits));
  else
    k_router_bwd<__nv_bfloat16><<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), idx, dweights, T,
                                                        E, K, scale, kind, static_cast<__nv_bfloat16*>(dlogits));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

int nmoe_router_bias_update(float* bias, const float* loads, int E, float gamma, cudaStream_t st) {
  if (E > 512) return -1;
  k_router_bias_update<<<1, 256, 0, st>>>(bias, loads, E, gamma);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // extern "C"
