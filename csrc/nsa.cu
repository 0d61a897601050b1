// Compressed branch of Native Sparse Attention: group-mean queries attend over keys / values that a small MLP has
// compressed from overlapping blocks of cmp_len tokens with stride cmp_stride, and the attention probabilities are
// summed into scores of the selection blocks (slc_block tokens) that the selection branch ranks.
//
//   s[t, c] = scale <q_t, kc_c>            visible when the block of c has ended:  c * stride + len - 1 <= t
//   m_t     = max(0, max_c s[t, c]),  e = exp(s - m_t),  den_t = max(sum_c e, 1e-6),  p = e / den_t
//   out_t   = sum_c p[t, c] vc_c
//   score[t, n] = sum_{c : bin(c) == n} p[t, c],   bin(c) = min((c * stride + len / 2) / slc_block, Ns - 1)
//
// (the floor of the maximum at 0 and of the denominator at 1e-6 make a query with nothing visible produce zeros and
// are part of the layer's definition, models/attention/nsa.py).  Scores go to a top-k and carry no gradient; the
// backward of `out` is two kernels without atomics: dQ per query block, dKc / dVc per compressed-key block.
// Everything is fp32 arithmetic on CUDA cores: with Tc = T / stride keys the whole branch is ~1 GFLOP per head group at
// T = 4096, and what matters is that no [T, Tc] tensor makes round trips through HBM between five eager kernels.
// Replaces the Triton kernels of the reference (nmoe/triton/nsa.py:27-317: compressed attention forward / backward with
// fused block-score aggregation).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/ptx.cuh"

namespace nmoe {

constexpr int NSA_WARPS = 8;
constexpr int NSA_QB = 32;        // queries per CTA (forward, dQ): 4 per warp
constexpr int NSA_CK = 128;       // compressed keys per shared-memory chunk
constexpr int NSA_KPW = 1;       // compressed keys per warp in the dKc / dVc kernel
constexpr int NSA_KB = NSA_WARPS * NSA_KPW;
constexpr int NSA_MAX_NS = 256;   // selection blocks per sequence (T <= 16384 at 64-token blocks)

struct NsaCmpArgs {
  int B, T, KV, Tc, Ns;
  int cmp_len, cmp_stride, slc_block;
  float scale;
  const __nv_bfloat16* q;     // [B, T, KV, D]
  const __nv_bfloat16* kc;    // [B, Tc, KV, D]
  const __nv_bfloat16* vc;    // [B, Tc, KV, D]
  __nv_bfloat16* out;         // [B, T, KV, D]
  float* scores;              // [B, T, KV, Ns] or null
  float* stats;               // [B, KV, T, 2] = (m_t, den_t)
  // backward
  const __nv_bfloat16* dout;  // [B, T, KV, D]
  __nv_bfloat16* dq;          // [B, T, KV, D]
  float* dkc;                 // [B, Tc, KV, D] fp32
  float* dvc;                 // [B, Tc, KV, D] fp32
};

// number of compressed keys visible to query t
NMOE_DEVICE int nsa_visible(int t, int len, int stride, int Tc) {
  const int v = t - len + 1;
  if (v < 0) return 0;
  const int n = v / stride + 1;
  return n < Tc ? n : Tc;
}

// rows of `rows` x D bf16 -> shared memory with a row pitch of D + 2 (odd word pitch: a warp reading one column of
// 32 different rows touches 32 banks)
template <int D>
NMOE_DEVICE void nsa_stage_rows(__nv_bfloat16* dst, const __nv_bfloat16* src, long long src_pitch, int rows, int valid) {
  constexpr int P = D + 2;
  for (int i = threadIdx.x; i < rows * (D / 2); i += blockDim.x) {
    const int r = i / (D / 2), c2 = i % (D / 2);
    uint32_t v = 0u;
    if (r < valid) v = *reinterpret_cast<const uint32_t*>(src + static_cast<long long>(r) * src_pitch + 2 * c2);
    *reinterpret_cast<uint32_t*>(dst + r * P + 2 * c2) = v;
  }
}

NMOE_DEVICE float nsa_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
NMOE_DEVICE float nsa_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
NMOE_DEVICE float2 nsa_bf2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// Shared memory (forward, dQ):  Ks [CK][D+2] bf16 | Vs [CK][D+2] bf16 | qs [QB][D] f32 | ps [WARPS][CK] f32 |
//                               bins [QB][Ns] f32 (forward) or dos [QB][D] f32 (dQ)
template <int D>
__global__ void __launch_bounds__(NSA_WARPS * 32) k_nsa_cmp_fwd(const NsaCmpArgs a) {
  constexpr int P = D + 2;
  constexpr int NP = D / 64;                 // column pairs per lane: {2 lane, 2 lane + 1} (+ 64)
  extern __shared__ __align__(16) uint8_t nsa_smem[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(nsa_smem);
  __nv_bfloat16* Vs = Ks + NSA_CK * P;
  float* qs = reinterpret_cast<float*>(Vs + NSA_CK * P);
  float* ps = qs + NSA_QB * D;
  float* bins = ps + NSA_WARPS * NSA_CK;
  const int b = blockIdx.z, kv = blockIdx.y, t0 = blockIdx.x * NSA_QB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long pitch = static_cast<long long>(a.KV) * D;
  const __nv_bfloat16* qbase = a.q + (static_cast<long long>(b) * a.T * a.KV + kv) * D;
  const __nv_bfloat16* kbase = a.kc + (static_cast<long long>(b) * a.Tc * a.KV + kv) * D;
  const __nv_bfloat16* vbase = a.vc + (static_cast<long long>(b) * a.Tc * a.KV + kv) * D;
  for (int i = threadIdx.x; i < NSA_QB * D; i += blockDim.x) {
    const int r = i / D, d = i % D, t = t0 + r;
    qs[i] = t < a.T ? __bfloat162float(qbase[t * pitch + d]) * a.scale : 0.f;
  }
  for (int i = threadIdx.x; i < NSA_QB * a.Ns; i += blockDim.x) bins[i] = 0.f;
  const int t_last = min(t0 + NSA_QB, a.T) - 1;
  const int n_blk = nsa_visible(t_last, a.cmp_len, a.cmp_stride, a.Tc);
  float m[4], l[4], o[4][2 * NP];
#pragma unroll
  for (int qi = 0; qi < 4; ++qi) {
    m[qi] = 0.f; l[qi] = 0.f;
#pragma unroll
    for (int x = 0; x < 2 * NP; ++x) o[qi][x] = 0.f;
  }
  for (int c0 = 0; c0 < n_blk; c0 += NSA_CK) {
    __syncthreads();
    nsa_stage_rows<D>(Ks, kbase + c0 * pitch, pitch, NSA_CK, min(NSA_CK, a.Tc - c0));
    nsa_stage_rows<D>(Vs, vbase + c0 * pitch, pitch, NSA_CK, min(NSA_CK, a.Tc - c0));
    __syncthreads();
#pragma unroll
    for (int qi = 0; qi < 4; ++qi) {
      const int r = warp * 4 + qi, t = t0 + r;
      if (t >= a.T) continue;
      const int nvis = nsa_visible(t, a.cmp_len, a.cmp_stride, a.Tc);
      if (nvis <= c0) continue;
      float s[4] = {0.f, 0.f, 0.f, 0.f};
      const float* qv = qs + r * D;
      for (int d2 = 0; d2 < D / 2; ++d2) {
        const float q0 = qv[2 * d2], q1 = qv[2 * d2 + 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 kk = nsa_bf2(Ks + (lane + 32 * j) * P + 2 * d2);
          s[j] = fmaf(q0, kk.x, fmaf(q1, kk.y, s[j]));
        }
      }
      float cmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (c0 + lane + 32 * j >= nvis) s[j] = -INFINITY;
        cmax = fmaxf(cmax, s[j]);
      }
      cmax = nsa_warp_max(cmax);
      const float m_new = fmaxf(m[qi], cmax);
      const float corr = __expf(m[qi] - m_new);
      float psum = 0.f;
      float* bq = bins + r * a.Ns;
      if (corr != 1.f) {
        for (int n = lane; n < a.Ns; n += 32) bq[n] *= corr;
        __syncwarp();
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + lane + 32 * j;
        const float p = c < nvis ? __expf(s[j] - m_new) : 0.f;
        psum += p;
        ps[warp * NSA_CK + lane + 32 * j] = p;
        if (c < nvis) atomicAdd(bq + min((c * a.cmp_stride + a.cmp_len / 2) / a.slc_block, a.Ns - 1), p);
      }
      psum = nsa_warp_sum(psum);
      l[qi] = l[qi] * corr + psum;
#pragma unroll
      for (int x = 0; x < 2 * NP; ++x) o[qi][x] *= corr;
      m[qi] = m_new;
      __syncwarp();
      const int kmax = min(NSA_CK, nvis - c0);
      const float* pw = ps + warp * NSA_CK;
      for (int c = 0; c < kmax; ++c) {
        const float pc = pw[c];
#pragma unroll
        for (int h = 0; h < NP; ++h) {
          const float2 vv = nsa_bf2(Vs + c * P + 64 * h + 2 * lane);
          o[qi][2 * h] = fmaf(pc, vv.x, o[qi][2 * h]);
          o[qi][2 * h + 1] = fmaf(pc, vv.y, o[qi][2 * h + 1]);
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int qi = 0; qi < 4; ++qi) {
    const int r = warp * 4 + qi, t = t0 + r;
    if (t >= a.T) continue;
    const float den = fmaxf(l[qi], 1e-6f), inv = 1.f / den;
    __nv_bfloat16* orow = a.out + (static_cast<long long>(b) * a.T * a.KV + kv) * D + t * pitch;
#pragma unroll
    for (int h = 0; h < NP; ++h)
      *reinterpret_cast<__nv_bfloat162*>(orow + 64 * h + 2 * lane) = __floats2bfloat162_rn(o[qi][2 * h] * inv, o[qi][2 * h + 1] * inv);
    if (lane == 0) {
      float* st = a.stats + ((static_cast<long long>(b) * a.KV + kv) * a.T + t) * 2;
      st[0] = m[qi]; st[1] = den;
    }
    if (a.scores != nullptr) {
      __syncwarp();
      float* srow = a.scores + ((static_cast<long long>(b) * a.T + t) * a.KV + kv) * a.Ns;
      for (int n = lane; n < a.Ns; n += 32) srow[n] = bins[r * a.Ns + n] * inv;
    }
  }
}

// dQ: one CTA per 32 queries, streaming the visible compressed keys; also writes delta_t = <dO_t, out_t> (0 for a query
// whose denominator sat on its floor: there the output is not normalised and the softmax has no coupling term).
template <int D>
__global__ void __launch_bounds__(NSA_WARPS * 32) k_nsa_cmp_dq(const NsaCmpArgs a, float* __restrict__ delta) {
  constexpr int P = D + 2;
  constexpr int NP = D / 64;
  extern __shared__ __align__(16) uint8_t nsa_smem[];
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(nsa_smem);
  __nv_bfloat16* Vs = Ks + NSA_CK * P;
  float* qs = reinterpret_cast<float*>(Vs + NSA_CK * P);
  float* ps = qs + NSA_QB * D;
  float* dos = ps + NSA_WARPS * NSA_CK;
  const int b = blockIdx.z, kv = blockIdx.y, t0 = blockIdx.x * NSA_QB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long pitch = static_cast<long long>(a.KV) * D;
  const long long tok0 = (static_cast<long long>(b) * a.T * a.KV + kv) * D;
  const __nv_bfloat16* kbase = a.kc + (static_cast<long long>(b) * a.Tc * a.KV + kv) * D;
  const __nv_bfloat16* vbase = a.vc + (static_cast<long long>(b) * a.Tc * a.KV + kv) * D;
  for (int i = threadIdx.x; i < NSA_QB * D; i += blockDim.x) {
    const int r = i / D, d = i % D, t = t0 + r;
    qs[i] = t < a.T ? __bfloat162float(a.q[tok0 + t * pitch + d]) * a.scale : 0.f;
    dos[i] = t < a.T ? __bfloat162float(a.dout[tok0 + t * pitch + d]) : 0.f;
  }
  __syncthreads();
  float m[4], inv[4], dl[4], g[4][2 * NP];
#pragma unroll
  for (int qi = 0; qi < 4; ++qi) {
    const int r = warp * 4 + qi, t = t0 + r;
    m[qi] = 0.f; inv[qi] = 0.f; dl[qi] = 0.f;
#pragma unroll
    for (int x = 0; x < 2 * NP; ++x) g[qi][x] = 0.f;
    if (t >= a.T) continue;
    const float* st = a.stats + ((static_cast<long long>(b) * a.KV + kv) * a.T + t) * 2;
    m[qi] = st[0];
    const float den = st[1];
    inv[qi] = 1.f / den;
    float d = 0.f;
    if (den > 1e-6f) {
      for (int x = lane; x < D; x += 32) d += dos[r * D + x] * __bfloat162float(a.out[tok0 + t * pitch + x]);
      d = nsa_warp_sum(d);
    }
    dl[qi] = d;
    if (lane == 0) delta[(static_cast<long long>(b) * a.KV + kv) * a.T + t] = d;
  }
  const int t_last = min(t0 + NSA_QB, a.T) - 1;
  const int n_blk = nsa_visible(t_last, a.cmp_len, a.cmp_stride, a.Tc);
  for (int c0 = 0; c0 < n_blk; c0 += NSA_CK) {
    __syncthreads();
    nsa_stage_rows<D>(Ks, kbase + c0 * pitch, pitch, NSA_CK, min(NSA_CK, a.Tc - c0));
    nsa_stage_rows<D>(Vs, vbase + c0 * pitch, pitch, NSA_CK, min(NSA_CK, a.Tc - c0));
    __syncthreads();
#pragma unroll
    for (int qi = 0; qi < 4; ++qi) {
      const int r = warp * 4 + qi, t = t0 + r;
      if (t >= a.T) continue;
      const int nvis = nsa_visible(t, a.cmp_len, a.cmp_stride, a.Tc);
      if (nvis <= c0) continue;
      float s[4] = {0.f, 0.f, 0.f, 0.f}, dp[4] = {0.f, 0.f, 0.f, 0.f};
      const float* qv = qs + r * D;
      const float* dv = dos + r * D;
      for (int d2 = 0; d2 < D / 2; ++d2) {
        const float q0 = qv[2 * d2], q1 = qv[2 * d2 + 1], e0 = dv[2 * d2], e1 = dv[2 * d2 + 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 kk = nsa_bf2(Ks + (lane + 32 * j) * P + 2 * d2);
          const float2 vv = nsa_bf2(Vs + (lane + 32 * j) * P + 2 * d2);
          s[j] = fmaf(q0, kk.x, fmaf(q1, kk.y, s[j]));
          dp[j] = fmaf(e0, vv.x, fmaf(e1, vv.y, dp[j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + lane + 32 * j;
        const float p = c < nvis ? __expf(s[j] - m[qi]) * inv[qi] : 0.f;
        ps[warp * NSA_CK + lane + 32 * j] = p * (dp[j] - dl[qi]);
      }
      __syncwarp();
      const int kmax = min(NSA_CK, nvis - c0);
      const float* pw = ps + warp * NSA_CK;
      for (int c = 0; c < kmax; ++c) {
        const float ds = pw[c];
#pragma unroll
        for (int h = 0; h < NP; ++h) {
          const float2 kk = nsa_bf2(Ks + c * P + 64 * h + 2 * lane);
          g[qi][2 * h] = fmaf(ds, kk.x, g[qi][2 * h]);
          g[qi][2 * h + 1] = fmaf(ds, kk.y, g[qi][2 * h + 1]);
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int qi = 0; qi < 4; ++qi) {
    const int t = t0 + warp * 4 + qi;
    if (t >= a.T) continue;
    __nv_bfloat16* row = a.dq + tok0 + t * pitch;
#pragma unroll
    for (int h = 0; h < NP; ++h)
      *reinterpret_cast<__nv_bfloat162*>(row + 64 * h + 2 * lane) =
          __floats2bfloat162_rn(g[qi][2 * h] * a.scale, g[qi][2 * h + 1] * a.scale);
  }
}

// dKc / dVc: one CTA per NSA_KB compressed keys (one per warp: Tc is small, so few keys per CTA is what fills the
// machine), streaming the queries that can see them in chunks of CK.
// Shared memory: Qs [CK][D+2] bf16 | dOs [CK][D+2] bf16 | ks [KB][D] f32 (scaled) | vs [KB][D] f32 |
//                pw [WARPS][CK] f32 | dw [WARPS][CK] f32 | qstat [CK][3] f32 (m, 1/den, delta)
template <int D>
__global__ void __launch_bounds__(NSA_WARPS * 32) k_nsa_cmp_dkv(const NsaCmpArgs a, const float* __restrict__ delta) {
  constexpr int P = D + 2;
  constexpr int NP = D / 64;
  extern __shared__ __align__(16) uint8_t nsa_smem[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(nsa_smem);
  __nv_bfloat16* dOs = Qs + NSA_CK * P;
  float* ks = reinterpret_cast<float*>(dOs + NSA_CK * P);
  float* vs = ks + NSA_KB * D;
  float* pw = vs + NSA_KB * D;
  float* dw = pw + NSA_WARPS * NSA_CK;
  float* qstat = dw + NSA_WARPS * NSA_CK;
  const int b = blockIdx.z, kv = blockIdx.y, cb = blockIdx.x * NSA_KB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long pitch = static_cast<long long>(a.KV) * D;
  const long long tok0 = (static_cast<long long>(b) * a.T * a.KV + kv) * D;
  const long long key0 = (static_cast<long long>(b) * a.Tc * a.KV + kv) * D;
  for (int i = threadIdx.x; i < NSA_KB * D; i += blockDim.x) {
    const int r = i / D, d = i % D, c = cb + r;
    ks[i] = c < a.Tc ? __bfloat162float(a.kc[key0 + c * pitch + d]) * a.scale : 0.f;
    vs[i] = c < a.Tc ? __bfloat162float(a.vc[key0 + c * pitch + d]) : 0.f;
  }
  float gk[NSA_KPW][2 * NP], gv[NSA_KPW][2 * NP];
#pragma unroll
  for (int ki = 0; ki < NSA_KPW; ++ki)
#pragma unroll
    for (int x = 0; x < 2 * NP; ++x) { gk[ki][x] = 0.f; gv[ki][x] = 0.f; }
  const int t_first = cb * a.cmp_stride + a.cmp_len - 1;          // first query that sees the CTA's first key
  for (int q0 = (t_first / NSA_CK) * NSA_CK; q0 < a.T; q0 += NSA_CK) {
    __syncthreads();
    const int valid = min(NSA_CK, a.T - q0);
    nsa_stage_rows<D>(Qs, a.q + tok0 + q0 * pitch, pitch, NSA_CK, valid);
    nsa_stage_rows<D>(dOs, a.dout + tok0 + q0 * pitch, pitch, NSA_CK, valid);
    for (int i = threadIdx.x; i < NSA_CK; i += blockDim.x) {
      const int t = q0 + i;
      float m = 0.f, inv = 0.f, dl = 0.f;
      if (t < a.T) {
        const long long si = (static_cast<long long>(b) * a.KV + kv) * a.T + t;
        m = a.stats[2 * si]; inv = 1.f / a.stats[2 * si + 1]; dl = delta[si];
      }
      qstat[3 * i] = m; qstat[3 * i + 1] = inv; qstat[3 * i + 2] = dl;
    }
    __syncthreads();
#pragma unroll
    for (int ki = 0; ki < NSA_KPW; ++ki) {
      const int r = warp * NSA_KPW + ki, c = cb + r;
      if (c >= a.Tc) continue;
      const int t_min = c * a.cmp_stride + a.cmp_len - 1;
      if (t_min >= q0 + valid) continue;
      float s[4] = {0.f, 0.f, 0.f, 0.f}, dp[4] = {0.f, 0.f, 0.f, 0.f};
      const float* kvp = ks + r * D;
      const float* vvp = vs + r * D;
      for (int d2 = 0; d2 < D / 2; ++d2) {
        const float k0 = kvp[2 * d2], k1 = kvp[2 * d2 + 1], v0 = vvp[2 * d2], v1 = vvp[2 * d2 + 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 qq = nsa_bf2(Qs + (lane + 32 * j) * P + 2 * d2);
          const float2 ee = nsa_bf2(dOs + (lane + 32 * j) * P + 2 * d2);
          s[j] = fmaf(k0, qq.x, fmaf(k1, qq.y, s[j]));
          dp[j] = fmaf(v0, ee.x, fmaf(v1, ee.y, dp[j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = lane + 32 * j, t = q0 + i;
        const bool vis = t < a.T && t >= t_min;
        const float p = vis ? __expf(s[j] - qstat[3 * i]) * qstat[3 * i + 1] : 0.f;
        pw[warp * NSA_CK + i] = p;
        dw[warp * NSA_CK + i] = p * (dp[j] - qstat[3 * i + 2]);
      }
      __syncwarp();
      const int i_lo = max(0, t_min - q0);
      const float* pp = pw + warp * NSA_CK;
      const float* dd = dw + warp * NSA_CK;
      for (int i = i_lo; i < valid; ++i) {
        const float p = pp[i], ds = dd[i];
#pragma unroll
        for (int h = 0; h < NP; ++h) {
          const float2 ee = nsa_bf2(dOs + i * P + 64 * h + 2 * lane);
          const float2 qq = nsa_bf2(Qs + i * P + 64 * h + 2 * lane);
          gv[ki][2 * h] = fmaf(p, ee.x, gv[ki][2 * h]);
          gv[ki][2 * h + 1] = fmaf(p, ee.y, gv[ki][2 * h + 1]);
          gk[ki][2 * h] = fmaf(ds, qq.x, gk[ki][2 * h]);
          gk[ki][2 * h + 1] = fmaf(ds, qq.y, gk[ki][2 * h + 1]);
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int ki = 0; ki < NSA_KPW; ++ki) {
    const int c = cb + warp * NSA_KPW + ki;
    if (c >= a.Tc) continue;
    float* rk = a.dkc + key0 + c * pitch;
    float* rv = a.dvc + key0 + c * pitch;
#pragma unroll
    for (int h = 0; h < NP; ++h) {
      *reinterpret_cast<float2*>(rk + 64 * h + 2 * lane) = make_float2(gk[ki][2 * h] * a.scale, gk[ki][2 * h + 1] * a.scale);
      *reinterpret_cast<float2*>(rv + 64 * h + 2 * lane) = make_float2(gv[ki][2 * h], gv[ki][2 * h + 1]);
    }
  }
}

template <int D>
static int nsa_smem_fwd(int Ns) {
  return 2 * NSA_CK * (D + 2) * 2 + (NSA_QB * D + NSA_WARPS * NSA_CK + NSA_QB * (Ns > D ? Ns : D)) * 4;
}
template <int D>
static int nsa_smem_dkv() {
  return 2 * NSA_CK * (D + 2) * 2 + (2 * NSA_KB * D + 2 * NSA_WARPS * NSA_CK + 3 * NSA_CK) * 4;
}

template <int D>
static int nsa_fwd_launch(const NsaCmpArgs& a, cudaStream_t st) {
  const int smem = nsa_smem_fwd<D>(a.Ns);
  cudaError_t e = cudaFuncSetAttribute(k_nsa_cmp_fwd<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((a.T + NSA_QB - 1) / NSA_QB, a.KV, a.B);
  k_nsa_cmp_fwd<D><<<grid, NSA_WARPS * 32, smem, st>>>(a);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

template <int D>
static int nsa_bwd_launch(const NsaCmpArgs& a, float* delta, cudaStream_t st) {
  const int smem_q = nsa_smem_fwd<D>(0), smem_k = nsa_smem_dkv<D>();
  cudaError_t e = cudaFuncSetAttribute(k_nsa_cmp_dq<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaFuncSetAttribute(k_nsa_cmp_dkv<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_k);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 gq((a.T + NSA_QB - 1) / NSA_QB, a.KV, a.B), gk((a.Tc + NSA_KB - 1) / NSA_KB, a.KV, a.B);
  k_nsa_cmp_dq<D><<<gq, NSA_WARPS * 32, smem_q, st>>>(a, delta);
  k_nsa_cmp_dkv<D><<<gk, NSA_WARPS * 32, smem_k, st>>>(a, delta);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // namespace nmoe

using namespace nmoe;

static int nsa_fill(NsaCmpArgs& a, int B, int T, int KV, int Tc, int Ns, int D, int cmp_len, int cmp_stride, int slc_block,
                    float scale) {
  if (D != 64 && D != 128) return -1;
  if (B <= 0 || T <= 0 || KV <= 0 || Tc <= 0 || Ns < 1 || Ns > NSA_MAX_NS || cmp_len < 1 || cmp_stride < 1 || slc_block < 1)
    return -2;
  a.B = B; a.T = T; a.KV = KV; a.Tc = Tc; a.Ns = Ns;
  a.cmp_len = cmp_len; a.cmp_stride = cmp_stride; a.slc_block = slc_block; a.scale = scale;
  return 0;
}

// q / out [B,T,KV,D], kc / vc [B,Tc,KV,D] bf16 contiguous; scores [B,T,KV,Ns] fp32 (may be null); stats [B,KV,T,2] fp32.
extern "C" int nmoe_nsa_cmp_fwd(const void* q, const void* kc, const void* vc, void* out, float* scores, float* stats, int B,
                                int T, int KV, int Tc, int Ns, int D, int cmp_len, int cmp_stride, int slc_block,
                                float scale, cudaStream_t st) {
  NsaCmpArgs a{};
  const int rc = nsa_fill(a, B, T, KV, Tc, Ns, D, cmp_len, cmp_stride, slc_block, scale);
  if (rc != 0) return rc;
  a.q = static_cast<const __nv_bfloat16*>(q); a.kc = static_cast<const __nv_bfloat16*>(kc);
  a.vc = static_cast<const __nv_bfloat16*>(vc); a.out = static_cast<__nv_bfloat16*>(out);
  a.scores = scores; a.stats = stats;
  return D == 128 ? nsa_fwd_launch<128>(a, st) : nsa_fwd_launch<64>(a, st);
}

// dq [B,T,KV,D] bf16; dkc / dvc [B,Tc,KV,D] fp32; delta [B,KV,T] fp32 scratch.  Every element of the three gradients is
// written.
extern "C" int nmoe_nsa_cmp_bwd(const void* q, const void* kc, const void* vc, const void* out, const void* dout,
                                const float* stats, void* dq, float* dkc, float* dvc, float* delta, int B, int T, int KV,
                                int Tc, int D, int cmp_len, int cmp_stride, float scale, cudaStream_t st) {
  NsaCmpArgs a{};
  const int rc = nsa_fill(a, B, T, KV, Tc, 1, D, cmp_len, cmp_stride, 1, scale);
  if (rc != 0) return rc;
  a.q = static_cast<const __nv_bfloat16*>(q); a.kc = static_cast<const __nv_bfloat16*>(kc);
  a.vc = static_cast<const __nv_bfloat16*>(vc); a.out = static_cast<__nv_bfloat16*>(const_cast<void*>(out));
  a.dout = static_cast<const __nv_bfloat16*>(dout); a.stats = const_cast<float*>(stats);
  a.dq = static_cast<__nv_bfloat16*>(dq); a.dkc = dkc; a.dvc = dvc;
  return D == 128 ? nsa_bwd_launch<128>(a, delta, st) : nsa_bwd_launch<64>(a, delta, st);
}
