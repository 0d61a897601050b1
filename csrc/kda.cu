// Chunk scan of the gated delta rule (Kimi Delta Attention and other delta-rule linear attentions).
//
// With the WY / UT transform the in-chunk dependencies of the delta rule are solved by one triangular solve per
// chunk that does not involve the running state, so for a chunk of C tokens
//     W = U - P S                      written values                       [C, Dv]
//     S <- diag(dec) S + K2^T W (+ G)  state after the chunk                [Dk, Dv]
// where U [C, Dv], P [C, Dk], K2 [C, Dk], dec [Dk] (and the optional additive term G [Dk, Dv]) are computed for all
// chunks at once with batched matrix products.  The only sequential part is this recurrence over chunks, and that is
// what the kernel below runs: one CTA per (batch x head, slice of Dv columns) keeps its slice of S in shared memory,
// walks the chunks in order (or in reverse), writes W of every chunk and, on request, the state each chunk started
// from.  The backward pass of the layer is the same recurrence run in reverse on transformed operands
// (dW = U' + KiE dS, dS <- dec dS + (-P)^T dW + Qd^T dO), so one kernel serves both directions.
//
// Everything is fp32 (linear-attention states do not tolerate bf16 accumulation over thousands of tokens).
// Replaces the chunked Triton kernels of the reference (nmoe/triton/kda.py:202-1080: chunk_gated_delta_rule forward
// and backward, the WY representation and the inter-chunk state passing).
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/ptx.cuh"

namespace nmoe {

constexpr int KDA_C = 64;        // tokens per chunk
constexpr int KDA_THREADS = 256;
// Dv columns per CTA (VL) is a template parameter: 64, 32 or 16.  The recurrence is a dependency chain per (head,
// column slice), so with few heads a narrower slice puts more CTAs on the machine and shortens every chain; the price
// is that P and K2 of a chunk are read (from L2) once per slice.

struct KdaScanArgs {
  int n_chunks, Dk, Dv, reverse;
  const float* U;      // [BH, n, C, Dv]
  const float* P;      // [BH, n, C, Dk]
  const float* K2;     // [BH, n, C, Dk]
  const float* dec;    // [BH, n, Dk]
  const float* G;      // [BH, n, Dk, Dv] or null
  const float* S0;     // [BH, Dk, Dv] or null (zero initial state)
  float* W;            // [BH, n, C, Dv]
  float* S_hist;       // [BH, n, Dk, Dv] or null: state each chunk started from (in scan order)
  float* S_final;      // [BH, Dk, Dv] or null
};

// Shared memory: S [Dk][VL] | Wc [C][VL] | X [C][Dk]
template <int KDA_VL>
__global__ void __launch_bounds__(KDA_THREADS) k_kda_scan(const KdaScanArgs a) {
  constexpr int NQ = KDA_VL / 4;               // column quads of the slice
  constexpr int RG = KDA_THREADS / NQ;         // row groups: 16 / 32 / 64
  constexpr int RPT = KDA_C / RG;              // rows of a [C][VL] tile per thread: 4 / 2 / 1
  constexpr int GS = KDA_VL == 16 ? 2 : 4;     // state rows per thread and pass of the update
  extern __shared__ float kda_smem[];
  const int Dk = a.Dk, Dv = a.Dv;
  float* S = kda_smem;                       // [Dk][VL]
  float* Wc = S + Dk * KDA_VL;               // [C][VL]
  float* X = Wc + KDA_C * KDA_VL;            // [C][Dk]
  const int bh = blockIdx.x;
  const int v_base = blockIdx.y * KDA_VL;
  const int t = threadIdx.x;
  // [C][VL] outputs: thread -> RPT rows x 4 columns
  const int vq = (t % NQ) * 4;               // column quad inside the slice
  const int rq = (t / NQ) * RPT;             // first of its rows

  // initial state
  for (int i = t; i < Dk * (KDA_VL / 4); i += KDA_THREADS) {
    const int k = i / (KDA_VL / 4), q = (i % (KDA_VL / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.S0 != nullptr) v = *reinterpret_cast<const float4*>(a.S0 + (static_cast<size_t>(bh) * Dk + k) * Dv + v_base + q);
    *reinterpret_cast<float4*>(S + k * KDA_VL + q) = v;
  }
  __syncthreads();

  for (int step = 0; step < a.n_chunks; ++step) {
    const int c = a.reverse ? a.n_chunks - 1 - step : step;
    const size_t chunk = static_cast<size_t>(bh) * a.n_chunks + c;
    // state this chunk starts from
    if (a.S_hist != nullptr) {
      float* dst = a.S_hist + chunk * Dk * Dv;
      for (int i = t; i < Dk * (KDA_VL / 4); i += KDA_THREADS) {
        const int k = i / (KDA_VL / 4), q = (i % (KDA_VL / 4)) * 4;
        *reinterpret_cast<float4*>(dst + static_cast<size_t>(k) * Dv + v_base + q) = *reinterpret_cast<const float4*>(S + k * KDA_VL + q);
      }
    }
    // X <- P[c]
    const float* Pc = a.P + chunk * KDA_C * Dk;
    for (int i = t * 4; i < KDA_C * Dk; i += KDA_THREADS * 4)
      *reinterpret_cast<float4*>(X + i) = *reinterpret_cast<const float4*>(Pc + i);
    __syncthreads();
    // W = U - P S
    {
      float acc[RPT][4];
      const float* Uc = a.U + chunk * KDA_C * Dv;
#pragma unroll
      for (int j = 0; j < RPT; ++j) {
        const float4 u = *reinterpret_cast<const float4*>(Uc + static_cast<size_t>(rq + j) * Dv + v_base + vq);
        acc[j][0] = u.x; acc[j][1] = u.y; acc[j][2] = u.z; acc[j][3] = u.w;
      }
      for (int k = 0; k < Dk; k += 4) {
        float4 s4[4];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) s4[kk] = *reinterpret_cast<const float4*>(S + (k + kk) * KDA_VL + vq);
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          const float4 p4 = *reinterpret_cast<const float4*>(X + (rq + j) * Dk + k);
          const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            acc[j][0] = fmaf(-pv[kk], s4[kk].x, acc[j][0]); acc[j][1] = fmaf(-pv[kk], s4[kk].y, acc[j][1]);
            acc[j][2] = fmaf(-pv[kk], s4[kk].z, acc[j][2]); acc[j][3] = fmaf(-pv[kk], s4[kk].w, acc[j][3]);
          }
        }
      }
      float* Wg = a.W + chunk * KDA_C * Dv;
#pragma unroll
      for (int j = 0; j < RPT; ++j) {
        const float4 w = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
        *reinterpret_cast<float4*>(Wc + (rq + j) * KDA_VL + vq) = w;
        *reinterpret_cast<float4*>(Wg + static_cast<size_t>(rq + j) * Dv + v_base + vq) = w;
      }
    }
    __syncthreads();
    // X <- K2[c]
    const float* Kc = a.K2 + chunk * KDA_C * Dk;
    for (int i = t * 4; i < KDA_C * Dk; i += KDA_THREADS * 4)
      *reinterpret_cast<float4*>(X + i) = *reinterpret_cast<const float4*>(Kc + i);
    __syncthreads();
    // S = dec S + K2^T W (+ G): thread -> rows k = kq + 16*i, 4 columns; Dk/16 rows per thread in groups of 4
    {
      const float* dc = a.dec + chunk * Dk;
      const float* Gc = a.G != nullptr ? a.G + chunk * Dk * Dv : nullptr;
      const int kq = t / NQ;                  // 0..RG-1
      for (int k0 = kq; k0 < Dk; k0 += GS * RG) {  // rows k0, k0 + RG, ...
        float acc[GS][4];
#pragma unroll
        for (int i = 0; i < GS; ++i)
#pragma unroll
          for (int x = 0; x < 4; ++x) acc[i][x] = 0.f;
        for (int j = 0; j < KDA_C; ++j) {
          const float4 w = *reinterpret_cast<const float4*>(Wc + j * KDA_VL + vq);
#pragma unroll
          for (int i = 0; i < GS; ++i) {
            const int k = k0 + RG * i;
            const float kv = k < Dk ? X[j * Dk + k] : 0.f;
            acc[i][0] = fmaf(kv, w.x, acc[i][0]); acc[i][1] = fmaf(kv, w.y, acc[i][1]);
            acc[i][2] = fmaf(kv, w.z, acc[i][2]); acc[i][3] = fmaf(kv, w.w, acc[i][3]);
          }
        }
#pragma unroll
        for (int i = 0; i < GS; ++i) {
          const int k = k0 + RG * i;
          if (k >= Dk) continue;
          const float d = dc[k];
          float4 s = *reinterpret_cast<const float4*>(S + k * KDA_VL + vq);
          s.x = fmaf(d, s.x, acc[i][0]); s.y = fmaf(d, s.y, acc[i][1]);
          s.z = fmaf(d, s.z, acc[i][2]); s.w = fmaf(d, s.w, acc[i][3]);
          if (Gc != nullptr) {
            const float4 g = *reinterpret_cast<const float4*>(Gc + static_cast<size_t>(k) * Dv + v_base + vq);
            s.x += g.x; s.y += g.y; s.z += g.z; s.w += g.w;
          }
          *reinterpret_cast<float4*>(S + k * KDA_VL + vq) = s;
        }
      }
    }
    __syncthreads();
  }
  if (a.S_final != nullptr) {
    for (int i = t; i < Dk * (KDA_VL / 4); i += KDA_THREADS) {
      const int k = i / (KDA_VL / 4), q = (i % (KDA_VL / 4)) * 4;
      *reinterpret_cast<float4*>(a.S_final + (static_cast<size_t>(bh) * Dk + k) * Dv + v_base + q) =
          *reinterpret_cast<const float4*>(S + k * KDA_VL + q);
    }
  }
}

}  // namespace nmoe

using namespace nmoe;

// All tensors fp32 and contiguous with the shapes given in KdaScanArgs; chunk length is 64 tokens.
// Dk % 4 == 0 (<= 256), Dv % 64 == 0 (the column slice per CTA is chosen from the grid size).  reverse != 0 walks the chunks from last to first (S_hist then holds, per
// chunk, the state the reverse walk entered it with).
extern "C" int nmoe_kda_scan(const float* U, const float* P, const float* K2, const float* dec, const float* G,
                             const float* S0, float* W, float* S_hist, float* S_final, int BH, int n_chunks, int Dk,
                             int Dv, int reverse, cudaStream_t st) {
  if (BH == 0 || n_chunks == 0) return 0;
  if (Dk % 4 != 0 || Dk > 256 || Dv % 64 != 0) return -1;
  KdaScanArgs a;
  a.n_chunks = n_chunks; a.Dk = Dk; a.Dv = Dv; a.reverse = reverse;
  a.U = U; a.P = P; a.K2 = K2; a.dec = dec; a.G = G; a.S0 = S0; a.W = W; a.S_hist = S_hist; a.S_final = S_final;
  // the widest column slice that still gives every SM a CTA (narrowest otherwise)
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int vl = (static_cast<long long>(BH) * (Dv / 64) >= sms) ? 64 : (static_cast<long long>(BH) * (Dv / 32) >= sms) ? 32 : 16;
  const int smem = (Dk * vl + KDA_C * vl + KDA_C * Dk) * static_cast<int>(sizeof(float));
  dim3 grid(BH, Dv / vl);
  cudaError_t e;
#define KDA_GO(VL_)                                                                                             \
  e = cudaFuncSetAttribute(k_kda_scan<VL_>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);                 \
  if (e != cudaSuccess) return static_cast<int>(e);                                                             \
  k_kda_scan<VL_><<<grid, KDA_THREADS, smem, st>>>(a)
  if (vl == 64) { KDA_GO(64); } else if (vl == 32) { KDA_GO(32); } else { KDA_GO(16); }
#undef KDA_GO
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
