// Muon orthogonaliser: for every matrix of a stack [E, R, C], Frobenius-normalise and run `steps`
// Newton-Schulz iterations  X <- a X + (b A + c A^2) X,  A = X X^T,  on the short side
// (X is taken as [min(R,C), max(R,C)]).  The whole iteration lives here: two small SIMT kernels
// (normalise + optional transpose, axpby) around the tcgen05 bf16 GEMM of this library, whose
// accumulate mode folds the "a X +" term into the last product of a step.
//
// workspace (bf16 elements): 2*m*n + 3*m*m   with m = min(R,C), n = max(R,C)
//
// Reference counterpart: nmoe/csrc/muon.cu:288-499 (cuBLAS strided-batched TF32 on fp32 copies,
// persistent plan).  Here the products run in bf16 with fp32 accumulation in tensor memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/ptx.cuh"

extern "C" int nmoe_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                              long long ldc, int a_mn, int b_mn, int mode, int E, const int* tile_expert,
                              const int* n_m_tiles, const int* offs, long long a_rows, long long b_rows, int out_fp32,
                              int accumulate, int bn, void* status, const void* push_runs, void* const* peer_ret,
                              void* const* peer_retg, const float* rowval, int push_pairs, int world, cudaStream_t st);
extern "C" int nmoe_gemm_bf16_pair(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                                   long long ldc, int a_mn, int b_mn, int mode, int E, const int* tile_expert,
                                   const int* n_m_tiles, const int* offs, long long a_rows, long long b_rows, int out_fp32,
                                   int accumulate, void* status, cudaStream_t st);

namespace nmoe {

// sum of squares of one matrix -> ssq[0] (must be zero on entry)
__global__ void __launch_bounds__(256) k_muon_sumsq(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ ssq) {
  float acc = 0.f;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i + 8 <= n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    const int4 p = ld_nc_v4(x + i);
    const float2 a = unpack_bf16x2(p.x), b = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
    acc += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0 && acc != 0.f) atomicAdd(ssq, acc);
}

// out[m, n] = x / (||x||_F + eps); x is [R, C] row-major, out is x (transpose = 0) or x^T (transpose = 1)
__global__ void __launch_bounds__(256) k_muon_normalize(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                        int R, int C, int transpose, const float* __restrict__ ssq, float eps) {
  __shared__ __nv_bfloat16 tile[32][33];
  const float inv = 1.f / (sqrtf(*ssq) + eps);
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;      // 32 x 8
  for (int j = ty; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + tx;
    float v = (r < R && c < C) ? __bfloat162float(x[static_cast<long long>(r) * C + c]) * inv : 0.f;
    if (!transpose) { if (r < R && c < C) out[static_cast<long long>(r) * C + c] = __float2bfloat16(v); }
    else tile[j][tx] = __float2bfloat16(v);
  }
  if (transpose) {
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
      const int c = c0 + j, r = r0 + tx;                         // out is [C, R]
      if (r < R && c < C) out[static_cast<long long>(c) * R + r] = tile[tx][j];
    }
  }
}

// out = alpha * x + beta * y (y may be null); optionally written transposed ([m,n] -> [n,m])
__global__ void __launch_bounds__(256) k_muon_axpby(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                                    __nv_bfloat16* __restrict__ out, long long n, float alpha, float beta) {
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i + 8 <= n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    const int4 p = ld_nc_v4(x + i);
    float v[8];
    const float2 a = unpack_bf16x2(p.x), b = unpack_bf16x2(p.y), c = unpack_bf16x2(p.z), d = unpack_bf16x2(p.w);
    v[0] = a.x * alpha; v[1] = a.y * alpha; v[2] = b.x * alpha; v[3] = b.y * alpha;
    v[4] = c.x * alpha; v[5] = c.y * alpha; v[6] = d.x * alpha; v[7] = d.y * alpha;
    if (y != nullptr) {
      const int4 q = ld_nc_v4(y + i);
      const float2 e = unpack_bf16x2(q.x), f = unpack_bf16x2(q.y), g = unpack_bf16x2(q.z), h = unpack_bf16x2(q.w);
      v[0] += e.x * beta; v[1] += e.y * beta; v[2] += f.x * beta; v[3] += f.y * beta;
      v[4] += g.x * beta; v[5] += g.y * beta; v[6] += h.x * beta; v[7] += h.y * beta;
    }
    int4 o;
    o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]); o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<int4*>(out + i) = o;
  }
}

__global__ void __launch_bounds__(256) k_muon_transpose(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                        int R, int C) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8)
    if (r0 + j < R && c0 + tx < C) tile[j][tx] = x[static_cast<long long>(r0 + j) * C + c0 + tx];
  __syncthreads();
  for (int j = ty; j < 32; j += 8)
    if (r0 + tx < R && c0 + j < C) out[static_cast<long long>(c0 + j) * R + r0 + tx] = tile[tx][j];
}

static int muon_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, int b_mn,
                     int accumulate, void* status, cudaStream_t st) {
  const long long b_rows = b_mn ? K : N;
  if (M >= 512 && N >= 256 && (N % 8) == 0)
    return nmoe_gemm_bf16_pair(A, B, C, M, N, K, lda, ldb, N, 0, b_mn, 0, 1, nullptr, nullptr, nullptr, M, b_rows, 0, accumulate,
                               status, st);
  return nmoe_gemm_bf16(A, B, C, M, N, K, lda, ldb, N, 0, b_mn, 0, 1, nullptr, nullptr, nullptr, M, b_rows, 0, accumulate, 0,
                        status, nullptr, nullptr, nullptr, nullptr, 0, 0, st);
}

}  // namespace nmoe

using namespace nmoe;

extern "C" long long nmoe_muon_workspace_elems(int R, int C) {
  const long long m = R < C ? R : C, n = R < C ? C : R;
  return 2 * m * n + 3 * m * m;
}

// x, out: [E, R, C] bf16 (may alias); ssq: E floats of scratch; workspace: nmoe_muon_workspace_elems(R, C) bf16.
// R, C multiples of 8.
extern "C" int nmoe_muon_orth(const void* x, void* out, int E, int R, int C, int steps, float a, float b, float c, float eps,
                              void* workspace, float* ssq, void* status, cudaStream_t st) {
  if (E == 0) return 0;
  if ((R % 8) != 0 || (C % 8) != 0) return -1;
  const int transpose = R > C;
  const int m = transpose ? C : R, n = transpose ? R : C;
  auto* ws = static_cast<__nv_bfloat16*>(workspace);
  __nv_bfloat16* X0 = ws;
  __nv_bfloat16* X1 = X0 + static_cast<long long>(m) * n;
  __nv_bfloat16* A = X1 + static_cast<long long>(m) * n;
  __nv_bfloat16* A2 = A + static_cast<long long>(m) * m;
  __nv_bfloat16* Bm = A2 + static_cast<long long>(m) * m;
  cudaError_t e = cudaMemsetAsync(ssq, 0, sizeof(float) * E, st);
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long mat = static_cast<long long>(R) * C;
  const long long mn = static_cast<long long>(m) * n, mm = static_cast<long long>(m) * m;
  const unsigned ew_blocks = 592;
  for (int i = 0; i < E; ++i) {
    const __nv_bfloat16* xi = static_cast<const __nv_bfloat16*>(x) + i * mat;
    __nv_bfloat16* oi = static_cast<__nv_bfloat16*>(out) + i * mat;
    k_muon_sumsq<<<ew_blocks, 256, 0, st>>>(xi, mat, ssq + i);
    k_muon_normalize<<<dim3((C + 31) / 32, (R + 31) / 32), 256, 0, st>>>(xi, X0, R, C, transpose, ssq + i, eps);
    __nv_bfloat16* cur = X0;
    __nv_bfloat16* nxt = X1;
    for (int s = 0; s < steps; ++s) {
      int rc = muon_gemm(cur, cur, A, m, m, n, n, n, 0, 0, status, st);                 // A = X X^T
      if (rc) return rc;
      rc = muon_gemm(A, A, A2, m, m, m, m, m, 0, 0, status, st);                        // A^2 (A symmetric)
      if (rc) return rc;
      k_muon_axpby<<<ew_blocks, 256, 0, st>>>(A, A2, Bm, mm, b, c);                       // B = b A + c A^2
      k_muon_axpby<<<ew_blocks, 256, 0, st>>>(cur, nullptr, nxt, mn, a, 0.f);             // X' = a X
      rc = muon_gemm(Bm, cur, nxt, m, n, m, m, n, 1, 1, status, st);                    // X' += B X
      if (rc) return rc;
      __nv_bfloat16* t = cur; cur = nxt; nxt = t;
    }
    if (transpose)
      k_muon_transpose<<<dim3((n + 31) / 32, (m + 31) / 32), 256, 0, st>>>(cur, oi, m, n);
    else
      k_muon_axpby<<<ew_blocks, 256, 0, st>>>(cur, nullptr, oi, mn, 1.f, 0.f);
  }
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
