// Token-level sparsity masks for the attention kernels (csrc/attention.cu, attention_bwd.cu).
//
// A mask is a bit matrix: row (b, q) holds one bit per key, packed into W = 2*ceil(S/64) 32-bit words; the
// backward's dK/dV kernel reads the transpose (row (b, k), one bit per query).  Three producers:
//
//   nmoe_mask_topk       per query row of a score matrix [B, S, S] (fp32, -inf = not eligible), set the bits of the
//                        k largest scores among keys <= q.  One CTA per row: the row is held in shared memory, the
//                        k-th largest value is found by a 4-pass radix select on the order-preserving integer image
//                        of the floats, ties at the threshold are admitted in key order until k bits are set.
//                        Replaces the sort inside torch.topk for DeepSeek sparse attention (the reference streams
//                        its top-k in Triton: nmoe/triton/dsa.py:225-345) and never materialises index lists.
//   nmoe_mask_from_blocks  per query, a list of selected key blocks (NSA selection branch: nmoe/attention/nsa.py
//                        :331-341) -> bits of every key of those blocks.
//   nmoe_mask_positions  the same set of key positions for every query (NSA compressed branch: compressed token j
//                        sits at the position of the last token it covers, so the causal rule of the attention
//                        kernel is exactly the reference's visibility rule for compressed blocks).
//   nmoe_mask_transpose  bit transpose [B, S, W] -> [B, S, W].
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/ptx.cuh"

namespace nmoe {

NMOE_DEVICE uint32_t float_order_key(float f) {
  // monotone map float -> uint32 (larger float = larger key); -inf maps to the smallest key of any finite value's range
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// grid = B*S rows, 256 threads; shared: S keys (uint32) + 256 histogram bins + W per-word tie counts.
__global__ void __launch_bounds__(256) k_mask_topk(const float* __restrict__ scores, int S, int W, int k,
                                                   uint32_t* __restrict__ mask) {
  extern __shared__ uint32_t sm[];
  uint32_t* keys = sm;                 // [S]   0 = not eligible
  uint32_t* hist = sm + S;             // [256]
  uint32_t* tie_pre = hist + 256;      // [W]   ties (== threshold) in the words before this one
  __shared__ uint32_t s_prefix, s_need;
  __shared__ int s_total;
  const long long rowi = blockIdx.x;
  const int q = static_cast<int>(rowi % S);
  const float* srow = scores + rowi * S;
  uint32_t* mrow = mask + rowi * W;
  const int n = q + 1;                 // eligible keys: 0..q
  const uint32_t kNegInf = float_order_key(-INFINITY);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_total = 0;
  __syncthreads();
  int eligible = 0;
  for (int j = threadIdx.x; j < S; j += 256) {
    uint32_t key = 0;
    if (j < n) {
      const float f = srow[j];
      key = (f == f) ? float_order_key(f) : 0u;       // NaN is never selected
      if (key <= kNegInf) key = 0; else ++eligible;   // -inf scores are never selected
    }
    keys[j] = key;
  }
  atomicAdd(&s_total, eligible);
  __syncthreads();
  const int total = s_total;
  const int kk = min(k, total);
  uint32_t thr = 0, ties_wanted = 0;   // default: every eligible key (key > 0) is selected
  if (kk == 0) {
    for (int w = threadIdx.x; w < W; w += 256) mrow[w] = 0u;
    return;
  }
  if (kk < total) {
    // radix select on the key bits, most significant byte first: the key of the kk-th largest element
    if (threadIdx.x == 0) { s_prefix = 0; s_need = static_cast<uint32_t>(kk); }
    __syncthreads();
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      hist[threadIdx.x] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix;
      const uint32_t pmask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
      for (int j = threadIdx.x; j < n; j += 256) {
        const uint32_t key = keys[j];
        if (key != 0 && (key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        const uint32_t need = s_need;
        uint32_t run = 0;
        int bin = 255;
        for (; bin > 0; --bin) {
          if (run + hist[bin] >= need) break;
          run += hist[bin];
        }
        s_need = need - run;           // how many are still wanted inside the chosen bin
        s_prefix = prefix | (static_cast<uint32_t>(bin) << shift);
      }
      __syncthreads();
    }
    thr = s_prefix;
    ties_wanted = s_need;              // elements equal to thr to admit, lowest key index first
  }
  // ties per word, exclusive prefix over words (key order), then the bits
  for (int w = warp; w < W; w += 8) {
    const int j = w * 32 + lane;
    const uint32_t key = j < S ? keys[j] : 0u;
    const uint32_t eq = __ballot_sync(0xffffffffu, thr != 0 && key == thr);
    if (lane == 0) tie_pre[w] = __popc(eq);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t run = 0;
    for (int w = 0; w < W; ++w) { const uint32_t c = tie_pre[w]; tie_pre[w] = run; run += c; }
  }
  __syncthreads();
  for (int w = warp; w < W; w += 8) {
    const int j = w * 32 + lane;
    const uint32_t key = j < S ? keys[j] : 0u;
    const uint32_t gt = __ballot_sync(0xffffffffu, key > thr);
    const uint32_t eq = __ballot_sync(0xffffffffu, thr != 0 && key == thr);
    const uint32_t rank = tie_pre[w] + __popc(eq & ((1u << lane) - 1u));
    const uint32_t tie_ok = __ballot_sync(0xffffffffu, ((eq >> lane) & 1u) && rank < ties_wanted);
    if (lane == 0) mrow[w] = gt | tie_ok;
  }
}

// blocks [B, S, n_sel] int32 (block index, -1 = unused) -> bits of keys [blk*bs, (blk+1)*bs) for each query.
__global__ void k_mask_from_blocks(const int* __restrict__ blocks, int n_sel, int block_size, int S, int W,
                                   uint32_t* __restrict__ mask, long long rows) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int* br = blocks + row * n_sel;
  uint32_t* mrow = mask + row * W;
  for (int w = lane; w < W; w += 32) {
    uint32_t bits = 0;
    const int k_lo = w * 32, k_hi = k_lo + 31;
    for (int s = 0; s < n_sel; ++s) {
      const int blk = br[s];
      if (blk < 0) continue;
      const int lo = blk * block_size, hi = lo + block_size - 1;
      if (hi < k_lo || lo > k_hi) continue;
      const int a = max(lo, k_lo) - k_lo, b = min(hi, k_hi) - k_lo;
      bits |= (b - a == 31) ? 0xffffffffu : (((1u << (b - a + 1)) - 1u) << a);
    }
    mrow[w] = bits;
  }
}

// the same key set for every query row: positions [n_pos] int32 (sorted or not)
__global__ void k_mask_positions(const int* __restrict__ positions, int n_pos, int S, int W, uint32_t* __restrict__ mask,
                                 long long rows) {
  extern __shared__ uint32_t words[];      // [W]
  for (int w = threadIdx.x; w < W; w += blockDim.x) words[w] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pos; i += blockDim.x) {
    const int ppos = positions[i];
    if (ppos >= 0 && ppos < S) atomicOr(&words[ppos >> 5], 1u << (ppos & 31));
  }
  __syncthreads();
  for (long long row = blockIdx.x; row < rows; row += gridDim.x)
    for (int w = threadIdx.x; w < W; w += blockDim.x) mask[row * W + w] = words[w];
}

// out[(b, k), q/32] bit q%32 = in[(b, q), k/32] bit k%32.  One warp transposes a 32x32 bit tile.
__global__ void k_mask_transpose(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int S, int W) {
  const int lane = threadIdx.x & 31;
  const int tile_q = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);   // 32-query group
  const int tile_k = blockIdx.y;                                            // 32-key word
  const int b = blockIdx.z;
  if (tile_q * 32 >= S || tile_k >= W) return;
  const int q = tile_q * 32 + lane;
  const uint32_t word = q < S ? in[(static_cast<size_t>(b) * S + q) * W + tile_k] : 0u;
  const int k = tile_k * 32 + lane;
  uint32_t outw = 0;
#pragma unroll
  for (int t = 0; t < 32; ++t) {
    // bit t of every lane's word -> lane t gets the ballot: out row k = tile_k*32 + t, bit = lane (query)
    const uint32_t bal = __ballot_sync(0xffffffffu, (word >> t) & 1u);
    if (lane == t) outw = bal;
  }
  if (k < S) out[(static_cast<size_t>(b) * S + k) * W + tile_q] = outw;
}

}  // namespace nmoe

using namespace nmoe;

extern "C" {

int nmoe_mask_words(int S) { return 2 * ((S + 63) / 64); }

// scores [B, S, S] fp32 (row q: scores of keys; entries beyond q are ignored), mask [B, S, W] out.
int nmoe_mask_topk(const float* scores, int B, int S, int k, void* mask, cudaStream_t st) {
  if (B == 0 || S == 0) return 0;
  if (k <= 0) return -1;
  const int W = nmoe_mask_words(S);
  const size_t smem = (static_cast<size_t>(S) + 256 + W) * 4;
  if (smem > 200 * 1024) return -2;                 // rows up to ~50k keys
  cudaError_t e = cudaFuncSetAttribute(k_mask_topk, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  if (e != cudaSuccess) return static_cast<int>(e);
  k_mask_topk<<<static_cast<unsigned>(static_cast<long long>(B) * S), 256, smem, st>>>(scores, S, W, k,
                                                                                    static_cast<uint32_t*>(mask));
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

int nmoe_mask_from_blocks(const int* blocks, int B, int S, int n_sel, int block_size, void* mask, cudaStream_t st) {
  if (B == 0 || S == 0) return 0;
  const long long rows = static_cast<long long>(B) * S;
  k_mask_from_blocks<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(blocks, n_sel, block_size, S, nmoe_mask_words(S),
                                                                           static_cast<uint32_t*>(mask), rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

int nmoe_mask_positions(const int* positions, int n_pos, int B, int S, void* mask, cudaStream_t st) {
  if (B == 0 || S == 0) return 0;
  const int W = nmoe_mask_words(S);
  k_mask_positions<<<148 * 2, 256, W * 4, st>>>(positions, n_pos, S, W, static_cast<uint32_t*>(mask),
                                               static_cast<long long>(B) * S);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

int nmoe_mask_transpose(const void* in, void* out, int B, int S, cudaStream_t st) {
  if (B == 0 || S == 0) return 0;
  const int W = nmoe_mask_words(S);
  dim3 grid(((S + 31) / 32 + 7) / 8, W, B);
  k_mask_transpose<<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), S, W);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // extern "C"
