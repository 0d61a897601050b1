// ZeRO-2 step as ONE kernel over peer memory: reduce-scatter + grad scale + AdamW + all-gather.
//
// Every rank keeps the full flat bf16 gradient and parameter buffers of a group in a
// peer-mapped slab.  Rank r owns shard r.  The kernel
//   1. announces "my gradients are final" to every peer and waits (bounded) for theirs,
//   2. for each 8-element vector of its shard: loads that vector from all W ranks' gradient
//      buffers straight over NVLink, sums in fp32 in rank order, scales by 1/W, applies AdamW
//      (bf16 moments, fp32 math, decoupled decay first) and stores the new bf16 parameters into
//      all W ranks' parameter buffers with 16-byte system-scope stores,
//   3. after the last block finishes, releases a "my shard is published" flag to every peer -- unless a block
//      gave up waiting in step 1: then the shard was not updated, nothing is published, and the peers' own
//      bounded waits on this rank's flag run out and report too, instead of training on a half-updated shard.
// A following wait (nmoe_rdep_wait on the done flags) closes the step.  Replaces NCCL
// reduce_scatter_tensor + six eager AdamW ops + all_gather_into_tensor (nmoe/zero2.py:221-279).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/ptx.cuh"

namespace nmoe {

constexpr int kZMaxRanks = 8;

struct Zero2Args {
  int rank, world;
  long long shard_elems;            // elements per shard (multiple of 8)
  const __nv_bfloat16* peer_grad[kZMaxRanks];
  __nv_bfloat16* peer_param[kZMaxRanks];
  uint32_t* peer_ready_flags[kZMaxRanks];   // peer's array [world]; we write entry `rank`
  uint32_t* peer_done_flags[kZMaxRanks];
  const uint32_t* my_ready_flags;
  __nv_bfloat16* m;                 // [shard_elems]
  __nv_bfloat16* v;
  float lr, beta1, beta2, eps, wd, inv_bc1, inv_bc2_sqrt, grad_scale;
  uint32_t epoch;
  uint32_t spin_budget;
  int* done_counter;
  float* gradnorm_sq;               // optional: += sum of squares of the averaged shard gradient
  StatusRecord* status;
};

__global__ void __launch_bounds__(256) k_zero2_fused(const Zero2Args a) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  // 1. announce + wait
  if (blockIdx.x == 0 && threadIdx.x < a.world)
    st_release_sys_u32(a.peer_ready_flags[threadIdx.x] + a.rank, a.epoch);
  __syncthreads();
  if (threadIdx.x < a.world) {
    if (!wait_flag_ge_sys(a.my_ready_flags + threadIdx.x, a.epoch, a.spin_budget)) {
      report_status(a.status, kStatusWaitTimeout, 500, threadIdx.x, static_cast<int>(a.epoch));
      s_ok = 0;
    }
  }
  __syncthreads();
  float nsq = 0.f;
  if (s_ok) {
    const long long base = static_cast<long long>(a.rank) * a.shard_elems;
    const long long nvec = a.shard_elems >> 3;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < a.world; ++r) {
        const int4 gv = ld_relaxed_sys_v4(reinterpret_cast<const int4*>(a.peer_grad[r] + base) + i);
        const float2 f0 = unpack_bf16x2(gv.x), f1 = unpack_bf16x2(gv.y), f2 = unpack_bf16x2(gv.z), f3 = unpack_bf16x2(gv.w);
        g[0] += f0.x; g[1] += f0.y; g[2] += f1.x; g[3] += f1.y;
        g[4] += f2.x; g[5] += f2.y; g[6] += f3.x; g[7] += f3.y;
      }
      int4 pv = *(reinterpret_cast<const int4*>(a.peer_param[a.rank] + base) + i);
      int4 mv = *(reinterpret_cast<const int4*>(a.m) + i);
      int4 vv = *(reinterpret_cast<const int4*>(a.v) + i);
      uint32_t* pw = reinterpret_cast<uint32_t*>(&pv);
      uint32_t* mw = reinterpret_cast<uint32_t*>(&mv);
      uint32_t* vw = reinterpret_cast<uint32_t*>(&vv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 pf = unpack_bf16x2(pw[j]), mf = unpack_bf16x2(mw[j]), vf = unpack_bf16x2(vw[j]);
        const float g0 = g[2 * j] * a.grad_scale, g1 = g[2 * j + 1] * a.grad_scale;
        nsq += g0 * g0 + g1 * g1;
        pf.x *= (1.f - a.lr * a.wd); pf.y *= (1.f - a.lr * a.wd);
        mf.x = a.beta1 * mf.x + (1.f - a.beta1) * g0; mf.y = a.beta1 * mf.y + (1.f - a.beta1) * g1;
        vf.x = a.beta2 * vf.x + (1.f - a.beta2) * g0 * g0; vf.y = a.beta2 * vf.y + (1.f - a.beta2) * g1 * g1;
        pf.x -= a.lr * a.inv_bc1 * mf.x / (sqrtf(vf.x) * a.inv_bc2_sqrt + a.eps);
        pf.y -= a.lr * a.inv_bc1 * mf.y / (sqrtf(vf.y) * a.inv_bc2_sqrt + a.eps);
        pw[j] = pack_bf16x2(pf.x, pf.y); mw[j] = pack_bf16x2(mf.x, mf.y); vw[j] = pack_bf16x2(vf.x, vf.y);
      }
      *(reinterpret_cast<int4*>(a.m) + i) = mv;
      *(reinterpret_cast<int4*>(a.v) + i) = vv;
      for (int r = 0; r < a.world; ++r)
        st_relaxed_sys_v4(reinterpret_cast<int4*>(a.peer_param[r] + base) + i, pv);
    }
  }
  if (a.gradnorm_sq != nullptr) {
    nsq = warp_sum(nsq);
    if ((threadIdx.x & 31) == 0 && nsq != 0.f) atomicAdd(a.gradnorm_sq, nsq);
  }
  // 3. grid completion -> publish
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last, s_failed;
  if (threadIdx.x == 0) {
    constexpr int kFailedBit = 1 << 30;
    if (!s_ok) atomicOr(a.done_counter, kFailedBit);
    const int old = atomicAdd(a.done_counter, 1);
    s_last = ((old & (kFailedBit - 1)) == static_cast<int>(gridDim.x) - 1);
    s_failed = s_last ? ((atomicOr(a.done_counter, 0) & kFailedBit) != 0) : 0;
  }
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (!s_failed && threadIdx.x < a.world) st_release_sys_u32(a.peer_done_flags[threadIdx.x] + a.rank, a.epoch);
    if (threadIdx.x == 0) *a.done_counter = 0;
  }
}

}  // namespace nmoe

using namespace nmoe;

extern "C" int nmoe_zero2_fused(int rank, int world, long long shard_elems, void* const* peer_grad,
                                void* const* peer_param, void* const* peer_ready_flags, void* const* peer_done_flags,
                                void* m, void* v, float lr, float beta1, float beta2, float eps, float wd, int step,
                                float grad_scale, unsigned epoch, unsigned spin_budget, int* done_counter,
                                float* gradnorm_sq, void* status, cudaStream_t st) {
  if (world > kZMaxRanks || (shard_elems % 8) != 0) return -1;
  if (shard_elems == 0) return 0;
  Zero2Args a;
  a.rank = rank; a.world = world; a.shard_elems = shard_elems;
  for (int r = 0; r < world; ++r) {
    a.peer_grad[r] = static_cast<const __nv_bfloat16*>(peer_grad[r]);
    a.peer_param[r] = static_cast<__nv_bfloat16*>(peer_param[r]);
    a.peer_ready_flags[r] = static_cast<uint32_t*>(peer_ready_flags[r]);
    a.peer_done_flags[r] = static_cast<uint32_t*>(peer_done_flags[r]);
  }
  a.my_ready_flags = a.peer_ready_flags[rank];
  a.m = static_cast<__nv_bfloat16*>(m); a.v = static_cast<__nv_bfloat16*>(v);
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.inv_bc1 = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
  a.inv_bc2_sqrt = 1.f / sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  a.grad_scale = grad_scale; a.epoch = epoch;
  a.spin_budget = spin_budget ? spin_budget : 20u * 1000u * 1000u;
  a.done_counter = done_counter; a.gradnorm_sq = gradnorm_sq; a.status = static_cast<StatusRecord*>(status);
  const long long nvec = shard_elems / 8;
  long long blocks = (nvec + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  k_zero2_fused<<<static_cast<unsigned>(blocks), 256, 0, st>>>(a);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
