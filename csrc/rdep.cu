// RDEP: expert parallelism by direct placement into the owner's memory, with no all-to-all.
//
// A rank that holds T tokens with top-K routing does, per MoE layer:
//   count   stable rank of every (token, slot) pair inside its expert        (local)
//   plan    publish my per-expert counts into every peer's table, wait for theirs, and derive
//           -- identically on every rank -- the 128-row-aligned segment layout of every owner
//   place   store each row (bf16) straight into its final position in the owner's activation
//           buffer over NVLink (16-byte system-scope stores), plus a 16-byte meta record
//           {source rank, token*K+slot, gate}; the owner zero-fills the padding rows of its own
//           segments; the last block releases a per-peer "rows have landed" flag
//   wait    bounded spin until all peers' flags reached this call's epoch
// The owner then runs grouped GEMMs over its padded segments.  Rows go back in RUNS: inside an expert's segment
// the rows of one source rank are contiguous (placement is rank-major), so the owner writes each (expert, source)
// run as one contiguous block into the source's return buffer, which is laid out in the source's own expert-major
// order (offset = rows that source sent to lower experts).  Every transfer over NVLink is therefore a sequential
// stream of whole rows -- from the last GEMM's epilogue or from the push kernel -- and needs no per-row metadata.
// A reduce kernel on the source gathers its K slots by index, applies the gates and sums in a fixed order.
//
// Placement is deterministic (no remote atomics): position = segment start + rows of lower
// ranks + stable local rank.  Every spin has an iteration bound and reports through a
// StatusRecord instead of trapping.
//
// Replaces nmoe/csrc/rdep.cu:767-861 (dispatch), :1225-1367 (sort/offsets/pad map),
// :1308-1440 (gathers), :2698-2900 (return + reduce), :3699-3762 (barriers) of the reference.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/epilogue.cuh"
#include "common/ptx.cuh"
#include "common/quant_dev.cuh"

namespace nmoe {

constexpr int kMaxRanks = 8;
constexpr int kMaxExperts = 512;
constexpr int kCountThreads = 1024;
constexpr uint32_t kFlagSpinBudget = 20u * 1000u * 1000u;   // ~ seconds with nanosleep(64)

struct RdepMeta {          // 16 bytes, written by the source next to each row
  int32_t src_rank;
  int32_t tok_slot;        // token * K + slot on the source
  float gate;
  int32_t valid;           // 1 for a real row, 0 for padding
};

// ------------------------------------------------------------------ count
// Block b owns pairs [b*1024, (b+1)*1024).  Outputs the per-block histogram and each pair's
// stable rank among the pairs of the same expert inside the block.
__global__ void __launch_bounds__(kCountThreads)
k_rdep_count(const int* __restrict__ eid, int n_pairs, int E, int* __restrict__ block_hist,
             int* __restrict__ rank_in_block, StatusRecord* status) {
  extern __shared__ int s_warp_hist[];   // [32][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) s_warp_hist[i] = 0;
  __syncthreads();
  const int i = blockIdx.x * kCountThreads + threadIdx.x;
  int e = -1;
  if (i < n_pairs) {
    e = eid[i];
    if (e < 0 || e >= E) {
      report_status(status, kStatusBadIndex, 400, i, e);
      e = -1;
    }
  }
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int r_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && r_in_warp == 0) s_warp_hist[warp * E + e] = __popc(peers);
  __syncthreads();
  // exclusive scan over warps, per expert
  for (int x = threadIdx.x; x < E; x += blockDim.x) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = s_warp_hist[w * E + x];
      s_warp_hist[w * E + x] = run;
      run += c;
    }
    block_hist[blockIdx.x * E + x] = run;
  }
  __syncthreads();
  if (i < n_pairs) rank_in_block[i] = (e >= 0) ? s_warp_hist[warp * E + e] + r_in_warp : -1;
}

// ------------------------------------------------------------------ plan
struct PlanArgs {
  int rank, world, E, n_local, n_blocks, capacity_rows, epoch;
  int align;                    // segment alignment in rows: 128, or 256 when the two-SM grouped GEMM is used
  int* block_hist;              // [n_blocks][E] in: counts, out: exclusive prefix over blocks
  int* peer_counts[kMaxRanks];  // peer r's table [world][E]; we write row `rank`
  uint32_t* peer_count_flags[kMaxRanks];   // peer r's flags [world]; we write entry `rank`
  int* my_counts_table;         // == peer_counts[rank]
  uint32_t* my_count_flags;     // == peer_count_flags[rank]
  int* base;                    // out [E]: first position of my rows of expert e in the owner's buffer
  int* offs_pad;                // out [n_local+1]: my (owner) padded segment offsets
  int* seg_rows;                // out [n_local]: real rows in each of my segments
  int* tile_expert;             // out [capacity_rows/128]
  int* n_m_tiles;               // out [1]
  int* send_counts;             // out [E]: my counts (for stats / loads)
  int* send_prefix;             // out [E]: exclusive prefix of my counts = row of my first pair of expert e in MY return buffer
  // out [3][n_local][world], owner side, for local expert le and source rank s:
  //   [0] first row of s's run inside my buffer, [1] its length (0 when the expert was dropped),
  //   [2] first row of that run inside s's return buffer
  int* runs;
  StatusRecord* status;
};

__global__ void __launch_bounds__(512) k_rdep_plan(const PlanArgs a) {
  __shared__ int s_cnt[kMaxExperts];
  __shared__ int s_total[kMaxExperts];
  __shared__ int s_lower[kMaxExperts];
  __shared__ int s_ok;
  const int E = a.E;
  // 1. prefix over blocks -> my counts
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int b = 0; b < a.n_blocks; ++b) {
      const int c = a.block_hist[b * E + e];
      a.block_hist[b * E + e] = run;
      run += c;
    }
    s_cnt[e] = run;
    a.send_counts[e] = run;
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // 2. publish my counts to every peer, then flag
  for (int r = 0; r < a.world; ++r)
    for (int e = threadIdx.x; e < E; e += blockDim.x) a.peer_counts[r][a.rank * E + e] = s_cnt[e];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world) st_release_sys_u32(a.peer_count_flags[threadIdx.x] + a.rank, static_cast<uint32_t>(a.epoch));
  // 3. wait for every peer's counts
  if (threadIdx.x < a.world) {
    if (!wait_flag_ge_sys(a.my_count_flags + threadIdx.x, static_cast<uint32_t>(a.epoch), kFlagSpinBudget)) {
      report_status(a.status, kStatusWaitTimeout, 410, threadIdx.x, a.epoch);
      s_ok = 0;
    }
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0) *a.n_m_tiles = 0;
    for (int e = threadIdx.x; e < E; e += blockDim.x) a.base[e] = -1;
    return;
  }
  // 4. totals and rows of lower ranks
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, low = 0;
    for (int r = 0; r < a.world; ++r) {
      const int c = reinterpret_cast<volatile int*>(a.my_counts_table)[r * E + e];
      if (r < a.rank) low += c;
      tot += c;
    }
    s_total[e] = tot;
    s_lower[e] = low;
  }
  __syncthreads();
  // 4b. return-run tables.  Thread s < world walks source s's counts once: the running sum over experts is where
  // that source keeps the rows of expert e in its return buffer.  Thread `world` scans my own counts the same way.
  if (threadIdx.x < a.world) {
    const int s = threadIdx.x;
    const int nlw = a.n_local * a.world;
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = reinterpret_cast<volatile int*>(a.my_counts_table)[s * E + e];
      const int le = e - a.rank * a.n_local;
      if (le >= 0 && le < a.n_local) {
        a.runs[nlw + le * a.world + s] = c;          // length (zeroed below if the expert is dropped)
        a.runs[2 * nlw + le * a.world + s] = run;    // row in s's return buffer
      }
      run += c;
    }
  } else if (threadIdx.x == a.world) {
    int run = 0;
    for (int e = 0; e < E; ++e) { a.send_prefix[e] = run; run += s_cnt[e]; }
  }
  __syncthreads();
  // 5. segment starts per owner (serial per owner; E is small)
  if (threadIdx.x < a.world) {
    const int o = threadIdx.x;
    int run = 0;
    for (int le = 0; le < a.n_local; ++le) {
      const int e = o * a.n_local + le;
      const int padded = (s_total[e] + a.align - 1) & ~(a.align - 1);
      if (run + padded > a.capacity_rows) {
        report_status(a.status, kStatusCapacity, 411, o, run + padded);
        a.base[e] = -1;          // rows for this expert are dropped by `place`
      } else {
        a.base[e] = run + s_lower[e];
      }
      if (o == a.rank) {
        // where each source's run starts inside my segment (rank-major), or an empty run when the expert is dropped
        const bool dropped = run + padded > a.capacity_rows;
        int at = run;
        for (int s = 0; s < a.world; ++s) {
          const int c = reinterpret_cast<volatile int*>(a.my_counts_table)[s * E + e];
          a.runs[le * a.world + s] = at;
          if (dropped) a.runs[a.n_local * a.world + le * a.world + s] = 0;
          at += c;
        }
        a.offs_pad[le] = run;
        a.seg_rows[le] = (run + padded > a.capacity_rows) ? 0 : s_total[e];
        if (run + padded <= a.capacity_rows)
          for (int t = run / 128; t < (run + padded) / 128; ++t) a.tile_expert[t] = le;
      }
      if (run + padded <= a.capacity_rows) run += padded;
    }
    if (o == a.rank) {
      a.offs_pad[a.n_local] = run;
      *a.n_m_tiles = run / 128;
    }
  }
}

// ------------------------------------------------------------------ place
struct PlaceArgs {
  int rank, world, E, n_local, T, K, H, epoch;
  const __nv_bfloat16* x;        // [T, H]
  const int* eid;                // [T*K]
  const float* gates;            // [T*K] or null (backward re-dispatch / dY dispatch)
  const int* rank_in_block;      // [T*K]
  const int* block_prefix;       // [n_blocks][E]
  const int* base;               // [E]
  const int* send_prefix;        // [E] row of my first pair of expert e in my return buffer
  int* lpos_out;                 // [T*K] out: row of the pair in my return buffer (-1 = dropped)
  __nv_bfloat16* peer_x[kMaxRanks];     // owner activation buffers [capacity, H]
  RdepMeta* peer_meta[kMaxRanks];       // owner meta [capacity] (null: do not write meta)
  uint32_t* peer_data_flags[kMaxRanks]; // owner's flags [world]; we release entry `rank`
  int* pos_out;                  // [T*K] out: owner << 24 | position... stored as two arrays below
  int* owner_out;                // [T*K] or null
  const int* offs_pad;           // my segments (for pad zero-fill)
  const int* seg_rows;
  int* done_counter;             // grid-completion counter (zeroed by the last block)
  int pad_blocks;                // trailing blocks that zero-fill my padding rows
  StatusRecord* status;
};

__global__ void __launch_bounds__(256) k_rdep_place(const PlaceArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_blocks = gridDim.x - a.pad_blocks;
  const int nvec = a.H >> 3;
  if (static_cast<int>(blockIdx.x) < row_blocks) {
    // one warp per token: lane k (< K) resolves the destination of slot k, then the row is read ONCE in
    // chunks of 256 16-byte vectors and every chunk is stored to the K owners
    for (int tok = blockIdx.x * 8 + warp; tok < a.T; tok += row_blocks * 8) {
      int pos = -1, owner = 0;
      if (lane < a.K) {
        const int i = tok * a.K + lane;
        const int e = a.eid[i];
        const int rb = a.rank_in_block[i];
        int lp = -1;
        if (e >= 0 && e < a.E && rb >= 0 && a.base[e] >= 0) {
          owner = e / a.n_local;
          const int within = a.block_prefix[(i / kCountThreads) * a.E + e] + rb;
          pos = a.base[e] + within;
          lp = a.send_prefix[e] + within;
        }
        a.pos_out[i] = pos;
        if (a.lpos_out) a.lpos_out[i] = lp;
        if (a.owner_out) a.owner_out[i] = owner;
        if (pos >= 0 && a.peer_meta[owner] != nullptr) {
          int4 m;
          m.x = a.rank;
          m.y = i;
          m.z = __float_as_int(a.gates ? a.gates[i] : 1.f);
          m.w = 1;
          st_relaxed_sys_v4(a.peer_meta[owner] + pos, m);
        }
      }
      const int4* src = reinterpret_cast<const int4*>(a.x + static_cast<size_t>(tok) * a.H);
      for (int c0 = 0; c0 < nvec; c0 += 256) {
        int4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = c0 + j * 32 + lane;
          v[j] = c < nvec ? __ldg(src + c) : make_int4(0, 0, 0, 0);
        }
        for (int k = 0; k < a.K; ++k) {
          const int pk = __shfl_sync(0xffffffffu, pos, k);
          const int ok = __shfl_sync(0xffffffffu, owner, k);
          if (pk < 0) continue;
          int4* dst = reinterpret_cast<int4*>(a.peer_x[ok] + static_cast<size_t>(pk) * a.H);
          if (ok == a.rank) {
            // rows that stay on this GPU: ordinary stores (the flag release at the end of the grid orders them)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int c = c0 + j * 32 + lane;
              if (c < nvec) dst[c] = v[j];
            }
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int c = c0 + j * 32 + lane;
              if (c < nvec) st_relaxed_sys_v4(dst + c, v[j]);
            }
          }
        }
      }
    }
  } else {
    // zero-fill the padding rows of my own segments (local stores)
    const int pb = blockIdx.x - row_blocks;
    for (int le = 0; le < a.n_local; ++le) {
      const int r0 = a.offs_pad[le] + a.seg_rows[le];
      const int r1 = a.offs_pad[le + 1];
      for (int r = r0 + pb * 8 + warp; r < r1; r += a.pad_blocks * 8) {
        int4* dst = reinterpret_cast<int4*>(a.peer_x[a.rank] + static_cast<size_t>(r) * a.H);
        for (int c = lane; c < nvec; c += 32) dst[c] = make_int4(0, 0, 0, 0);
        if (lane == 0 && a.peer_meta[a.rank] != nullptr) {
          int4 m = make_int4(a.rank, 0, 0, 0);
          *reinterpret_cast<int4*>(a.peer_meta[a.rank] + r) = m;
        }
      }
    }
  }
  // grid completion -> release flags to every owner
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(a.done_counter, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < a.world)
      st_release_sys_u32(a.peer_data_flags[threadIdx.x] + a.rank, static_cast<uint32_t>(a.epoch));
    if (threadIdx.x == 0) *a.done_counter = 0;
  }
}

// ------------------------------------------------------------------ place (quantising)
// Same placement, but each row is quantised in registers to MXFP8 (E4M3 + one E8M0 scale per 32
// elements) and what crosses NVLink is H bytes of values plus H/32 scale bytes, written straight
// into the owner's GEMM-ready buffers: values row-major, scales at their tensor-core atom offsets
// (four scale bytes per 4-byte store).  Padding rows of the owner's segments get zero values and
// unit scales so that they stay finite through the expert MLP.
struct PlaceMxArgs {
  PlaceArgs base;
  uint8_t* peer_xq[kMaxRanks];     // [capacity, H] e4m3
  uint8_t* peer_sf[kMaxRanks];     // atoms [capacity/128][H/128]
  int sf_cols_padded;
  int fp4;                 // 0: E4M3 bytes (row = H bytes); 1: E2M1 nibbles (row = H/2 bytes)
};

__global__ void __launch_bounds__(256) k_rdep_place_mx(const PlaceMxArgs am) {
  const PlaceArgs& a = am.base;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row_blocks = gridDim.x - a.pad_blocks;
  const int nblk = a.H >> 5;
  if (static_cast<int>(blockIdx.x) < row_blocks) {
    // One warp per TOKEN: its row is loaded and quantised once, then stored to each of its K destinations (lane k
    // works out slot k's destination; the others get it by shuffle).  K <= 32.
    const int row_bytes = am.fp4 ? (a.H >> 1) : a.H;
    for (int tok = blockIdx.x * 8 + warp; tok < a.T; tok += row_blocks * 8) {
      int my_pos = -1, my_owner = 0;
      if (lane < a.K) {
        const int i = tok * a.K + lane;
        const int e = a.eid[i];
        const int rb = a.rank_in_block[i];
        int lp = -1;
        if (e >= 0 && e < a.E && rb >= 0 && a.base[e] >= 0) {
          my_owner = e / a.n_local;
          const int within = a.block_prefix[(i / kCountThreads) * a.E + e] + rb;
          my_pos = a.base[e] + within;
          lp = a.send_prefix[e] + within;
        }
        a.pos_out[i] = my_pos;
        if (a.lpos_out) a.lpos_out[i] = lp;
      }
      const __nv_bfloat16* src = a.x + static_cast<size_t>(tok) * a.H;
      for (int b0 = 0; b0 < nblk; b0 += 32) {
        const int b = b0 + lane;
        uint32_t s = 127;
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (b < nblk) {
          float v[32];
          load_block_bf16(src + b * 32, v);
          s = am.fp4 ? quant_block_e2m1_regs(v, w) : quant_block_e4m3_regs(v, w);
        }
        const uint32_t packed = s | (__shfl_down_sync(0xffffffffu, s, 1) << 8) | (__shfl_down_sync(0xffffffffu, s, 2) << 16) |
                                (__shfl_down_sync(0xffffffffu, s, 3) << 24);
        for (int k = 0; k < a.K; ++k) {
          const int pos = __shfl_sync(0xffffffffu, my_pos, k);
          const int owner = __shfl_sync(0xffffffffu, my_owner, k);
          if (pos < 0 || b >= nblk) continue;
          uint8_t* qdst = am.peer_xq[owner] + static_cast<size_t>(pos) * row_bytes;
          if (am.fp4) {
            st_relaxed_sys_v4(qdst + b * 16, make_int4(w[0], w[1], w[2], w[3]));
          } else {
            st_relaxed_sys_v4(qdst + b * 32, make_int4(w[0], w[1], w[2], w[3]));
            st_relaxed_sys_v4(qdst + b * 32 + 16, make_int4(w[4], w[5], w[6], w[7]));
          }
          if ((lane & 3) == 0)
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(am.peer_sf[owner] + sf_mma_offset(pos, b, am.sf_cols_padded)),
                         "r"(packed) : "memory");
        }
      }
      if (lane < a.K && my_pos >= 0 && a.peer_meta[my_owner] != nullptr) {
        const int i = tok * a.K + lane;
        int4 m;
        m.x = a.rank; m.y = i; m.z = __float_as_int(a.gates ? a.gates[i] : 1.f); m.w = 1;
        st_relaxed_sys_v4(a.peer_meta[my_owner] + my_pos, m);
      }
    }
  } else {
    const int pb = blockIdx.x - row_blocks;
    for (int le = 0; le < a.n_local; ++le) {
      const int r0 = a.offs_pad[le] + a.seg_rows[le];
      const int r1 = a.offs_pad[le + 1];
      for (int r = r0 + pb * 8 + warp; r < r1; r += a.pad_blocks * 8) {
        const int row_bytes = am.fp4 ? (a.H >> 1) : a.H;
        int4* dst = reinterpret_cast<int4*>(am.peer_xq[a.rank] + static_cast<size_t>(r) * row_bytes);
        for (int c = lane; c < (row_bytes >> 4); c += 32) dst[c] = make_int4(0, 0, 0, 0);
        for (int b = lane * 4; b < nblk; b += 128)
          *reinterpret_cast<uint32_t*>(am.peer_sf[a.rank] + sf_mma_offset(r, b, am.sf_cols_padded)) = 0x7f7f7f7fu;
        if (lane == 0 && a.peer_meta[a.rank] != nullptr)
          *reinterpret_cast<int4*>(a.peer_meta[a.rank] + r) = make_int4(a.rank, 0, 0, 0);
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(a.done_counter, 1) == static_cast<int>(gridDim.x) - 1);
  __syncthreads();
  if (s_last) {
    __threadfence_system();
    if (threadIdx.x < a.world)
      st_release_sys_u32(a.peer_data_flags[threadIdx.x] + a.rank, static_cast<uint32_t>(a.epoch));
    if (threadIdx.x == 0) *a.done_counter = 0;
  }
}

// ------------------------------------------------------------------ flags
// Release `epoch` into entry `rank` of every peer's flag array (used after a kernel whose
// stores to peers must be visible, e.g. the return push of the last GEMM).
__global__ void k_rdep_signal(uint32_t* const* peer_flags, int rank, int world, uint32_t epoch) {
  __threadfence_system();
  if (threadIdx.x < world) st_release_sys_u32(peer_flags[threadIdx.x] + rank, epoch);
}
struct PeerFlagPtrs { uint32_t* p[kMaxRanks]; };
__global__ void k_rdep_signal_v(const PeerFlagPtrs f, int rank, int world, uint32_t epoch) {
  __threadfence_system();
  if (threadIdx.x < world) st_release_sys_u32(f.p[threadIdx.x] + rank, epoch);
}

// Bounded wait until my flags [world] all reached `epoch`.  budget_iters bounds the spin.
__global__ void k_rdep_wait(const uint32_t* my_flags, int world, uint32_t epoch, uint32_t budget_iters,
                            StatusRecord* status, int where) {
  if (threadIdx.x < world) {
    if (!wait_flag_ge_sys(my_flags + threadIdx.x, epoch, budget_iters))
      report_status(status, kStatusWaitTimeout, where, threadIdx.x, static_cast<int>(epoch));
  }
  __threadfence_system();
}

// ------------------------------------------------------------------ return / reduce
// Owner side, unfused variant: push rows of y[capacity, H] (scaled by the row's gate when
// use_gate) into the source's return buffer ret[tok_slot, H].
struct PushArgs {
  int H, n_rows_cap;
  const __nv_bfloat16* y;
  const int* runs;                  // [3][n_local][world]: run start in my buffer, run length, start in the source's buffer
  const int* tile_expert;           // local expert of every 128-row tile
  const int* n_m_tiles;
  __nv_bfloat16* peer_ret[kMaxRanks];
  float* peer_retg[kMaxRanks];      // optional per-row scalar return (gate gradients)
  const float* rowval;              // optional per-row scalar to return
  int world, n_local, n_pairs;      // n_pairs = rows of a source's return buffer (bound for every destination row)
  StatusRecord* status;
};

__global__ void __launch_bounds__(256) k_rdep_push(const PushArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows = min(*a.n_m_tiles * 128, a.n_rows_cap);
  const int nvec = a.H >> 3;
  // consecutive warps take consecutive rows: at any moment the grid writes a sliding window of consecutive
  // destination rows per source
  for (int r = blockIdx.x * 8 + warp; r < rows; r += gridDim.x * 8) {
    int src, ts;
    if (!run_lookup(a.runs, a.n_local, a.world, __ldg(a.tile_expert + (r >> 7)), r, src, ts)) continue;
    if (ts < 0 || ts >= a.n_pairs) {
      if (lane == 0) report_status(a.status, kStatusBadIndex, 430, r, ts);
      continue;
    }
    if (a.y != nullptr) {
      const int4* s = reinterpret_cast<const int4*>(a.y + static_cast<size_t>(r) * a.H);
      int4* d = reinterpret_cast<int4*>(a.peer_ret[src] + static_cast<size_t>(ts) * a.H);
      // eight loads in flight per lane (4 KB of the row per pass), then the remote stores back to back
      for (int c0 = 0; c0 < nvec; c0 += 256) {
        int4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = c0 + j * 32 + lane;
          if (c < nvec) v[j] = ld_nc_v4(s + c);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int c = c0 + j * 32 + lane;
          if (c < nvec) st_relaxed_sys_v4(d + c, v[j]);
        }
      }
    }
    if (lane == 0 && a.rowval != nullptr) a.peer_retg[src][ts] = a.rowval[r];
  }
  __threadfence_system();
}

// Owner side, copy-engine variant of k_rdep_push: every row chunk travels global -> shared -> peer global as two
// bulk asynchronous copies (the TMA unit moves the bytes; the warp only issues them), so one lane keeps kilobytes in
// flight per instruction instead of 16 bytes per store.  A warp owns a ring of kPushSlots shared-memory slots of
// kPushChunk bytes; rows longer than a slot go in chunks.  A destination row outside the source's return buffer
// (only possible with a corrupt run table) is skipped and reported, never written.
constexpr int kPushChunk = 4096;
constexpr int kPushSlots = 3;
constexpr int kPushWarps = 8;

NMOE_DEVICE void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
NMOE_DEVICE void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}

__global__ void __launch_bounds__(kPushWarps * 32) k_rdep_push_bulk(const PushArgs a) {
  extern __shared__ __align__(128) uint8_t push_smem[];
  __shared__ uint64_t bars[kPushWarps * kPushSlots];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* slots = push_smem + static_cast<size_t>(warp) * kPushSlots * kPushChunk;
  uint64_t* bar = bars + warp * kPushSlots;
  if (lane == 0) {
    for (int s = 0; s < kPushSlots; ++s) mbar_init(&bar[s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  const int rows = min(*a.n_m_tiles * 128, a.n_rows_cap);
  const int row_bytes = a.H * 2;
  const int chunks = (row_bytes + kPushChunk - 1) / kPushChunk;
  int slot = 0;
  uint32_t phase_bits = 0;       // bit s = parity of the next completion of slot s
  bool ok = true;
  for (int r = blockIdx.x * kPushWarps + warp; ok && r < rows; r += gridDim.x * kPushWarps) {
    int src, ts;
    if (!run_lookup(a.runs, a.n_local, a.world, __ldg(a.tile_expert + (r >> 7)), r, src, ts)) continue;
    if (ts < 0 || ts >= a.n_pairs) {
      if (lane == 0) report_status(a.status, kStatusBadIndex, 430, r, ts);
      continue;
    }
    if (a.y != nullptr) {
      const uint8_t* srow = reinterpret_cast<const uint8_t*>(a.y + static_cast<size_t>(r) * a.H);
      uint8_t* drow = reinterpret_cast<uint8_t*>(a.peer_ret[src] + static_cast<size_t>(ts) * a.H);
      for (int c = 0; c < chunks; ++c) {
        const int off = c * kPushChunk;
        const uint32_t nb = static_cast<uint32_t>(min(kPushChunk, row_bytes - off));
        uint8_t* sm = slots + slot * kPushChunk;
        if (lane == 0) {
          // the slot is free once the bulk store issued kPushSlots chunks ago has read it
          asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPushSlots - 1) : "memory");
          mbar_expect_tx(&bar[slot], nb);
          bulk_g2s(sm, srow + off, nb, &bar[slot]);
        }
        __syncwarp();
        if (!mbar_wait(&bar[slot], (phase_bits >> slot) & 1u)) {
          if (lane == 0) report_status(a.status, kStatusWaitTimeout, 431, r, c);
          ok = false;
          break;
        }
        phase_bits ^= 1u << slot;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          bulk_s2g(drow + off, sm, nb);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        if (++slot == kPushSlots) slot = 0;
      }
    }
    if (lane == 0 && a.rowval != nullptr) a.peer_retg[src][ts] = a.rowval[r];
  }
  if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all bytes written before the kernel ends
  __syncwarp();
  __threadfence_system();
}

// Source side: out[t] = sum_k gate[t,k] * ret[lpos[t*K + k]] over the slots that were delivered (lpos >= 0), fp32,
// fixed slot order (bit-reproducible).  gates == nullptr: plain sum (input-gradient return).
__global__ void __launch_bounds__(256)
k_rdep_reduce(const __nv_bfloat16* __restrict__ ret, const int* __restrict__ lpos, const float* __restrict__ gates,
              __nv_bfloat16* __restrict__ out, int T, int K, int H) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    // lane k holds slot k's row index and gate (K <= 32); handed out by shuffles below
    const int my_row = lane < K ? lpos[t * K + lane] : -1;
    const float my_gate = (lane < K && gates != nullptr) ? gates[t * K + lane] : 1.f;
    for (int c = lane; c < nvec; c += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k0 = 0; k0 < K; k0 += 8) {
        // up to eight independent loads in flight, then the sum in slot order
        int4 v[8];
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int k = k0 + j;
          const int row = __shfl_sync(0xffffffffu, my_row, k & 31);
          g[j] = __shfl_sync(0xffffffffu, my_gate, k & 31);
          v[j] = (k < K && row >= 0)
                     ? ld_relaxed_sys_v4(reinterpret_cast<const int4*>(ret + static_cast<size_t>(row) * H) + c)
                     : make_int4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 f0 = unpack_bf16x2(v[j].x), f1 = unpack_bf16x2(v[j].y), f2 = unpack_bf16x2(v[j].z), f3 = unpack_bf16x2(v[j].w);
          acc[0] = fmaf(g[j], f0.x, acc[0]); acc[1] = fmaf(g[j], f0.y, acc[1]);
          acc[2] = fmaf(g[j], f1.x, acc[2]); acc[3] = fmaf(g[j], f1.y, acc[3]);
          acc[4] = fmaf(g[j], f2.x, acc[4]); acc[5] = fmaf(g[j], f2.y, acc[5]);
          acc[6] = fmaf(g[j], f3.x, acc[6]); acc[7] = fmaf(g[j], f3.y, acc[7]);
        }
      }
      int4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<int4*>(out + static_cast<size_t>(t) * H)[c] = o;
    }
  }
}

// Source side: per-pair scalars returned by the owners (gate gradients) back into (token, slot) order.
__global__ void k_rdep_gather_scalar(const float* __restrict__ retg, const int* __restrict__ lpos, float* __restrict__ out,
                                     int n_pairs) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += gridDim.x * blockDim.x) {
    const int r = lpos[i];
    out[i] = r >= 0 ? retg[r] : 0.f;
  }
}

// Owner side helper: gather gate[pos] from meta into a dense fp32 vector (row scale for SwiGLU bwd).
__global__ void k_rdep_row_gates(const RdepMeta* __restrict__ meta, const int* __restrict__ n_m_tiles, int cap,
                                 float* __restrict__ out) {
  const int rows = min(*n_m_tiles * 128, cap);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x)
    out[r] = meta[r].valid ? meta[r].gate : 0.f;
}

__global__ void k_rdep_clamp_tiles(int* n_m_tiles, int limit_tiles, int* seen) {
  const int n = *n_m_tiles;
  if (seen != nullptr) *reinterpret_cast<volatile int*>(seen) = n;
  if (n > limit_tiles) *n_m_tiles = limit_tiles;
}

}  // namespace nmoe

using namespace nmoe;

#define CHECK_LAUNCH() do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return static_cast<int>(e_); } while (0)

extern "C" {

int nmoe_rdep_count_blocks(int n_pairs) { return (n_pairs + kCountThreads - 1) / kCountThreads; }

int nmoe_rdep_count(const int* eid, int n_pairs, int E, int* block_hist, int* rank_in_block, void* status,
                    cudaStream_t st) {
  if (E > kMaxExperts) return -1;
  const int nb = nmoe_rdep_count_blocks(n_pairs);
  if (nb == 0) return 0;
  const size_t smem = 32 * static_cast<size_t>(E) * sizeof(int);
  cudaFuncSetAttribute(k_rdep_count, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  k_rdep_count<<<nb, kCountThreads, smem, st>>>(eid, n_pairs, E, block_hist, rank_in_block,
                                               static_cast<StatusRecord*>(status));
  CHECK_LAUNCH();
  return 0;
}

// peer_counts / peer_count_flags: arrays of `world` device pointers (host memory).
int nmoe_rdep_plan(int rank, int world, int E, int n_local, int n_blocks, int capacity_rows, int epoch, int align,
                   int* block_hist, void* const* peer_counts, void* const* peer_count_flags, int* base,
                   int* offs_pad, int* seg_rows, int* tile_expert, int* n_m_tiles, int* send_counts, int* send_prefix,
                   int* runs, void* status, cudaStream_t st) {
  if (world > kMaxRanks || E > kMaxExperts || E != n_local * world) return -1;
  if (align != 128 && align != 256) return -2;
  PlanArgs a;
  a.align = align;
  a.rank = rank; a.world = world; a.E = E; a.n_local = n_local; a.n_blocks = n_blocks;
  a.capacity_rows = capacity_rows; a.epoch = epoch; a.block_hist = block_hist;
  for (int r = 0; r < world; ++r) {
    a.peer_counts[r] = static_cast<int*>(peer_counts[r]);
    a.peer_count_flags[r] = static_cast<uint32_t*>(peer_count_flags[r]);
  }
  a.my_counts_table = a.peer_counts[rank];
  a.my_count_flags = a.peer_count_flags[rank];
  a.base = base; a.offs_pad = offs_pad; a.seg_rows = seg_rows; a.tile_expert = tile_expert;
  a.n_m_tiles = n_m_tiles; a.send_counts = send_counts; a.send_prefix = send_prefix; a.runs = runs;
  a.status = static_cast<StatusRecord*>(status);
  k_rdep_plan<<<1, 512, 0, st>>>(a);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_rdep_place(int rank, int world, int E, int n_local, int T, int K, int H, int epoch, const void* x,
                    const int* eid, const float* gates, const int* rank_in_block, const int* block_prefix,
                    const int* base, void* const* peer_x, void* const* peer_meta, void* const* peer_data_flags,
                    int* pos_out, int* owner_out, const int* offs_pad, const int* seg_rows, int* done_counter,
                    void* status, const int* send_prefix, int* lpos_out, cudaStream_t st) {
  if (world > kMaxRanks || (H % 8) != 0) return -1;
  PlaceArgs a;
  a.send_prefix = send_prefix; a.lpos_out = lpos_out;
  a.rank = rank; a.world = world; a.E = E; a.n_local = n_local; a.T = T; a.K = K; a.H = H; a.epoch = epoch;
  a.x = static_cast<const __nv_bfloat16*>(x); a.eid = eid; a.gates = gates; a.rank_in_block = rank_in_block;
  a.block_prefix = block_prefix; a.base = base;
  for (int r = 0; r < world; ++r) {
    a.peer_x[r] = static_cast<__nv_bfloat16*>(peer_x[r]);
    a.peer_meta[r] = peer_meta ? static_cast<RdepMeta*>(peer_meta[r]) : nullptr;
    a.peer_data_flags[r] = static_cast<uint32_t*>(peer_data_flags[r]);
  }
  a.pos_out = pos_out; a.owner_out = owner_out; a.offs_pad = offs_pad; a.seg_rows = seg_rows;
  a.done_counter = done_counter; a.pad_blocks = 16; a.status = static_cast<StatusRecord*>(status);
  if (K > 32) return -1;
  int row_blocks = (T + 7) / 8;              // one warp per token
  if (row_blocks > 148 * 8) row_blocks = 148 * 8;
  if (row_blocks < 1) row_blocks = 1;
  k_rdep_place<<<row_blocks + a.pad_blocks, 256, 0, st>>>(a);
  CHECK_LAUNCH();
  return 0;
}

// Quantising placement: x rows -> owner's e4m3 (fp4 = 0) or e2m1 (fp4 = 1) buffer peer_xq + scale atoms peer_sf.
int nmoe_rdep_place_mx(int rank, int world, int E, int n_local, int T, int K, int H, int epoch, const void* x,
                       const int* eid, const float* gates, const int* rank_in_block, const int* block_prefix,
                       const int* base, void* const* peer_xq, void* const* peer_sf, void* const* peer_meta,
                       void* const* peer_data_flags, int* pos_out, const int* offs_pad, const int* seg_rows,
                       int* done_counter, void* status, int fp4, const int* send_prefix, int* lpos_out,
                       cudaStream_t st) {
  // 32-element blocks, 16-byte row stores; the scale bytes of a partial last atom are written as padding (127)
  if (world > kMaxRanks || (H % 32) != 0 || (fp4 && (H % 64) != 0)) return -1;
  PlaceMxArgs am;
  am.fp4 = fp4;
  PlaceArgs& a = am.base;
  a.send_prefix = send_prefix; a.lpos_out = lpos_out;
  a.rank = rank; a.world = world; a.E = E; a.n_local = n_local; a.T = T; a.K = K; a.H = H; a.epoch = epoch;
  a.x = static_cast<const __nv_bfloat16*>(x); a.eid = eid; a.gates = gates; a.rank_in_block = rank_in_block;
  a.block_prefix = block_prefix; a.base = base;
  for (int r = 0; r < world; ++r) {
    a.peer_x[r] = nullptr;
    am.peer_xq[r] = static_cast<uint8_t*>(peer_xq[r]);
    am.peer_sf[r] = static_cast<uint8_t*>(peer_sf[r]);
    a.peer_meta[r] = peer_meta ? static_cast<RdepMeta*>(peer_meta[r]) : nullptr;
    a.peer_data_flags[r] = static_cast<uint32_t*>(peer_data_flags[r]);
  }
  am.sf_cols_padded = ((H / 32) + 3) & ~3;
  a.pos_out = pos_out; a.owner_out = nullptr; a.offs_pad = offs_pad; a.seg_rows = seg_rows;
  a.done_counter = done_counter; a.pad_blocks = 16; a.status = static_cast<StatusRecord*>(status);
  const int n_pairs = T * K;
  int row_blocks = (n_pairs + 7) / 8;
  if (row_blocks > 148 * 8) row_blocks = 148 * 8;
  if (row_blocks < 1) row_blocks = 1;
  k_rdep_place_mx<<<row_blocks + a.pad_blocks, 256, 0, st>>>(am);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_rdep_signal(void* const* peer_flags, int rank, int world, unsigned epoch, cudaStream_t st) {
  if (world > kMaxRanks) return -1;
  PeerFlagPtrs f;
  for (int r = 0; r < world; ++r) f.p[r] = static_cast<uint32_t*>(peer_flags[r]);
  k_rdep_signal_v<<<1, 32, 0, st>>>(f, rank, world, epoch);
  CHECK_LAUNCH();
  return 0;
}

// budget_iters == 0 selects the default (seconds).  Tests pass a small budget to exercise the timeout path.
int nmoe_rdep_wait(const void* my_flags, int world, unsigned epoch, unsigned budget_iters, void* status, int where,
                   cudaStream_t st) {
  if (world > kMaxRanks) return -1;
  k_rdep_wait<<<1, 32, 0, st>>>(static_cast<const uint32_t*>(my_flags), world, epoch,
                                budget_iters ? budget_iters : kFlagSpinBudget, static_cast<StatusRecord*>(status), where);
  CHECK_LAUNCH();
  return 0;
}

// Owner -> sources return of y[capacity, H] in runs (see the header comment).  impl 0: per-lane 16-byte system-scope
// stores; impl 1: bulk asynchronous copies through shared memory.  runs / tile_expert come from nmoe_rdep_plan;
// n_pairs = T*K of the SOURCE ranks (rows of a return buffer).  y == nullptr sends only the per-row scalars.
int nmoe_rdep_push(const void* y, const int* runs, const int* tile_expert, const int* n_m_tiles, int cap_rows, int H,
                   void* const* peer_ret, void* const* peer_retg, const float* rowval, int world, int n_local,
                   int n_pairs, void* status, int impl, cudaStream_t st) {
  if (world > kMaxRanks || (H % 8) != 0) return -1;
  PushArgs a;
  a.world = world; a.n_local = n_local; a.n_pairs = n_pairs; a.status = static_cast<StatusRecord*>(status);
  a.H = H; a.n_rows_cap = cap_rows;
  a.y = static_cast<const __nv_bfloat16*>(y); a.runs = runs; a.tile_expert = tile_expert; a.n_m_tiles = n_m_tiles;
  for (int r = 0; r < kMaxRanks; ++r) {
    a.peer_ret[r] = (peer_ret && r < world) ? static_cast<__nv_bfloat16*>(peer_ret[r]) : nullptr;
    a.peer_retg[r] = (peer_retg && r < world) ? static_cast<float*>(peer_retg[r]) : nullptr;
  }
  a.rowval = rowval;
  if (impl == 1) {
    const int smem = kPushWarps * kPushSlots * kPushChunk;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(k_rdep_push_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      configured = true;
    }
    k_rdep_push_bulk<<<148 * 2, kPushWarps * 32, smem, st>>>(a);
  } else {
    k_rdep_push<<<148 * 8, 256, 0, st>>>(a);
  }
  CHECK_LAUNCH();
  return 0;
}

// out[t] = sum_k gates[t,k] * ret[lpos[t,k]]  (gates may be null: plain sum)
int nmoe_rdep_reduce(const void* ret, const int* lpos, const float* gates, void* out, int T, int K, int H,
                     cudaStream_t st) {
  if (T == 0) return 0;
  if ((H % 8) != 0 || K > 32) return -1;
  int blocks = (T + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  k_rdep_reduce<<<blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(ret), lpos, gates,
                                       static_cast<__nv_bfloat16*>(out), T, K, H);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_rdep_gather_scalar(const float* retg, const int* lpos, float* out, int n_pairs, cudaStream_t st) {
  if (n_pairs == 0) return 0;
  k_rdep_gather_scalar<<<(n_pairs + 255) / 256 < 1184 ? (n_pairs + 255) / 256 : 1184, 256, 0, st>>>(retg, lpos, out, n_pairs);
  CHECK_LAUNCH();
  return 0;
}

// Rows that landed on this rank against the rows the layer's tensors were sized for (see Rdep.rows_of): the count
// goes to `seen` (pinned host memory the host looks at later, without waiting) and n_m_tiles is cut to the limit, so
// that every consumer -- they all read n_m_tiles on the device -- stays inside its tensors.  Rows beyond the limit are
// not computed; the host notices from `seen` one step late, says so and enlarges the limit.
int nmoe_rdep_clamp_tiles(int* n_m_tiles, int limit_tiles, int* seen, cudaStream_t st) {
  k_rdep_clamp_tiles<<<1, 1, 0, st>>>(n_m_tiles, limit_tiles, seen);
  CHECK_LAUNCH();
  return 0;
}

int nmoe_rdep_row_gates(const void* meta, const int* n_m_tiles, int cap, float* out, cudaStream_t st) {
  k_rdep_row_gates<<<148, 256, 0, st>>>(static_cast<const RdepMeta*>(meta), n_m_tiles, cap, out);
  CHECK_LAUNCH();
  return 0;
}

// ---- peer memory (CUDA IPC).  Buffers come from cudaMalloc so that their handles can be exported.
int nmoe_peer_alloc(size_t bytes, void** out) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(*out, 0, bytes);
  return static_cast<int>(e);
}
int nmoe_peer_free(void* p) { return static_cast<int>(cudaFree(p)); }
int nmoe_peer_get_handle(void* p, void* handle64) {
  return static_cast<int>(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p));
}
int nmoe_peer_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h = *static_cast<const cudaIpcMemHandle_t*>(handle64);
  return static_cast<int>(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
int nmoe_peer_close(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }

}  // extern "C"
