// Inter-node leg of RDEP over NVSHMEM (built as its own library, libnmoe_hybrid.so, only where NVSHMEM is present:
// the device code needs relocatable device code and the NVSHMEM device library; the main library needs neither).
//
// Inside a node every GPU reaches every other through peer-mapped memory (csrc/rdep.cu).  Across nodes a row bound
// for an expert on node n is put into the staging buffer of the PROXY on that node -- the GPU with the sender's own
// local index -- which then feeds it to the intra-node placement like one of its own rows.  One proxy per (sender,
// node) keeps the number of network endpoints per GPU at nodes-1 instead of world-1.
//
//   k_hybrid_put_rows   sender: one warp per remote row, nvshmemx_putmem_nbi_warp of the row and of its 16-byte
//                       record {origin PE, origin pair index, gate, global expert} into its own slice of the proxy's
//                       staging area (slices are per origin PE, positions are the sender's running count per node:
//                       no remote atomics), then fence + one signal per proxy carrying epoch and row count
//   k_hybrid_wait       proxy: bounded wait until every origin PE's signal shows this epoch; on expiry a status
//                       record is written and the kernel returns (never an endless spin, never a trap)
//   k_hybrid_return     owner side, reverse direction: output rows (gate applied) are put straight into the origin
//                       PE's (token, slot) return buffer, which is symmetric memory as well
//
// Host entry points cover bootstrap by unique id (rank 0 creates it, the caller broadcasts it), symmetric allocation,
// quiet / barrier on a stream and teardown.
//
// Reference counterpart: nmoe/csrc/rdep_nvshmem.cu:233-812 (dispatch), :1442-1604 (return), :2412-2505 (bootstrap) and
// the bindings nmoe/csrc/bindings.cpp:929-995.  Not timed on a single node.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <nvshmem.h>
#include <nvshmemx.h>

#include "../common/status.h"

namespace nmoe {

struct HybridRecord {      // travels with every row
  int32_t origin_pe;
  int32_t origin_pair;     // token * K + slot on the origin
  float gate;
  int32_t expert;          // global expert id
};

__device__ __forceinline__ void hybrid_report(StatusRecord* st, int code, int where, int a, int b) {
  if (st != nullptr && atomicCAS(&st->code, 0, code) == 0) { st->where = where; st->a = a; st->b = b; }
}

// rows: [n_rows, H] bf16 local; dst_node[r] = destination node of row r (or -1: stays inside this node);
// slot[r] = position inside this PE's slice of the proxy's staging area (running count per node, made by the caller's
// routing plan); staging / records: symmetric; layout [origin PE][slice_rows][H] and [origin PE][slice_rows].
__global__ void __launch_bounds__(256)
k_hybrid_put_rows(const __nv_bfloat16* __restrict__ rows, const HybridRecord* __restrict__ recs,
                  const int* __restrict__ dst_node, const int* __restrict__ slot, int n_rows, int H, int slice_rows,
                  int my_pe, int local_world, __nv_bfloat16* staging, HybridRecord* records) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  const int my_local = my_pe % local_world;
  for (int r = warp; r < n_rows; r += n_warps) {
    const int node = dst_node[r];
    if (node < 0) continue;
    const int s = slot[r];
    if (s < 0 || s >= slice_rows) continue;                       // over the slice: dropped by the plan, never written
    const int proxy = node * local_world + my_local;
    const size_t at = static_cast<size_t>(my_pe) * slice_rows + s;
    nvshmemx_putmem_nbi_warp(staging + at * H, rows + static_cast<size_t>(r) * H, static_cast<size_t>(H) * 2, proxy);
    nvshmemx_putmem_nbi_warp(records + at, recs + r, sizeof(HybridRecord), proxy);
  }
}

// After the puts: order them before the signals, then tell every proxy how many rows came from this PE.
// counts[node] = rows sent to that node; signals: symmetric uint64 [world]; value = epoch << 32 | count.
__global__ void k_hybrid_signal(const int* __restrict__ counts, int n_nodes, int my_node, int my_pe, int local_world,
                                uint64_t epoch, uint64_t* signals) {
  nvshmem_fence();
  const int node = threadIdx.x;
  if (node < n_nodes && node != my_node) {
    const int proxy = node * local_world + (my_pe % local_world);
    nvshmemx_signal_op(signals + my_pe, (epoch << 32) | static_cast<uint32_t>(counts[node]), NVSHMEM_SIGNAL_SET, proxy);
  }
}

// Proxy: wait until the signal of every origin PE on other nodes (same local index) carries this epoch.
// counts_out[origin node] = rows that arrived from there.  Bounded: `budget` polls, then a status record.
__global__ void k_hybrid_wait(uint64_t* signals, int n_nodes, int my_node, int my_pe, int local_world, uint64_t epoch,
                              unsigned budget, int* counts_out, StatusRecord* status) {
  const int node = threadIdx.x;
  if (node >= n_nodes) return;
  if (node == my_node) { counts_out[node] = 0; return; }
  const int origin = node * local_world + (my_pe % local_world);
  uint64_t v = 0;
  bool seen = false;
  for (unsigned i = 0; i < budget; ++i) {
    v = nvshmem_signal_fetch(signals + origin);
    if ((v >> 32) >= epoch) { seen = true; break; }
    __nanosleep(128);
  }
  if (!seen) {
    hybrid_report(status, kStatusWaitTimeout, 900, origin, static_cast<int>(epoch));
    counts_out[node] = 0;
    return;
  }
  counts_out[node] = static_cast<int>(v & 0xffffffffu);
}

// Return leg: y rows (already gate-scaled) go to the origin PE's return buffer ret[origin_pair, H] (symmetric).
__global__ void __launch_bounds__(256)
k_hybrid_return(const __nv_bfloat16* __restrict__ y, const HybridRecord* __restrict__ recs, int n_rows, int H,
                int my_node, int local_world, int n_pairs, __nv_bfloat16* ret, StatusRecord* status) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int n_warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = warp; r < n_rows; r += n_warps) {
    const HybridRecord rec = recs[r];
    if (rec.origin_pe / local_world == my_node) continue;         // intra-node rows go back over peer memory
    if (rec.origin_pair < 0 || rec.origin_pair >= n_pairs) {
      if ((threadIdx.x & 31) == 0) hybrid_report(status, kStatusBadIndex, 901, r, rec.origin_pair);
      continue;
    }
    nvshmemx_putmem_nbi_warp(ret + static_cast<size_t>(rec.origin_pair) * H, y + static_cast<size_t>(r) * H,
                             static_cast<size_t>(H) * 2, rec.origin_pe);
  }
}

}  // namespace nmoe

using namespace nmoe;

namespace {
bool g_initialised = false;
#define HCHECK() do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return static_cast<int>(e_); } while (0)
}  // namespace

extern "C" {

int nmoe_hybrid_available() { return 1; }
int nmoe_hybrid_uid_bytes() { return static_cast<int>(sizeof(nvshmemx_uniqueid_t)); }

// rank 0 creates the id; the caller broadcasts the bytes to every rank (torch.distributed on the CPU group)
int nmoe_hybrid_get_uid(void* uid_out, size_t bytes) {
  if (uid_out == nullptr || bytes < sizeof(nvshmemx_uniqueid_t)) return -1;
  nvshmemx_uniqueid_t id = NVSHMEMX_UNIQUEID_INITIALIZER;
  const int rc = nvshmemx_get_uniqueid(&id);
  if (rc != 0) return rc;
  memcpy(uid_out, &id, sizeof(id));
  return 0;
}

int nmoe_hybrid_init(const void* uid, int rank, int world, int /*local_world*/) {
  if (g_initialised) return 0;
  if (uid == nullptr) return -1;
  nvshmemx_uniqueid_t id;
  memcpy(&id, uid, sizeof(id));
  nvshmemx_init_attr_t attr = NVSHMEMX_INIT_ATTR_INITIALIZER;
  int rc = nvshmemx_set_attr_uniqueid_args(rank, world, &id, &attr);
  if (rc != 0) return rc;
  rc = nvshmemx_init_attr(NVSHMEMX_INIT_WITH_UNIQUEID, &attr);
  if (rc != 0) return rc;
  g_initialised = true;
  return 0;
}

int nmoe_hybrid_alloc(size_t bytes, void** ptr_out) {
  if (!g_initialised || ptr_out == nullptr) return -1;
  *ptr_out = nvshmem_malloc(bytes);
  return *ptr_out != nullptr ? 0 : -2;
}
int nmoe_hybrid_free(void* ptr) {
  if (!g_initialised) return -1;
  nvshmem_free(ptr);
  return 0;
}
int nmoe_hybrid_quiet(void* stream) {
  if (!g_initialised) return -1;
  nvshmemx_quiet_on_stream(static_cast<cudaStream_t>(stream));
  return 0;
}
int nmoe_hybrid_barrier(void* stream) {
  if (!g_initialised) return -1;
  nvshmemx_barrier_all_on_stream(static_cast<cudaStream_t>(stream));
  return 0;
}
int nmoe_hybrid_finalize() {
  if (g_initialised) { nvshmem_finalize(); g_initialised = false; }
  return 0;
}

// Sender: put remote rows and their records to the proxies, then signal.  counts: device int[n_nodes].
int nmoe_hybrid_dispatch(const void* rows, const void* recs, const int* dst_node, const int* slot, const int* counts,
                         int n_rows, int H, int slice_rows, int my_pe, int world, int local_world, unsigned long long epoch,
                         void* staging, void* records, void* signals, void* stream) {
  if (!g_initialised || world % local_world != 0 || (H % 8) != 0) return -1;
  const int n_nodes = world / local_world;
  if (n_nodes > 1024) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n_rows > 0) {
    k_hybrid_put_rows<<<148 * 2, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(rows),
        static_cast<const HybridRecord*>(recs), dst_node, slot, n_rows, H, slice_rows, my_pe, local_world,
        static_cast<__nv_bfloat16*>(staging), static_cast<HybridRecord*>(records));
    HCHECK();
  }
  k_hybrid_signal<<<1, 1024, 0, st>>>(counts, n_nodes, my_pe / local_world, my_pe, local_world, epoch,
                                      static_cast<uint64_t*>(signals));
  HCHECK();
  return 0;
}

// Proxy: bounded wait for every origin's signal of this epoch; counts_out: device int[n_nodes].
int nmoe_hybrid_wait(void* signals, int my_pe, int world, int local_world, unsigned long long epoch, unsigned budget,
                     int* counts_out, void* status, void* stream) {
  if (!g_initialised || world % local_world != 0) return -1;
  const int n_nodes = world / local_world;
  if (n_nodes > 1024) return -1;
  k_hybrid_wait<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint64_t*>(signals), n_nodes,
      my_pe / local_world, my_pe, local_world, epoch, budget ? budget : 4000000u, counts_out,
      static_cast<StatusRecord*>(status));
  HCHECK();
  return 0;
}

// Owner: rows that came from other nodes go back to their origin's return buffer.
int nmoe_hybrid_return(const void* y, const void* recs, int n_rows, int H, int my_pe, int local_world, int n_pairs,
                       void* ret, void* status, void* stream) {
  if (!g_initialised || (H % 8) != 0) return -1;
  if (n_rows == 0) return 0;
  k_hybrid_return<<<148 * 2, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(y),
      static_cast<const HybridRecord*>(recs), n_rows, H, my_pe / local_world, local_world, n_pairs,
      static_cast<__nv_bfloat16*>(ret), static_cast<StatusRecord*>(status));
  HCHECK();
  return 0;
}

}  // extern "C"
