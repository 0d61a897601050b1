// Multi-node (hybrid) expert-parallel transport: entry points with the shape of the NVSHMEM-backed
// path (uid bootstrap, symmetric-heap allocation, quiet/barrier on a stream) so that callers and
// bindings do not change when a build with NVSHMEM is linked in.  This build has no NVSHMEM: every
// entry point reports kHybridUnavailable and touches nothing.  The routing rule the device code of
// such a build has to follow (inter-node traffic goes to the peer with the same local index on the
// destination node, which forwards inside its node over peer memory) is modelled on the host in
// nmoe_b200/parallel/hybrid.py and tested there.
//
// Reference counterpart: nmoe/csrc/rdep_nvshmem.cu/.cuh and the nvshmem_* bindings
// (nmoe/csrc/bindings.cpp:553-700).
#include <stddef.h>
#include <string.h>

namespace {
constexpr int kHybridUnavailable = -100;
}

extern "C" {

int nmoe_hybrid_available() { return 0; }

// 128-byte unique id that rank 0 creates and broadcasts out of band
int nmoe_hybrid_get_uid(void* uid_out, size_t bytes) {
  if (uid_out != nullptr && bytes > 0) memset(uid_out, 0, bytes);
  return kHybridUnavailable;
}

int nmoe_hybrid_init(const void* /*uid*/, int /*rank*/, int /*world*/, int /*local_world*/) { return kHybridUnavailable; }

int nmoe_hybrid_alloc(size_t /*bytes*/, void** ptr_out) {
  if (ptr_out != nullptr) *ptr_out = nullptr;
  return kHybridUnavailable;
}

int nmoe_hybrid_free(void* /*ptr*/) { return kHybridUnavailable; }

int nmoe_hybrid_quiet(void* /*stream*/) { return kHybridUnavailable; }

int nmoe_hybrid_barrier(void* /*stream*/) { return kHybridUnavailable; }

int nmoe_hybrid_finalize() { return kHybridUnavailable; }

}  // extern "C"
