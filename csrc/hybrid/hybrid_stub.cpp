// Stand-ins, inside the main library, for the entry points of the NVSHMEM-backed inter-node transport.  The real ones
// live in csrc/hybrid/rdep_nvshmem.cu and are built into their own library (libnmoe_hybrid.so) wherever an NVSHMEM
// installation is found; when that library is not loaded, callers resolve these symbols instead and every one of them
// reports kHybridUnavailable and touches nothing.
//
// Reference counterpart: nmoe/csrc/rdep_nvshmem.cu/.cuh and the nvshmem_* bindings (nmoe/csrc/bindings.cpp:929-995).
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
