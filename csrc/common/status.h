// Error reporting shared by every kernel in this library.
//
// Kernels never trap, assert or spin without a bound.  A kernel that gives up
// (a wait that ran out, an index that failed a bounds check) records one
// StatusRecord in a device-visible slot and returns; the host reads the slot
// after the stream has drained and raises a Python exception.  The context
// stays usable.
#pragma once
#include <stdint.h>

namespace nmoe {

enum StatusCode : int32_t {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,     // a bounded spin (mbarrier / flag / peer phase) ran out
  kStatusBadIndex = 2,        // an index failed a bounds check; the access was skipped
  kStatusCapacity = 3,        // a receive buffer would overflow; rows were dropped
  kStatusBadArgument = 4,
};

struct StatusRecord {
  int32_t code;       // StatusCode; first failure wins (atomicCAS from 0)
  int32_t where;      // kernel-specific site id
  int32_t a;          // site-specific detail (e.g. peer rank, stage)
  int32_t b;          // site-specific detail (e.g. phase, index)
};

}  // namespace nmoe
