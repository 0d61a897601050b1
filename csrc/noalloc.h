// Entry points that never allocate.  (No counterpart in the reference code base.)
//
// Some hosts of this library must not allocate device memory once they are running: an
// inference server that has handed every free byte to its KV-cache pool, a process that
// replays captured work and therefore may not grow an allocator mid-run, or an embedding in
// another runtime that owns the allocator and forbids foreign cudaMalloc calls.  For such
// callers the function below runs the RMSNorm backward exactly like nmoe_rmsnorm_bwd, but
// takes its fp32 partial-sum scratch from a fixed array that lives inside the library
// image instead of from a caller-provided (freshly allocated) buffer.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch covers: the backward uses at most
// NMOE_NOALLOC_RMSNORM_MAX_BLOCKS partial rows of H floats, so H may not exceed
// NMOE_NOALLOC_RMSNORM_MAX_H.  The array is 592 * 4096 * 4 bytes = 9.25 MiB and every GPU
// that loads the library keeps it resident until the process exits.
#define NMOE_NOALLOC_RMSNORM_MAX_BLOCKS 592
#define NMOE_NOALLOC_RMSNORM_MAX_H 4096

// dx[M,H], dw[H] from dy[M,H], x[M,H], w[H] (bf16) and rstd[M] (fp32), all caller-owned.
// Returns 0 on success, -1 for an unsupported H (not a multiple of 8, or larger than
// NMOE_NOALLOC_RMSNORM_MAX_H), -3 if the device ordinal is beyond the per-device table, or a
// positive cudaError_t.  It calls no cudaMalloc/cudaFree and no allocating library routine.
//
// The first call on each device resolves the device address of the built-in scratch (one
// cudaGetSymbolAddress with that device current); make that first call outside of any
// stream capture.  Make it at start-up, before the process commits the rest of the device's
// memory: with lazy module loading, that first symbol lookup or kernel launch can be what
// loads this library's device image, built-in array included, and on a device with no
// memory left it fails.  After one successful call per device, no later call can need memory.
// Host threads may race on the first call; the address cache is atomic.
//
// All calls on a device share the one scratch array, so two calls whose
// kernels may overlap on the GPU (different streams without an ordering between them) race
// on it; issue them on one stream or order them yourself.  Nothing in the scratch needs to
// be cleared between calls: each call overwrites every partial row it later reads.
int nmoe_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                             int M, int H, int accumulate, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
