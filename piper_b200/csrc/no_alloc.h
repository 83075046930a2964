// RMSNorm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for
// embedders of this library that run where cudaMalloc (and therefore every
// allocating library routine, PyTorch's caching allocator included) is off
// limits: hosts that hand a plugin a fixed memory budget up front and forbid
// later allocations, and real-time loops that must not take the allocator's
// locks or risk its implicit device synchronisation.  The normal entry point (piper::rmsnorm_bwd) needs a
// caller-provided scratch buffer for its per-strip partial sums of the weight
// gradient; here that scratch is a fixed array inside the library image.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest feature dimension the built-in scratch array is sized for.  The
// array holds PIPER_NOALLOC_MAX_STRIPS * PIPER_NOALLOC_MAX_D floats (about
// 9.25 MiB); every GPU that loads the library reserves that much until the
// process exits.  The strip count is the fixed bound of the regular entry
// point (two strips per SM of a 148-SM part, independent of the device), so
// it never exceeds PIPER_NOALLOC_MAX_STRIPS.
#define PIPER_NOALLOC_MAX_D 8192
#define PIPER_NOALLOC_MAX_STRIPS 296

// dx[T, D] (bf16) = gradient of y = rmsnorm(x) * w with respect to x, and
// dw[D] (fp32) = gradient with respect to w (added to the existing contents
// when accumulate != 0, overwritten otherwise).  dy, x: bf16 [T, D]; w: bf16
// [D]; rstd: fp32 [T] as saved by the forward pass.  All pointers are device
// pointers supplied by the caller; the work is enqueued on `stream`.
//
// Returns 0 on success.  Returns -1 without launching anything when D is not
// a multiple of 8, D exceeds PIPER_NOALLOC_MAX_D, or T is negative or larger
// than INT_MAX (rows are indexed with 32-bit ints); -2 when
// the one-time set-up failed; -3 when a launch failed.
// piper_noalloc_last_error() then describes the problem.
//
// The call allocates nothing and frees nothing.  Its first use on a device
// looks up the device address of the scratch array (one cudaGetSymbolAddress
// call, with that device current); make that first call outside of any
// stream capture.  All calls on a device share the one scratch array, so two
// calls whose kernels can overlap on the GPU (different streams without an
// ordering between them) race on it: serialise them.  The array keeps
// whatever the previous call left; that is harmless because every strip
// rewrites its full row before the reduction reads it.
int piper_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                              float* dw, int accumulate, long long T, int D, cudaStream_t stream);

// Text of the most recent error reported by the call above on this thread
// ("" if none).
const char* piper_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
