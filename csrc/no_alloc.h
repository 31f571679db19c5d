// RMSNorm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference project; it exists for
// users of this library who run inside someone else's memory budget: a plug-in
// in a serving process whose allocator is owned by the host framework, a
// callback that runs while a memory pool is frozen, or a sandbox where
// cudaMalloc is simply not permitted.  The regular entry point
// (rb_rmsnorm_bwd, api.h) asks such a caller for a scratch buffer it has no way
// to obtain.  This variant brings its own: the per-block partial sums of the
// weight gradient live in one file-scope __device__ array inside the library,
// so the caller passes inputs and outputs only.
//
// What you pay and what you must respect:
//  * Every GPU that loads the library holds the array (about 9.3 MiB) until the
//    process exits.
//  * Capacity is fixed: cols <= RB_NOALLOC_RMSNORM_MAX_COLS and
//    rb_rmsnorm_bwd_parts(rows, cols) * cols <= RB_NOALLOC_RMSNORM_SCRATCH_FLOATS.
//    Larger problems are refused with RB_ERR_NOALLOC_TOO_LARGE (a message goes
//    to stderr); nothing is launched.
//  * The first call on each device looks up the array's device address, with
//    that device current.  Make that first call outside any stream capture.
//    The looked-up address is cached in a per-device table that is filled
//    without a lock: two host threads that race on the first use of a device
//    both look the address up and both store the same value, so the race is
//    benign (the address of a __device__ array never changes while the module
//    is loaded).
//  * All calls on a device share the one array and it keeps whatever the last
//    call left in it.  The kernels overwrite every element they later read, so
//    nothing has to be cleared between calls, but two calls whose kernels
//    overlap on the GPU (different streams, no ordering) race on it.  Order
//    them yourself.
//  * No cudaMalloc, cudaFree or any allocating library routine is called.
#pragma once
#include <cuda_runtime.h>

#define RB_NOALLOC_RMSNORM_MAX_COLS 8192
#define RB_NOALLOC_RMSNORM_SCRATCH_FLOATS (296 * 8192)
#define RB_ERR_NOALLOC_TOO_LARGE (-20)
#define RB_ERR_NOALLOC_SETUP (-21)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and results as rb_rmsnorm_bwd without the scratch pointer:
// x, dy, dx are [rows][cols], w and dw are [cols]; dtype 0 = bf16, 1 = fp16, 2 = fp32.
// Returns 0, a cudaError_t value, or one of the RB_ERR_NOALLOC_* codes.
int rb_rmsnorm_bwd_static(const void* x, const void* w, const void* dy, void* dx, void* dw, int rows, int cols, float eps,
                          int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
