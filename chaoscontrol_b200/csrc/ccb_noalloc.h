// Allocation-free entry point of libccb200.
//
// This header has no counterpart in the reference project: it exists for hosts
// that link libccb200 directly (a C or C++ serving harness, a plug-in inside
// another runtime) and are not allowed to call cudaMalloc -- typically because
// device memory was carved up once at start-up and every later allocation is
// either forbidden by policy or would fail.  Such a caller still owns the
// input and output buffers; what it cannot provide is the temporary workspace
// the regular launcher expects from its caller.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in workspace covers.
#define CCB_NOALLOC_RMSNORM_MAX_ROWS 65536
#define CCB_NOALLOC_RMSNORM_MAX_DIM 1024

// RMSNorm backward without any allocation.
//
//   gx[r, :]  = inv_rms[r] * (go[r, :] * w - xhat[r, :] * mean(go[r, :] * w * xhat[r, :]))
//   gw_out[d] = sum_r go[r, d] * xhat[r, d]            with xhat = x * inv_rms
//
// Same math and same kernels as ccb_rmsnorm_bwd; the difference is where the
// per-block partial sums of the weight gradient live.  Here they go into a
// 1 MiB array that is part of the library image (every GPU that loads the
// library carries it until the process exits), so nothing is allocated or
// freed by this call, directly or through a library routine.
//
//   x, w, go, gx : bf16, x/go/gx are [R, D] row-major, w is [D]
//   inv_rms      : fp32 [R], as produced by ccb_rmsnorm_fwd
//   gw_out       : fp32 [D]
//
// Limits: R <= CCB_NOALLOC_RMSNORM_MAX_ROWS, D <= CCB_NOALLOC_RMSNORM_MAX_DIM,
// D even.  Anything larger returns -1 and ccb_last_error() says which limit
// was exceeded; nothing is launched in that case.
//
// First use on a device: the first call made while a given device is current
// looks up the device address of the built-in array (once per device) before
// launching.  Make that first call outside of any stream capture.
//
// Sharing: every call on a device uses the same array.  The array keeps
// whatever the previous call left in it; that is harmless here because each
// launch overwrites every slot it later reads, so nothing needs to start at
// zero.  Two calls whose kernels can overlap on the GPU (different streams
// without ordering between them) race on the array -- order them.
int ccb_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* go, const float* inv_rms,
                            void* gx, float* gw_out, int64_t R, int64_t D, void* stream);

#ifdef __cplusplus
}
#endif
