// Allocation-free variant of the RMSNorm backward entry point.
//
// This entry point has no counterpart in the reference implementation.  It exists for callers
// that are not allowed to call cudaMalloc (or any allocating library routine) when they need the
// kernel: code running while a CUDA graph is being captured elsewhere in the process, plugins
// that are handed a fixed memory budget by their host application, or real-time loops where an
// allocation could stall.  The regular entry point (dcpk_rmsnorm_bwd) expects the caller to
// provide a zeroed fp32 [hidden] buffer in which the weight gradient is accumulated; this
// variant keeps that accumulation buffer inside the library instead and hands back the weight
// gradient in bf16.
//
// The accumulation buffer is one file-scope device array of DCPK_NOALLOC_MAX_HIDDEN floats
// (32 KiB).  Every GPU that loads the library holds it until the process exits.
//
//  * Sizes: hidden must be 1024, 2048, 4096 or 8192 and at most DCPK_NOALLOC_MAX_HIDDEN; anything
//    else is rejected with return code -3 and a message on stderr.
//  * First call on a device: looks up the device address of the array (once per device, with that
//    device current).  Make that first call before starting any stream capture.  The looked-up
//    address is cached per device without a lock: host threads that race on the first call all
//    store the same value, which is harmless.
//  * The buffer is shared by all calls and keeps the previous call's contents; each call clears
//    the part it uses on `stream` before accumulating.  Two calls that overlap on the GPU (issued
//    on different streams without ordering) race on it - serialise them.
//  * No cudaMalloc / cudaFree / allocating library call is made, on the first call or later.
//
// Returns 0 on success, -3 for unsupported sizes, -5/-6 for CUDA errors.
#pragma once

#define DCPK_NOALLOC_MAX_HIDDEN 8192

#ifdef __cplusplus
extern "C" {
#endif

// x, w, dy, dx, dw_bf16: bf16; rstd: fp32 [n_rows] as produced by dcpk_rmsnorm_fwd.
// dx [n_rows, hidden] and dw_bf16 [hidden] are outputs; stream is a cudaStream_t.
int dcpk_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                             void* dw_bf16, int n_rows, int hidden, void* stream);

#ifdef __cplusplus
}
#endif
