// RMSNorm backward for callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference framework; it exists for hosts of
// this library that cannot call cudaMalloc themselves or tolerate a library doing it behind
// their back: code running inside a CUDA-graph capture or another no-sync region, plugins
// embedded in a serving process whose memory pool is owned by someone else, and real-time
// loops where an allocation could block on the driver.  The regular entry point
// (ttb_rmsnorm_bwd) asks the caller for a scratch buffer of per-CTA partial sums; this
// variant keeps that scratch in a fixed array that is part of the library image instead.
//
// Contract
//   * Inputs and outputs are the caller's: dy, x, scale (bf16 [rows, D] / [D]), rstd (fp32
//     [rows], as written by ttb_rmsnorm_fwd), dx (bf16 [rows, D]) and dscale (fp32 [D]).
//     `scale` may be null (weight-less norm); then `dscale` is not written and may be null.
//   * Limits: D is a multiple of 8 and at most TTB_RMSNORM_NOALLOC_MAX_D (8192); any number of
//     rows.  Larger D is refused with the "size beyond a static limit" code (-3).
//   * The scratch array holds TTB_RMSNORM_NOALLOC_MAX_CTAS x TTB_RMSNORM_NOALLOC_MAX_D floats
//     (4 MiB).  Every GPU that loads the library carries it until the process exits.
//   * The library links its own copy of the CUDA runtime, whose "current device" is per host thread and starts at
//     device 0.  A caller working on another device binds the calling thread first with ttb_ensure_device(dev);
//     otherwise the lookup below returns device 0's copy of the array and the launch goes there.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress)
//     and remembers it; make that first call outside of any stream capture.
//   * Nothing in the scratch needs to start at zero: each call overwrites every partial row it
//     later reads.  All calls share the one array, so two calls that overlap on the GPU
//     (different streams, or graphs replayed concurrently) race with each other — serialise
//     them.
//   * No cudaMalloc / cudaFree / allocating library routine is called on any path.
#pragma once

#define TTB_RMSNORM_NOALLOC_MAX_D 8192
#define TTB_RMSNORM_NOALLOC_MAX_CTAS 128

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success, -1 for a bad shape (D not a multiple of 8, rows <= 0), -2 when the
// scratch address lookup or the launch failed, -3 when D exceeds the static limit.
int ttb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* scale, const float* rstd, void* dx,
                            float* dscale, int rows, int D, void* stream);

#ifdef __cplusplus
}
#endif
