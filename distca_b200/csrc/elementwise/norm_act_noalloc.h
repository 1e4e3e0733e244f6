// RMSNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference.
//
// Who needs it: a process that hands all of its device memory to an arena or a caching allocator
// at start-up (any later cudaMalloc either fails or makes that allocator give blocks back, which
// synchronises the whole device), and code that runs on a thread where the implicit device-wide
// synchronisation of cudaMalloc / cudaFree would stall every other stream of the process, such as
// the thread that drives pipeline send/recv while compute runs. `dca_rmsnorm_bwd` asks such callers
// for a scratch buffer they have no way to provide; this variant brings its own.
//
// The scratch (per-CTA partial sums of the weight gradient) lives in a file-scope
// `static __device__` array inside the library, so EVERY GPU that loads the library holds
// kNoAllocScratchBytes of device memory from load until the process exits, used or not.
//
// Limits: hidden size H <= kNoAllocMaxH (and a multiple of 8); the number of partial rows is
// min(T, 2 * SM count) and must be <= kNoAllocMaxPartials. Larger problems are rejected with
// kErrTooLarge (-4) and a message on stderr; nothing is launched in that case.
//
// Rules of use
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress with
//    that device current) and reads the SM count; it launches nothing else extra. Make that first
//    call before starting any stream capture on the device. First calls that arrive from several host
//    threads at once are safe: the set-up runs once per device and the other callers wait for it.
//  * The function calls no cudaMalloc, cudaFree or allocating library routine.
//  * All calls on one device share the one array. Nothing in it has to start at zero (every launch
//    overwrites the rows it later reads), but two calls that overlap on the GPU (different streams,
//    no dependency between them) race on it and corrupt each other's weight gradient. Serialise them.
//  * Inputs and outputs are the caller's, exactly as for `dca_rmsnorm_bwd`:
//      x, g, dy, dres (may be null), dx : bf16; rstd : fp32 [T]; dg : bf16 or fp32 [H]
//      (dg_fp32), overwritten or accumulated into (dg_accumulate).
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  kNoAllocMaxH = 8192,
  kNoAllocMaxPartials = 320,
};
#define kNoAllocScratchBytes ((size_t)kNoAllocMaxPartials * kNoAllocMaxH * sizeof(float))  /* 10 MiB */

// Returns 0, a cudaError_t value, -1 (bad shape / alignment) or -4 (beyond the limits above).
int dca_rmsnorm_bwd_noalloc(const void* x, const void* g, const float* rstd, const void* dy, const void* dres,
                            void* dx, void* dg, int dg_fp32, int dg_accumulate, int T, int H, void* stream);

#ifdef __cplusplus
}
#endif
