// Entry point for callers that must not allocate device memory. It has no counterpart in the
// reference; it exists because of how this library is embedded.
//
// Who cannot allocate: code that runs while a CUDA graph is being captured on the stream, code in
// a real-time or serving loop that has promised its owner a fixed memory footprint (a cudaMalloc
// there can fail late or stall the whole device behind an implicit synchronisation), and plugins
// running inside another framework's memory pool that are handed pointers but no allocator.
// The regular LayerNorm/RMSNorm backward (inv_norm_bwd) asks its caller for a scratch buffer of
// grid*2*D floats; those callers have nowhere to get one from.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// Largest row width accepted by inv_norm_bwd_noalloc.
#define INV_NOALLOC_NORM_MAX_D 2048
// CTAs the no-allocation variant launches at most (one partial row of 2*D floats per CTA).
#define INV_NOALLOC_NORM_MAX_GRID 148

// LayerNorm (rms = 0) or RMSNorm (rms = 1) backward, same contract as inv_norm_bwd
// (dx written; dgamma and dbeta accumulated with +=, both fp32; dres optional) but without the
// scratch argument: the per-CTA partial sums live in a static device array of
// INV_NOALLOC_NORM_MAX_GRID * 2 * INV_NOALLOC_NORM_MAX_D floats (2.3 MiB) that every GPU loading
// this library holds until the process exits.
//
//  * Calls no cudaMalloc / cudaFree / allocating library routine. Inputs and outputs are the
//    caller's.
//  * D must be a multiple of 8 and at most INV_NOALLOC_NORM_MAX_D; anything else returns -7
//    (bad argument) and launches nothing.
//  * The first call on each device looks up the device address of the static array
//    (cudaGetSymbolAddress, with that device current) and caches it. Make that first call before
//    any stream capture begins.
//  * All calls on a device share the one array. Its previous contents never matter (every slot that
//    is read is written first by the same call), but two calls whose kernels overlap on the GPU
//    (different streams, no dependency) race on it. Order them on one stream or with events.
// Returns 0 on success, a negative code otherwise.
int inv_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres,
                         void* dx, float* dgamma, float* dbeta, int T, int D, int rms, void* stream);

#ifdef __cplusplus
}
#endif
