// Allocation-free entry point.  (This entry point has no counterpart in the reference
// framework; it exists for the callers described below.)
//
// Who needs it: code that must not allocate device memory when it calls into this library --
// for example a serving loop embedded in a host runtime that has already handed all device
// memory to its own pool, a plugin interface that only receives input and output buffers, or a
// latency-critical path where the implicit device synchronisation of cudaMalloc / cudaFree is
// not acceptable.  Such callers cannot use the regular normalisation backward, whose Python
// front-end allocates a per-call scratch buffer for the partial weight / bias gradients.
//
// fm_norm_bwd_static computes exactly what fm_norm_bwd computes (dx, dweight, dbias of
// LayerNorm or RMSNorm, with an optional residual-branch gradient added to dx), but keeps the
// partial sums in a scratch array that is part of the library image:
//
//   * the scratch is a file-scope __device__ array of FM_NOALLOC_MAX_BLOCKS x 2 x
//     FM_NOALLOC_MAX_H floats (about 9.7 MB); every GPU on which the library is loaded holds it
//     until the process exits;
//   * H must be a multiple of 8 and at most FM_NOALLOC_MAX_H; larger sizes are rejected with a
//     non-zero return code and a message in fm_last_error();
//   * the function never calls cudaMalloc, cudaFree or any allocating library routine; the
//     caller passes every input and output buffer;
//   * the buffers must live on the device that is current at the call (checked on dx; a
//     mismatch is rejected with a non-zero return code);
//   * the first call on a device looks up the device address of the scratch array (once per
//     device, with that device current).  Make that first call before starting any stream
//     capture on the device;
//   * all calls share the one array and it keeps the contents of the last call.  Each call
//     overwrites the part it reads, so nothing has to be cleared, but two calls that overlap on
//     the GPU (different streams, or different host threads on one device) race on it: run
//     calls on one device one after another.
#pragma once
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif

#define FM_NOALLOC_MAX_H 8192
#define FM_NOALLOC_MAX_BLOCKS 148

// kind: 0 LayerNorm (mean, rstd, db used), 1 RMSNorm (mean and db may be null).
// dy, x, res_grad (may be null), dx: bf16 [T, H]; w: bf16 [H]; mean, rstd: fp32 [T];
// dw, db: fp32 [H].  Returns 0 on success.
int fm_norm_bwd_static(const void* dy, const void* x, const void* w, const float* mean,
                       const float* rstd, const void* res_grad, void* dx, float* dw, float* db, int T,
                       int H, int kind, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
