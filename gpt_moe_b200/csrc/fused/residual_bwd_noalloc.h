// residual_bwd for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference program; it exists for hosts that embed the library where
// cudaMalloc is off limits - a process whose memory pool is owned and sized by someone else (an inference server's
// arena, a plugin inside another framework) or code running between the begin and end of a CUDA stream capture,
// where an allocation is illegal.  Such callers can still provide inputs and outputs, but not the small scratch
// buffer the regular `residual_bwd` binding allocates for its per-block partial sums.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Backward of x_new = x + beta * branch with respect to `branch` and `beta`:
//     dbranch[i] = bf16(beta * dxn[i])            for i in [0, n)
//     dbeta[0]   = sum_i dxn[i] * branch[i]       (fp32, fixed summation order)
// dxn: n fp32 values; branch and dbranch: n bf16 values; beta and dbeta: one fp32 value each; all device pointers,
// 16-byte aligned.  n must be a positive multiple of 4 and at most GM_RESIDUAL_BWD_NOALLOC_MAX_ELEMS.
// `stream` is a cudaStream_t (0 for the default stream).
//
// Scratch: the per-block partial sums live in a fixed array inside the library (GM_RESIDUAL_BWD_NOALLOC_SCRATCH_FLOATS
// floats per GPU, held by every GPU that loads the library until the process exits).  All calls on one GPU share that
// array, so two calls that overlap on the GPU (different streams, no dependency) race on it; serialise them.
//
// The first call on each device looks up the array's device address (one cudaGetSymbolAddress, no allocation); make that
// first call outside any stream capture.  No call allocates or frees device memory, in this library or in torch.
//
// Threads: the looked-up address is cached per device ordinal in a plain host array.  Two host threads that make the first
// call on one device at the same time both look the address up and store the same value, which is harmless; after that the
// cache is only read.  What the threads must not do is let their launches overlap on the GPU (see "Scratch" above).
// Device reset: the cache is keyed by the device ordinal, not by the context.  After cudaDeviceReset (or with a second
// context on the same ordinal) the cached address belongs to a context that no longer exists; call
// gm_residual_bwd_noalloc_forget() after a reset so that the next call looks the address up again.
//
// Returns 0 on success, 1 for an invalid size or null pointer, 2 if the set-up or one of THIS call's two launches reported a
// CUDA error (an error left pending by earlier work on the device is neither reported nor cleared by this function).
int gm_residual_bwd_noalloc(const float* dxn, const void* branch, const float* beta, void* dbranch, float* dbeta,
                            long long n, void* stream);

// Drop the cached scratch addresses of every device (after a cudaDeviceReset).  Allocates nothing.
void gm_residual_bwd_noalloc_forget(void);

#define GM_RESIDUAL_BWD_NOALLOC_SCRATCH_FLOATS 1184
#define GM_RESIDUAL_BWD_NOALLOC_MAX_ELEMS (1LL << 34)

#ifdef __cplusplus
}
#endif
