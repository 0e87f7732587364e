/* A few-token product that allocates nothing.
 *
 * This entry point has no counterpart in walkinglabs/microLLM-rocm: it exists for callers of
 * this library that are not allowed to allocate device memory at the time of the call -- a
 * host program that has handed all of its memory to its own pool, a plugin that runs inside
 * someone else's allocator, code on a path where cudaMalloc (which synchronises the device
 * and may fail under fragmentation) is forbidden.  The regular entry point, mlb_gemv_bf16,
 * wants the caller to pass scratch memory for the partial results of a product whose K
 * range is split over CTAs; this one keeps that scratch in a fixed array inside the library.
 *
 *   out[M, N] (fp32) = x[M, K] (bf16) * W[N, K]^T (bf16)  (+ bias[N])        1 <= M <= 16
 *
 * What to know before using it:
 *   - The scratch is a file-scope device array of MLB_GEMV_NOALLOC_SCRATCH_FLOATS floats
 *     (16 MiB).  Every GPU on which this library is loaded holds it until the process exits.
 *   - A product needs splits * M * N floats of it (the split count is chosen from N and K as
 *     in the regular path).  A product that needs more is refused with
 *     MLB_UNSUPPORTED_SIZE and a message; nothing is launched.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress) and remembers it.  Make that first call outside any CUDA stream
 *     capture.
 *   - All calls share the one array, and it keeps whatever the last call left in it.  Nothing
 *     in it has to be zero: every element a call reads it has written first.  Two calls that
 *     may run at the same time on the GPU (different streams, no ordering between them) race
 *     on it; order them.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine, and returns the same
 *     status codes as the rest of the library (0 = ok; mlb_last_error() has the message).
 */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MLB_GEMV_NOALLOC_SCRATCH_FLOATS (4u << 20)

/* x: [M, ldx] bf16, w: [N, ldw] bf16, bias: [N] fp32 or NULL, out: [M, ldo] fp32.
 * K a multiple of 32, ldx and ldw multiples of 8, x and w 16-byte aligned. */
int mlb_gemv_bf16_noalloc(const void* x, long long ldx, const void* w, long long ldw, const float* bias, float* out,
                          long long ldo, int M, int N, int K, cudaStream_t stream);

/* Floats of scratch the product above would need, or -1 if its sizes are refused anyway. */
long long mlb_gemv_bf16_noalloc_scratch_needed(int M, int N, int K);

#ifdef __cplusplus
}
#endif
