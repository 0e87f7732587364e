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
 *     (cudaGetSymbolAddress), the device's multiprocessor count and, for long K ranges, raises
 *     the kernel's shared-memory limit, and remembers all three (behind a mutex: first calls
 *     from several host threads are safe).  Make that first call outside any CUDA stream
 *     capture.  With CUDA's default lazy module loading it is also the moment the driver
 *     loads this library's module on that device and backs the 16 MiB array: that one call
 *     therefore does reserve device memory, may synchronise, and can fail for lack of memory.
 *     Treat it as a warm-up to make at initialisation, while allocating is still allowed;
 *     every later call on that device allocates nothing.
 *   - The kernel is launched with programmatic stream serialisation and fetches W before it
 *     waits for the kernel in front of it on the stream (x, bias and out are touched only
 *     after that wait).  W must therefore not be written by the kernel launched immediately
 *     before this call on the same stream (a dequantisation or a weight copy, say); if it is,
 *     put another launch or an event in between, or set MLB_PDL=0 in the environment, which
 *     turns the early start off for the whole library.
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
 * K a multiple of 32, ldx and ldw multiples of 8, x and w 16-byte aligned; a NULL x, w or out is
 * refused with MLB_INVALID_ARGUMENT before anything is launched. */
int mlb_gemv_bf16_noalloc(const void* x, long long ldx, const void* w, long long ldw, const float* bias, float* out,
                          long long ldo, int M, int N, int K, cudaStream_t stream);

/* Floats of scratch the product above would need on the current device (the split follows its
 * multiprocessor count), or -1 if its sizes are refused anyway. */
long long mlb_gemv_bf16_noalloc_scratch_needed(int M, int N, int K);

#ifdef __cplusplus
}
#endif
