// Shared declarations of the kernel library: exported-symbol macro, status codes, the
// last-error string, element load/store helpers and warp/block reductions.
//
// Every launcher is `extern "C"`, takes raw device pointers plus a CUDA stream, validates
// its sizes on the host and returns a status (0 = ok).  A refused size never launches a
// kernel: the caller reads the reason with mlb_last_error().  This is the C-ABI manner of
// the reference's bindings (bindings/capi/microllm_c.cpp:43-62: status code plus a
// thread-local message), applied to kernels instead of tensors.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <cmath>
#include <cstdlib>

#define MLB_EXPORT extern "C" __attribute__((visibility("default")))

enum MlbStatus : int {
    MLB_OK = 0,
    MLB_INVALID_ARGUMENT = 1,
    MLB_UNSUPPORTED_SIZE = 2,
    MLB_CUDA_ERROR = 3,
};

// dtype tags shared with the Python side
enum MlbDType : int { MLB_F32 = 0, MLB_BF16 = 1 };

namespace mlb {

inline char* error_buffer() {
    static thread_local char buffer[512] = {0};
    return buffer;
}

inline int fail(int status, const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(error_buffer(), 512, format, args);
    va_end(args);
    return status;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
    return MLB_OK;
}

// ---- per-device facts -----------------------------------------------------------------
// Function attributes (the dynamic shared memory a kernel may use, cluster sizes) and the number of
// multiprocessors belong to a DEVICE, not to the process: whatever a launcher sets up once, it sets up once
// per device, in arrays indexed by device_index().
constexpr int MAX_DEVICES = 64;

inline int device_index() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MAX_DEVICES) d = 0;
    return d;
}

// multiprocessors of the current device
inline int sm_count() {
    static int counts[MAX_DEVICES] = {0};
    const int d = device_index();
    if (counts[d] <= 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) return 1;
        counts[d] = n;
    }
    return counts[d];
}

// ---- element access: all arithmetic happens in fp32 ------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);   // round to nearest even, as the reference's
}                                    // float_to_bfloat16_bits (base/low_precision.h:69-74)

// ---- reductions with a fixed order (the result never depends on the batch) ------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` must
// hold 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = lane < warps ? scratch[lane] : 0.0f;
    return warp_sum(total);
}

// ---- programmatic dependent launch ---------------------------------------------------------
// A decode step is a chain of ~200 short kernels, each waiting for the one before.  Launched
// the plain way, every link pays the full launch latency after its predecessor has drained.
// With programmatic stream serialisation a kernel's CTAs may become resident while the
// predecessor still runs; they block in pdl_wait() until the predecessor has finished and its
// writes are visible, so only the launch latency overlaps, never the data dependence.
// Every kernel of this library calls pdl_prologue() before it touches memory that another
// kernel may have written.  MLB_PDL=0 in the environment turns the attribute off.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_prologue() { pdl_launch_dependents(); pdl_wait(); }

// ---- a warp held back, for tests -------------------------------------------------------------
// The warp-specialised kernels (copy warp, MMA warp, epilogue or softmax warps that meet at mbarriers) call
// lag_point() once per turn of each role's loop.  It is empty unless the object is built with -DMLB_LAG_WARP=w
// (and, for a kernel of CTA pairs or clusters, -DMLB_LAG_RANK=r): then warp w (of CTA r of its cluster) sleeps a few
// microseconds there, so that the other warps get as far ahead of it as the barriers allow.  What a kernel computes
// must not depend on which warp reaches a barrier first; the tests build such objects and compare.  Nothing else
// changes in those builds, and the package never loads them.
__device__ __forceinline__ void lag_point() {
#ifdef MLB_LAG_WARP
#ifdef MLB_LAG_RANK
    unsigned rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    if (rank != (unsigned)(MLB_LAG_RANK)) return;
#endif
    if ((int)(threadIdx.x >> 5) == (MLB_LAG_WARP)) __nanosleep(3000);
#endif
}

inline bool pdl_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* e = getenv("MLB_PDL");
        enabled = (e && e[0] == '0') ? 0 : 1;
    }
    return enabled == 1;
}

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);      // errors surface in check_launch()
}

}  // namespace mlb

// Every shared object of the library exports these two.
#define MLB_DEFINE_LAST_ERROR()                                                     \
    MLB_EXPORT const char* mlb_last_error() { return mlb::error_buffer(); }
