// The few-token product with its scratch memory inside the library: see gemv_noalloc.h for
// who needs this and what its limits are.  It has no counterpart in the reference.
//
// Same kernel as gemv_bf16.cu (gemv_kernel.cuh): the K range is cut over CTAs, each leaves
// an fp32 partial result, and a second small kernel adds them in split order into `out`.
// The partial results live in `noalloc_scratch`, a file-scope device array.  In host code
// that name is only a handle; its device address comes from cudaGetSymbolAddress, once per
// device, and that pointer is what the kernels are given.
#include "gemv_noalloc.h"

#include "common.cuh"
#include "gemv_kernel.cuh"

#include <mutex>

using namespace mlb;
using namespace mlb_gemv;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int MAX_DEVICES = 64;
constexpr int CTAS_PER_SM = 4;               // CTAs the split aims at, per multiprocessor of the current device
constexpr int MIN_K_PER_SPLIT = 256;

static __device__ __align__(256) float noalloc_scratch[MLB_GEMV_NOALLOC_SCRATCH_FLOATS];

// What the first call on a device finds out and later calls reuse: where the array lives there, how many
// multiprocessors the device has, and how much dynamic shared memory each kernel variant may already use
// (that limit is a per-device attribute of the function).  Guarded by `setup_mutex`: two host threads may
// make their first call at the same time.
struct DeviceSetup {
    float* scratch = nullptr;
    int sm_count = 0;
    size_t smem_configured[2] = {0, 0};
};
DeviceSetup device_setup[MAX_DEVICES];
std::mutex setup_mutex;

int current_device(int& device) {
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES)
        return fail(MLB_CUDA_ERROR, "gemv_noalloc: cannot tell the current device: %s", cudaGetErrorString(e));
    return MLB_OK;
}

int sm_count_of(int device, int& count) {
    std::lock_guard<std::mutex> lock(setup_mutex);
    if (device_setup[device].sm_count == 0) {
        int n = 0;
        cudaError_t e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess || n <= 0) return fail(MLB_CUDA_ERROR, "gemv_noalloc: cannot read the multiprocessor count: %s", cudaGetErrorString(e));
        device_setup[device].sm_count = n;
    }
    count = device_setup[device].sm_count;
    return MLB_OK;
}

// out[m, n] = sum over splits of partial[s, m, n], in split order
__global__ void noalloc_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out, long long ldo, int splits,
                                      int M, int N) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)M * N) return;
    const int m = (int)(i / N), n = (int)(i % N);
    float acc = partial[i];
    for (int s = 1; s < splits; ++s) acc += partial[(size_t)s * M * N + i];
    out[(size_t)m * ldo + n] = acc;
}

// the split choice of the regular path (kernels/gemm_bf16.py: gemv_splits)
void choose_splits(int N, int K, int sm_count, int& splits, int& k_per_split) {
    const int row_blocks = (N + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    splits = (sm_count * CTAS_PER_SM + row_blocks - 1) / row_blocks;
    if (splits > K / MIN_K_PER_SPLIT) splits = K / MIN_K_PER_SPLIT;
    if (splits < 1) splits = 1;
    k_per_split = ((K + splits - 1) / splits + 31) / 32 * 32;
    while ((long long)k_per_split * 2 * 16 > 160 * 1024) k_per_split = (k_per_split / 2 + 31) / 32 * 32;
    splits = (K + k_per_split - 1) / k_per_split;
}

int check_sizes(int M, int N, int K) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0) return fail(MLB_UNSUPPORTED_SIZE, "gemv_noalloc: M=%d must be 1..16 (N=%d K=%d)", M, N, K);
    if (K % 32 != 0) return fail(MLB_UNSUPPORTED_SIZE, "gemv_noalloc: K=%d must be a multiple of 32", K);
    return MLB_OK;
}

}  // namespace

MLB_EXPORT long long mlb_gemv_bf16_noalloc_scratch_needed(int M, int N, int K) {
    if (check_sizes(M, N, K) != MLB_OK) return -1;
    int device = -1, sms = 0;
    if (current_device(device) != MLB_OK || sm_count_of(device, sms) != MLB_OK) return -1;
    int splits, k_per_split;
    choose_splits(N, K, sms, splits, k_per_split);
    return (long long)splits * M * N;
}

MLB_EXPORT int mlb_gemv_bf16_noalloc(const void* x, long long ldx, const void* w, long long ldw, const float* bias,
                                     float* out, long long ldo, int M, int N, int K, cudaStream_t stream) {
    int status = check_sizes(M, N, K);
    if (status != MLB_OK) return status;
    if (ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K || ldo < N)
        return fail(MLB_UNSUPPORTED_SIZE, "gemv_noalloc: row pitches must be multiples of 8 and cover the rows");
    if (!x || !w || !out) return fail(MLB_INVALID_ARGUMENT, "gemv_noalloc: x, w and out must not be null");
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(MLB_UNSUPPORTED_SIZE, "gemv_noalloc: operands must be 16-byte aligned");
    int device = -1, sms = 0;
    status = current_device(device);
    if (status != MLB_OK) return status;
    status = sm_count_of(device, sms);
    if (status != MLB_OK) return status;
    int splits, k_per_split;
    choose_splits(N, K, sms, splits, k_per_split);
    const long long needed = (long long)splits * M * N;
    if (needed > (long long)MLB_GEMV_NOALLOC_SCRATCH_FLOATS)
        return fail(MLB_UNSUPPORTED_SIZE, "gemv_noalloc: this product needs %lld floats of scratch (%d splits x %d x %d) but the "
                    "library holds %u; use mlb_gemv_bf16 with your own scratch", needed, splits, M, N,
                    (unsigned)MLB_GEMV_NOALLOC_SCRATCH_FLOATS);

    const int nt = M <= 8 ? 1 : 2;
    int x_stride = k_per_split + 8;
    while ((x_stride * 2) % 128 != 64) x_stride += 8;
    const size_t smem = (size_t)nt * 8 * x_stride * 2;

    // once per device, with that device current: where the array lives; and, per device too, the shared
    // memory this kernel variant may use
    float* partial = nullptr;
    {
        std::lock_guard<std::mutex> lock(setup_mutex);
        DeviceSetup& setup = device_setup[device];
        cudaError_t e;
        if (setup.scratch == nullptr) {
            float* address = nullptr;
            e = cudaGetSymbolAddress((void**)&address, noalloc_scratch);
            if (e != cudaSuccess || address == nullptr)
                return fail(MLB_CUDA_ERROR, "gemv_noalloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
            setup.scratch = address;
        }
        partial = setup.scratch;
        if (smem > 48 * 1024 && smem > setup.smem_configured[nt - 1]) {
            e = nt == 1 ? cudaFuncSetAttribute(gemv_bf16_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                        : cudaFuncSetAttribute(gemv_bf16_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "gemv_noalloc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            setup.smem_configured[nt - 1] = smem;
        }
    }

    GemvParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, partial, nullptr, bias, ldx, ldw, 0, M, N, K,
                 k_per_split, x_stride, 0};
    dim3 grid((N + ROWS_PER_CTA - 1) / ROWS_PER_CTA, splits);
    if (nt == 1) launch_kernel(gemv_bf16_kernel<1, false>, grid, WARPS * 32, smem, stream, p);
    else launch_kernel(gemv_bf16_kernel<2, false>, grid, WARPS * 32, smem, stream, p);
    status = check_launch("gemv_noalloc");
    if (status != MLB_OK) return status;
    const long long n = (long long)M * N;
    launch_kernel(noalloc_reduce_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, (const float*)partial, out, ldo, splits, M, N);
    return check_launch("gemv_noalloc reduce");
}
