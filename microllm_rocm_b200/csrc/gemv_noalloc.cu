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

using namespace mlb;
using namespace mlb_gemv;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int MAX_DEVICES = 64;
constexpr int TARGET_CTAS = 148 * 4;
constexpr int MIN_K_PER_SPLIT = 256;

static __device__ __align__(256) float noalloc_scratch[MLB_GEMV_NOALLOC_SCRATCH_FLOATS];

// the array's device address on each device, looked up at the first call there
float* scratch_address[MAX_DEVICES] = {nullptr};

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
void choose_splits(int N, int K, int& splits, int& k_per_split) {
    const int row_blocks = (N + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    splits = (TARGET_CTAS + row_blocks - 1) / row_blocks;
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
    int splits, k_per_split;
    choose_splits(N, K, splits, k_per_split);
    return (long long)splits * M * N;
}

MLB_EXPORT int mlb_gemv_bf16_noalloc(const void* x, long long ldx, const void* w, long long ldw, const float* bias,
                                     float* out, long long ldo, int M, int N, int K, cudaStream_t stream) {
    int status = check_sizes(M, N, K);
    if (status != MLB_OK) return status;
    if (ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K || ldo < N)
        return fail(MLB_UNSUPPORTED_SIZE, "gemv_noalloc: row pitches must be multiples of 8 and cover the rows");
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(MLB_UNSUPPORTED_SIZE, "gemv_noalloc: operands must be 16-byte aligned");
    if (!out) return fail(MLB_INVALID_ARGUMENT, "gemv_noalloc: out is null");
    int splits, k_per_split;
    choose_splits(N, K, splits, k_per_split);
    const long long needed = (long long)splits * M * N;
    if (needed > (long long)MLB_GEMV_NOALLOC_SCRATCH_FLOATS)
        return fail(MLB_UNSUPPORTED_SIZE, "gemv_noalloc: this product needs %lld floats of scratch (%d splits x %d x %d) but the "
                    "library holds %u; use mlb_gemv_bf16 with your own scratch", needed, splits, M, N,
                    (unsigned)MLB_GEMV_NOALLOC_SCRATCH_FLOATS);

    // once per device, with that device current: where the array lives
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= MAX_DEVICES)
        return fail(MLB_CUDA_ERROR, "gemv_noalloc: cannot tell the current device: %s", cudaGetErrorString(e));
    if (scratch_address[device] == nullptr) {
        float* address = nullptr;
        e = cudaGetSymbolAddress((void**)&address, noalloc_scratch);
        if (e != cudaSuccess || address == nullptr)
            return fail(MLB_CUDA_ERROR, "gemv_noalloc: cudaGetSymbolAddress failed on device %d: %s", device, cudaGetErrorString(e));
        scratch_address[device] = address;
    }
    float* partial = scratch_address[device];

    const int nt = M <= 8 ? 1 : 2;
    int x_stride = k_per_split + 8;
    while ((x_stride * 2) % 128 != 64) x_stride += 8;
    const size_t smem = (size_t)nt * 8 * x_stride * 2;
    GemvParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, partial, nullptr, bias, ldx, ldw, 0, M, N, K,
                 k_per_split, x_stride, 0};
    dim3 grid((N + ROWS_PER_CTA - 1) / ROWS_PER_CTA, splits);
    static size_t configured[2] = {0, 0};
    if (smem > 48 * 1024 && smem > configured[nt - 1]) {
        e = nt == 1 ? cudaFuncSetAttribute(gemv_bf16_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                    : cudaFuncSetAttribute(gemv_bf16_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "gemv_noalloc: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured[nt - 1] = smem;
    }
    if (nt == 1) launch_kernel(gemv_bf16_kernel<1, false>, grid, WARPS * 32, smem, stream, p);
    else launch_kernel(gemv_bf16_kernel<2, false>, grid, WARPS * 32, smem, stream, p);
    status = check_launch("gemv_noalloc");
    if (status != MLB_OK) return status;
    const long long n = (long long)M * N;
    launch_kernel(noalloc_reduce_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, (const float*)partial, out, ldo, splits, M, N);
    return check_launch("gemv_noalloc reduce");
}
