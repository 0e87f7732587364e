// True 32-bit matrix product for the fp32 path:  C[M,N] (+)= A[M,K] * W[N,K]^T (+ bias[N]).
//
// CUDA cores only, plain fp32 FMA: no tensor cores, no TF32.  Each output element is
// accumulated by ONE thread over k = 0..K-1 in increasing order, so its value does not
// depend on M, on the tile it falls in, or on what else is in the batch.  This is the role
// of the reference's readable matmul (src/ops/hip/basic_kernels.hip:319-336: one thread per
// output element, serial K loop), with shared-memory tiling added for reuse.
// W is kept in the checkpoint's own [out, in] layout (K contiguous); the reference
// transposes every linear weight to [in, out] at load (src/model/model.cpp:1928-1982).
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <bool ACCUMULATE>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ W, const float* __restrict__ bias,
                float* __restrict__ C, int M, int N, int K, long long lda, long long ldw, long long ldc) {
    pdl_prologue();
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;           // 16 x 16 threads, each a 4 x 4 patch
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements of each operand, 4 per thread; k runs fastest in memory
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int row = e / BK, kk = e % BK;
            const int k = k0 + kk;
            const int m = m0 + row, n = n0 + row;
            As[kk][row] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.0f;
            Ws[kk][row] = (n < N && k < K) ? W[(size_t)n * ldw + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            float* dst = C + (size_t)m * ldc + n;
            *dst = ACCUMULATE ? (*dst + v) : v;
        }
    }
}

}  // namespace

// accumulate != 0:  C += A*W^T (+bias)   (the residual add of the o/down projections)
MLB_EXPORT int mlb_gemm_f32(const float* A, const float* W, const float* bias, float* C, int M, int N, int K,
                            long long lda, long long ldw, long long ldc, int accumulate, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0 || lda < K || ldw < K || ldc < N)
        return fail(MLB_INVALID_ARGUMENT, "gemm_f32: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return MLB_OK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) return fail(MLB_UNSUPPORTED_SIZE, "gemm_f32: M=%d exceeds %d rows per call", M, 65535 * BM);
    if (accumulate)
        launch_kernel(gemm_f32_kernel<true>, grid, 256, 0, stream, A, W, bias, C, M, N, K, lda, ldw, ldc);
    else
        launch_kernel(gemm_f32_kernel<false>, grid, 256, 0, stream, A, W, bias, C, M, N, K, lda, ldw, ldc);
    return check_launch("gemm_f32");
}
