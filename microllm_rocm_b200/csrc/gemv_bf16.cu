// Weight-streaming product for a handful of tokens (decode steps):
//     y[M, N] = x[M, K] * W[N, K]^T,   M <= 16.
//
// With so few tokens the product is pure memory traffic: every weight is read once and
// used M times.  The kernel is built around that: each warp owns 16 weight rows and walks
// its K range with 16-byte loads straight from global memory into the A fragments of
// mma.sync.m16n8k16 (W rows are the 16-row side, tokens the 8-column side), many loads in
// flight per thread, no staging of weights in shared memory.  The activations, a few KB,
// are staged once per CTA.  As in the attention kernel, thread t of a quad loads 8
// consecutive K elements and uses them as the fragments of two k-steps; x is read from
// shared memory with the same permutation.
//
// The K range may be cut over gridDim.y CTAs.  A split product leaves `splits` partial
// results [splits, M, N] in fp32; the kernel that consumes them (rotation + cache store, the
// fused residual add + norm) adds them up in split order, so no extra pass and no atomics.
// With DUAL two weight row blocks (gate rows r.., up rows up_offset + r..) run against the
// same activations and silu(gate) * up is stored as bf16 (no split: the activation is not linear).
//
// The tensor-memory kernel (gemm_stream.cu) pays a fixed price per launch (barrier set-up,
// tensor-memory allocation, one dependent tcgen05.mma chain) that amortises over larger token
// counts; up to 8 tokens this kernel is the one the engine uses.  The
// reference calls hipBLASLt for every projection whatever the batch
// (src/ops/optimized.cpp:44-70).
#include "common.cuh"
#include "gemv_kernel.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

using namespace mlb_gemv;

namespace {

template <int NT, bool DUAL>
int launch(const GemvParams& p, int splits, size_t smem, cudaStream_t stream) {
    static size_t configured_on[MAX_DEVICES] = {0};            // the attribute belongs to the device
    size_t& configured = configured_on[device_index()];
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_bf16_kernel<NT, DUAL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "gemv_bf16: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = smem;
    }
    dim3 grid((p.N + ROWS_PER_CTA - 1) / ROWS_PER_CTA, splits);
    launch_kernel(gemv_bf16_kernel<NT, DUAL>, grid, WARPS * 32, smem, stream, p);
    return check_launch("gemv_bf16");
}

}  // namespace

MLB_EXPORT int mlb_gemv_max_tokens() { return 16; }

// partial[splits, M, N] = x * W^T cut into `splits` K ranges of k_per_split elements (a multiple of
// 32; bias, if given, goes into split 0), or with dual: out[M, N] bf16 = silu(x Wg^T) * (x Wu^T) with
// Wg = W rows [0, N), Wu = W rows [up_offset, up_offset + N).  K must be a multiple of 32, the row
// pitches multiples of 8 and the bases 16-byte aligned.
MLB_EXPORT int mlb_gemv_bf16(const void* x, long long ldx, const void* w, long long ldw, int w_rows, const float* bias,
                             float* partial, void* out, long long ldo, int dual, int up_offset, int M, int N, int K,
                             int splits, int k_per_split, cudaStream_t stream) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0) return fail(MLB_UNSUPPORTED_SIZE, "gemv_bf16: M=%d must be 1..16 (N=%d K=%d)", M, N, K);
    if (K % 32 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K)
        return fail(MLB_UNSUPPORTED_SIZE, "gemv_bf16: K=%d must be a multiple of 32 and the row pitches multiples of 8", K);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(MLB_UNSUPPORTED_SIZE, "gemv_bf16: operands must be 16-byte aligned");
    if (splits < 1 || k_per_split <= 0 || k_per_split % 32 != 0 || (long long)splits * k_per_split < K)
        return fail(MLB_INVALID_ARGUMENT, "gemv_bf16: %d splits of %d do not cover K=%d in steps of 32", splits, k_per_split, K);
    if (dual && (splits != 1 || !out || up_offset < 0 || up_offset + N > w_rows))
        return fail(MLB_INVALID_ARGUMENT, "gemv_bf16: a dual product is not split and needs its up rows inside the weight");
    if (!dual && (!partial || N > w_rows)) return fail(MLB_INVALID_ARGUMENT, "gemv_bf16: missing output");
    const int nt = M <= 8 ? 1 : 2;
    int x_stride = k_per_split + 8;                        // pitch in bytes = 64 mod 128: 16-byte row loads
    while ((x_stride * 2) % 128 != 64) x_stride += 8;      // of two neighbouring rows hit different banks
    const size_t smem = (size_t)nt * 8 * x_stride * 2;
    if (smem > 200 * 1024) return fail(MLB_UNSUPPORTED_SIZE, "gemv_bf16: a K range of %d per CTA does not fit shared memory; split more", k_per_split);
    GemvParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, partial, out, bias, ldx, ldw, ldo, M, N, K,
                 k_per_split, x_stride, up_offset};
    if (nt == 1) return dual ? launch<1, true>(p, splits, smem, stream) : launch<1, false>(p, splits, smem, stream);
    return dual ? launch<2, true>(p, splits, smem, stream) : launch<2, false>(p, splits, smem, stream);
}
