// Few-token products that finish their own epilogue, so that a decode step needs neither
// partial results nor the small kernels that would consume them:
//
//   mlb_gemv_silu      act[M, I]  = silu(x Wg^T) * (x Wu^T)                     (gate/up + activation)
//   mlb_gemv_qkv_rope  q, k, v    = x Wqkv^T + b;  q, k rotated;  k, v stored into the paged cache
//   mlb_gemv_split     partial[S] = x W^T over S ranges of K                    (few partial sums for the consumer)
//
// Both stream the weights exactly like gemv_bf16_kernel (16-byte loads straight into
// mma.sync.m16n8k16 fragments, two register sets in flight, the first loads issued before the
// wait for the previous kernel), but a CTA owns ONE 16-row tile over the whole K range and
// its warps split K among themselves; the warps' accumulators meet in shared memory and are
// added in warp order, so the result does not depend on timing.
//
// The two rows a thread's fragments hold (g and g+8 of the tile) need not be neighbours in
// the weight.  The rotation kernel uses that: row g+8 is row g's partner of the split-half
// rotation (element i + D/2 of the same head), so that each pair (x_i, x_{i+D/2}) ends up in
// one thread and is rotated in registers.  Sines and cosines come from positions and inverse
// frequencies, both known before the previous kernel has finished: they are computed before the wait.
//
// Formulas: SiLU as the reference's two-branch sigmoid (src/ops/ops.cpp:72-76, 760-785);
// rotation x_i' = x_i cos - x_{i+D/2} sin, x_{i+D/2}' = x_i sin + x_{i+D/2} cos with
// angle = position * theta^(-2i/D) in fp32 (src/ops/ops.cpp:1246-1300); bias before the rotation
// (src/model/model.cpp:457-476).
#include "common.cuh"
#include "gemv_kernel.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

using namespace mlb_gemv;

namespace {

// One warp's share of a 16-row tile: rows (wa, wb) and, with DUAL, (ua, ub), chunks of 32 K elements.
template <int NT, bool DUAL, int B>
struct Streamer {
    struct Set { uint4 a[B], b[B], ua[DUAL ? B : 1], ub[DUAL ? B : 1]; };
    const __nv_bfloat16 *wa, *wb, *ua, *ub;        // at this warp's first chunk, + t*8
    int chunks;
    Set s0, s1;
    float acc[NT][4], acc_u[DUAL ? NT : 1][4];

    __device__ __forceinline__ void load(Set& s, int c0) {
#pragma unroll
        for (int u = 0; u < B; ++u) {
            if (c0 + u < chunks) {
                s.a[u] = ldg_stream(wa + (size_t)(c0 + u) * 32);
                s.b[u] = ldg_stream(wb + (size_t)(c0 + u) * 32);
                if (DUAL) {
                    s.ua[u] = ldg_stream(ua + (size_t)(c0 + u) * 32);
                    s.ub[u] = ldg_stream(ub + (size_t)(c0 + u) * 32);
                }
            }
        }
    }
    __device__ __forceinline__ void mma(const Set& s, int c0, const __nv_bfloat16* xs, int x_stride) {
#pragma unroll
        for (int u = 0; u < B; ++u) {
            if (c0 + u < chunks) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)n * 8 * x_stride + (c0 + u) * 32);
                    mma_bf16(acc[n], s.a[u].x, s.b[u].x, s.a[u].y, s.b[u].y, xv.x, xv.y);
                    mma_bf16(acc[n], s.a[u].z, s.b[u].z, s.a[u].w, s.b[u].w, xv.z, xv.w);
                    if (DUAL) {
                        mma_bf16(acc_u[n], s.ua[u].x, s.ub[u].x, s.ua[u].y, s.ub[u].y, xv.x, xv.y);
                        mma_bf16(acc_u[n], s.ua[u].z, s.ub[u].z, s.ua[u].w, s.ub[u].w, xv.z, xv.w);
                    }
                }
            }
        }
    }
    __device__ __forceinline__ void clear() {
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) { acc[n][e] = 0.0f; if (DUAL) acc_u[n][e] = 0.0f; }
    }
    __device__ __forceinline__ void preload() { load(s0, 0); load(s1, B); }
    __device__ __forceinline__ void run(const __nv_bfloat16* xs, int x_stride) {
        for (int c0 = 0; c0 < chunks; c0 += 2 * B) {
            mma(s0, c0, xs, x_stride);
            load(s0, c0 + 2 * B);
            mma(s1, c0 + B, xs, x_stride);
            load(s1, c0 + 3 * B);
        }
    }
};

// all NT*8 token rows of x over the whole K into shared memory; rows beyond M are zero
template <int NT>
__device__ __forceinline__ void stage_x(__nv_bfloat16* x_s, const __nv_bfloat16* x, long long ldx, int M, int K, int x_stride,
                                        int threads) {
    const int vec_per_row = K / 8;
    for (int i = threadIdx.x; i < NT * 8 * vec_per_row; i += threads) {
        const int r = i / vec_per_row, c = (i % vec_per_row) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < M) v = *reinterpret_cast<const uint4*>(x + (size_t)r * ldx + c);
        *reinterpret_cast<uint4*>(x_s + (size_t)r * x_stride + c) = v;
    }
}

// ------------------------------------------------------------------------------ gate/up + SiLU
struct SiluParams {
    const __nv_bfloat16* x;      // [M, ldx]
    const __nv_bfloat16* w;      // gate rows [0, I), up rows [up_offset, up_offset + I); pitch ldw
    __nv_bfloat16* out;          // [M, ldo]
    long long ldx, ldw, ldo;
    int M, I, K, up_offset, x_stride;
};

constexpr int SILU_WARPS = 4;
constexpr int SILU_BATCH = 2;

template <int NT>
__global__ void __launch_bounds__(SILU_WARPS * 32) gemv_silu_kernel(SiluParams p) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)NT * 8 * p.x_stride * 2);     // [W][2][NT*4][32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int f0 = blockIdx.x * 16;
    const int total_chunks = p.K / 32, per_warp = (total_chunks + SILU_WARPS - 1) / SILU_WARPS;
    const int c_begin = min(total_chunks, warp * per_warp);
    const int ra = min(f0 + g, p.I - 1), rb = min(f0 + g + 8, p.I - 1);       // rows past the end read the last row (never stored)

    Streamer<NT, true, SILU_BATCH> st;
    st.chunks = min(total_chunks, c_begin + per_warp) - c_begin;
    st.wa = p.w + (size_t)ra * p.ldw + c_begin * 32 + t * 8;
    st.wb = p.w + (size_t)rb * p.ldw + c_begin * 32 + t * 8;
    st.ua = st.wa + (size_t)p.up_offset * p.ldw;
    st.ub = st.wb + (size_t)p.up_offset * p.ldw;
    st.clear();
    st.preload();                                  // weights: before the wait for the previous kernel
    pdl_wait();
    stage_x<NT>(x_s, p.x, p.ldx, p.M, p.K, p.x_stride, SILU_WARPS * 32);
    __syncthreads();
    st.run(x_s + (size_t)g * p.x_stride + c_begin * 32 + t * 8, p.x_stride);

#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            red[((warp * 2 + 0) * NT * 4 + n * 4 + e) * 32 + lane] = st.acc[n][e];
            red[((warp * 2 + 1) * NT * 4 + n * 4 + e) * 32 + lane] = st.acc_u[n][e];
        }
    __syncthreads();
    // element e of column block n of lane (g, t): row g (e < 2) or g+8, token n*8 + 2t + (e & 1)
    for (int o = threadIdx.x; o < NT * 4 * 32; o += SILU_WARPS * 32) {
        const int ne = o >> 5, l2 = o & 31, n = ne >> 2, e = ne & 3;
        const int row = f0 + (l2 >> 2) + 8 * (e >> 1), tok = n * 8 + 2 * (l2 & 3) + (e & 1);
        float gate = 0.0f, up = 0.0f;
#pragma unroll
        for (int w = 0; w < SILU_WARPS; ++w) {
            gate += red[((w * 2 + 0) * NT * 4 + ne) * 32 + l2];
            up += red[((w * 2 + 1) * NT * 4 + ne) * 32 + l2];
        }
        if (row < p.I && tok < p.M) p.out[(size_t)tok * p.ldo + row] = __float2bfloat16_rn(silu(gate) * up);
    }
}

// ------------------------------------------------------------------------------ QKV + bias + rotation + cache store
struct QkvParams {
    const __nv_bfloat16* x;      // [M, ldx]
    const __nv_bfloat16* w;      // [(NH + 2 NKV) * D, ldw]: q heads, k heads, v heads
    const float* bias;           // [(NH + 2 NKV) * D] or null
    long long ldx, ldw;
    int M, K, x_stride;
    const int* positions;        // [M]
    const int* token_seq;        // [M]
    const int* block_table;      // [A, max_blocks]
    const float* inv_freq;       // [D/2] (unused when rotate == 0)
    __nv_bfloat16* q_out;        // [M, NH * D]
    __nv_bfloat16* pages;        // [num_pages, 2, NKV, page_size, D] or null (keys and values are dropped)
    int max_blocks, num_pages, page_size;
    int num_heads, num_kv_heads, head_dim, rotate;
    int* error_flag;
};

constexpr int QKV_WARPS = 8;
constexpr int QKV_BATCH = 4;

template <int NT>
__global__ void __launch_bounds__(QKV_WARPS * 32) gemv_qkv_rope_kernel(QkvParams p) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)NT * 8 * p.x_stride * 2);     // [W][NT*4][32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // the tile: pairs pb*8 .. pb*8+7 of one head; fragment row g is element i = pb*8 + g, row g+8 its partner i + D/2
    const int D = p.head_dim, half = D / 2, tiles_per_head = half / 8;
    const int head = blockIdx.x / tiles_per_head, pb = blockIdx.x % tiles_per_head;
    const int total_chunks = p.K / 32, per_warp = (total_chunks + QKV_WARPS - 1) / QKV_WARPS;
    const int c_begin = min(total_chunks, warp * per_warp);
    const int row_a = head * D + pb * 8 + g, row_b = row_a + half;

    Streamer<NT, false, QKV_BATCH> st;
    st.chunks = min(total_chunks, c_begin + per_warp) - c_begin;
    st.wa = p.w + (size_t)row_a * p.ldw + c_begin * 32 + t * 8;
    st.wb = p.w + (size_t)row_b * p.ldw + c_begin * 32 + t * 8;
    st.ua = st.ub = nullptr;
    st.clear();
    st.preload();

    // The epilogue's inputs, also before the wait.  Epilogue thread o < NT*64: column block n = o / 64,
    // token parity e01 = (o / 32) & 1, fragment lane l2 = o % 32 -> token n*8 + 2*(l2 & 3) + e01, pair l2 >> 2.
    const bool is_q = head < p.num_heads;
    const bool is_v = head >= p.num_heads + p.num_kv_heads;
    const int o = threadIdx.x;
    const int n_e = o >> 6, e01 = (o >> 5) & 1, l2 = o & 31;
    const int tok = n_e * 8 + 2 * (l2 & 3) + e01, pair = pb * 8 + (l2 >> 2);
    const bool finishing = o < NT * 64 && tok < p.M;
    float sn = 0.0f, cs = 1.0f, bias_a = 0.0f, bias_b = 0.0f;
    int pos = 0, page = -1;
    if (finishing) {
        pos = p.positions[tok];
        if (p.rotate && !is_v) sincosf((float)pos * p.inv_freq[pair], &sn, &cs);
        if (p.bias) { bias_a = p.bias[head * D + pair]; bias_b = p.bias[head * D + pair + half]; }
        if (!is_q && p.pages) {
            const int block = pos / p.page_size;
            if (pos >= 0 && block < p.max_blocks) page = p.block_table[(size_t)p.token_seq[tok] * p.max_blocks + block];
        }
    }
    pdl_wait();
    stage_x<NT>(x_s, p.x, p.ldx, p.M, p.K, p.x_stride, QKV_WARPS * 32);
    __syncthreads();
    st.run(x_s + (size_t)g * p.x_stride + c_begin * 32 + t * 8, p.x_stride);
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[((warp * NT + n) * 4 + e) * 32 + lane] = st.acc[n][e];
    __syncthreads();
    if (!finishing) return;
    float a = 0.0f, b = 0.0f;                      // element `pair` and its partner, summed over the warps in order
#pragma unroll
    for (int w = 0; w < QKV_WARPS; ++w) {
        a += red[((w * NT + n_e) * 4 + e01) * 32 + l2];
        b += red[((w * NT + n_e) * 4 + e01 + 2) * 32 + l2];
    }
    a += bias_a;
    b += bias_b;
    const float ra = a * cs - b * sn, rb = a * sn + b * cs;      // sn = 0, cs = 1 where nothing rotates
    if (is_q) {
        __nv_bfloat16* dst = p.q_out + ((size_t)tok * p.num_heads + head) * D;
        dst[pair] = __float2bfloat16_rn(ra);
        dst[pair + half] = __float2bfloat16_rn(rb);
        return;
    }
    if (!p.pages) return;
    if (page < 0 || page >= p.num_pages) {
        if (p.error_flag) atomicExch(p.error_flag, 1);
        return;
    }
    const int kvh = is_v ? head - p.num_heads - p.num_kv_heads : head - p.num_heads;
    __nv_bfloat16* dst = p.pages + ((((size_t)page * 2 + (is_v ? 1 : 0)) * p.num_kv_heads + kvh) * p.page_size + pos % p.page_size) * D;
    dst[pair] = __float2bfloat16_rn(ra);
    dst[pair + half] = __float2bfloat16_rn(rb);
}

// ------------------------------------------------------------------------------ plain product, K split inside the CTA
// partial[split, M, N] = x[:, k range of the split] * W[:, the same]^T.  The grid is (16-row tiles, splits):
// the warps of a CTA share the split's K range, so a product needs far fewer partial results than with one
// warp per K range (the consumer adds them up), and most of a warp's weights are on their way before the wait.
struct SplitParams {
    const __nv_bfloat16* x;      // [M, ldx]
    const __nv_bfloat16* w;      // [N, ldw]
    const float* bias;           // [N] or null; added by split 0
    float* partial;              // [splits, M, N]
    long long ldx, ldw;
    int M, N, K, k_per_cta, x_stride;
};

constexpr int SPLIT_WARPS = 8;
constexpr int SPLIT_BATCH = 4;

template <int NT>
__global__ void __launch_bounds__(SPLIT_WARPS * 32) gemv_split_kernel(SplitParams p) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)NT * 8 * p.x_stride * 2);     // [W][NT*4][32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int f0 = blockIdx.x * 16;
    const int k_begin = blockIdx.y * p.k_per_cta, k_len = max(0, min(p.K, k_begin + p.k_per_cta) - k_begin);
    const int total_chunks = k_len / 32, per_warp = (total_chunks + SPLIT_WARPS - 1) / SPLIT_WARPS;
    const int c_begin = min(total_chunks, warp * per_warp);
    const int ra = min(f0 + g, p.N - 1), rb = min(f0 + g + 8, p.N - 1);       // rows past the end read the last row (never stored)

    Streamer<NT, false, SPLIT_BATCH> st;
    st.chunks = min(total_chunks, c_begin + per_warp) - c_begin;
    st.wa = p.w + (size_t)ra * p.ldw + k_begin + c_begin * 32 + t * 8;
    st.wb = p.w + (size_t)rb * p.ldw + k_begin + c_begin * 32 + t * 8;
    st.ua = st.ub = nullptr;
    st.clear();
    st.preload();
    pdl_wait();
    stage_x<NT>(x_s, p.x + k_begin, p.ldx, p.M, k_len, p.x_stride, SPLIT_WARPS * 32);
    __syncthreads();
    st.run(x_s + (size_t)g * p.x_stride + c_begin * 32 + t * 8, p.x_stride);
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[((warp * NT + n) * 4 + e) * 32 + lane] = st.acc[n][e];
    __syncthreads();
    // element e of column block n of lane (g, t): row g (e < 2) or g+8, token n*8 + 2t + (e & 1)
    for (int o = threadIdx.x; o < NT * 4 * 32; o += SPLIT_WARPS * 32) {
        const int ne = o >> 5, l2 = o & 31, n = ne >> 2, e = ne & 3;
        const int row = f0 + (l2 >> 2) + 8 * (e >> 1), tok = n * 8 + 2 * (l2 & 3) + (e & 1);
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < SPLIT_WARPS; ++w) v += red[((w * NT + n) * 4 + e) * 32 + l2];
        if (row < p.N && tok < p.M) {
            if (p.bias && blockIdx.y == 0) v += p.bias[row];
            p.partial[((size_t)blockIdx.y * p.M + tok) * p.N + row] = v;
        }
    }
}

int x_pitch(int K) {
    int x_stride = K + 8;                                   // pitch in bytes = 64 mod 128: 16-byte row loads
    while ((x_stride * 2) % 128 != 64) x_stride += 8;       // of two neighbouring rows hit different banks
    return x_stride;
}

template <typename Kernel>
int reserve(Kernel kernel, size_t smem, size_t& configured, const char* what) {
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "%s: cannot reserve %zu bytes of shared memory: %s", what, smem, cudaGetErrorString(e));
        configured = smem;
    }
    return MLB_OK;
}

int check_operands(const char* what, const void* x, long long ldx, const void* w, long long ldw, int M, int K) {
    if (M <= 0 || M > 16 || K <= 0) return fail(MLB_UNSUPPORTED_SIZE, "%s: M=%d must be 1..16 (K=%d)", what, M, K);
    if (K % 32 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K)
        return fail(MLB_UNSUPPORTED_SIZE, "%s: K=%d must be a multiple of 32 and the row pitches multiples of 8", what, K);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(MLB_UNSUPPORTED_SIZE, "%s: operands must be 16-byte aligned", what);
    return MLB_OK;
}

}  // namespace

// largest K whose activations (16 token rows) still fit beside the reduction buffer
MLB_EXPORT int mlb_gemv_fused_max_k() { return 6144; }

// out[M, I] (bf16) = silu(x Wg^T) * (x Wu^T), Wg = W rows [0, I), Wu = W rows [up_offset, up_offset + I)
MLB_EXPORT int mlb_gemv_silu(const void* x, long long ldx, const void* w, long long ldw, int w_rows, int up_offset, void* out,
                             long long ldo, int M, int I, int K, cudaStream_t stream) {
    int status = check_operands("gemv_silu", x, ldx, w, ldw, M, K);
    if (status != MLB_OK) return status;
    if (I <= 0 || up_offset < I || up_offset + I > w_rows || ldo < I || !out)
        return fail(MLB_INVALID_ARGUMENT, "gemv_silu: gate rows [0, %d) and up rows [%d, %d) must lie inside the weight's %d rows", I, up_offset, up_offset + I, w_rows);
    if (K > mlb_gemv_fused_max_k()) return fail(MLB_UNSUPPORTED_SIZE, "gemv_silu: K=%d is more than %d", K, mlb_gemv_fused_max_k());
    const int nt = M <= 8 ? 1 : 2;
    SiluParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldx, ldw, ldo, M, I, K, up_offset, x_pitch(K)};
    const size_t smem = (size_t)nt * 8 * p.x_stride * 2 + (size_t)SILU_WARPS * 2 * nt * 4 * 32 * sizeof(float);
    static size_t configured1_on[MAX_DEVICES] = {0}, configured2_on[MAX_DEVICES] = {0};   // per device, as the attribute is
    size_t& configured1 = configured1_on[device_index()];
    size_t& configured2 = configured2_on[device_index()];
    const unsigned blocks = (unsigned)((I + 15) / 16);
    if (nt == 1) {
        status = reserve(gemv_silu_kernel<1>, smem, configured1, "gemv_silu");
        if (status != MLB_OK) return status;
        launch_kernel(gemv_silu_kernel<1>, blocks, SILU_WARPS * 32, smem, stream, p);
    } else {
        status = reserve(gemv_silu_kernel<2>, smem, configured2, "gemv_silu");
        if (status != MLB_OK) return status;
        launch_kernel(gemv_silu_kernel<2>, blocks, SILU_WARPS * 32, smem, stream, p);
    }
    return check_launch("gemv_silu");
}

// q_out[M, NH*D] = rotate(x Wq^T + bq); keys (rotated) and values go to slot positions[t] of sequence
// token_seq[t] in the paged cache.  rotate: 1 = split-half rotation over the whole head, 0 = none.
// head_dim must be a multiple of 16.
MLB_EXPORT int mlb_gemv_qkv_rope(const void* x, long long ldx, const void* w, long long ldw, const float* bias,
                                 const int* positions, const int* token_seq, const int* block_table, int max_blocks,
                                 const float* inv_freq, int rotate, void* q_out, void* pages, int num_pages, int page_size,
                                 int M, int K, int num_heads, int num_kv_heads, int head_dim, int* error_flag,
                                 cudaStream_t stream) {
    int status = check_operands("gemv_qkv_rope", x, ldx, w, ldw, M, K);
    if (status != MLB_OK) return status;
    if (num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || head_dim % 16 != 0)
        return fail(MLB_UNSUPPORTED_SIZE, "gemv_qkv_rope: head_dim %d must be a multiple of 16", head_dim);
    if (K > mlb_gemv_fused_max_k()) return fail(MLB_UNSUPPORTED_SIZE, "gemv_qkv_rope: K=%d is more than %d", K, mlb_gemv_fused_max_k());
    if (!positions || !q_out || (rotate && !inv_freq)) return fail(MLB_INVALID_ARGUMENT, "gemv_qkv_rope: positions, output or frequencies missing");
    if (pages && (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || !block_table || !token_seq))
        return fail(MLB_INVALID_ARGUMENT, "gemv_qkv_rope: cache geometry missing");
    const int nt = M <= 8 ? 1 : 2;
    QkvParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, ldx, ldw, M, K, x_pitch(K), positions, token_seq, block_table,
                inv_freq, (__nv_bfloat16*)q_out, (__nv_bfloat16*)pages, max_blocks, num_pages, page_size, num_heads, num_kv_heads,
                head_dim, rotate ? 1 : 0, error_flag};
    const size_t smem = (size_t)nt * 8 * p.x_stride * 2 + (size_t)QKV_WARPS * nt * 4 * 32 * sizeof(float);
    static size_t configured1_on[MAX_DEVICES] = {0}, configured2_on[MAX_DEVICES] = {0};   // per device, as the attribute is
    size_t& configured1 = configured1_on[device_index()];
    size_t& configured2 = configured2_on[device_index()];
    const unsigned blocks = (unsigned)((num_heads + 2 * num_kv_heads) * (head_dim / 16));
    if (nt == 1) {
        status = reserve(gemv_qkv_rope_kernel<1>, smem, configured1, "gemv_qkv_rope");
        if (status != MLB_OK) return status;
        launch_kernel(gemv_qkv_rope_kernel<1>, blocks, QKV_WARPS * 32, smem, stream, p);
    } else {
        status = reserve(gemv_qkv_rope_kernel<2>, smem, configured2, "gemv_qkv_rope");
        if (status != MLB_OK) return status;
        launch_kernel(gemv_qkv_rope_kernel<2>, blocks, QKV_WARPS * 32, smem, stream, p);
    }
    return check_launch("gemv_qkv_rope");
}

// partial[splits, M, N] (fp32) = x * W^T cut into `splits` K ranges of k_per_cta elements (a multiple of 32;
// bias, if given, goes into split 0); their sum over the splits, taken in order by the consumer, is the product.
MLB_EXPORT int mlb_gemv_split(const void* x, long long ldx, const void* w, long long ldw, int w_rows, const float* bias,
                              float* partial, int M, int N, int K, int splits, int k_per_cta, cudaStream_t stream) {
    int status = check_operands("gemv_split", x, ldx, w, ldw, M, K);
    if (status != MLB_OK) return status;
    if (N <= 0 || N > w_rows || !partial) return fail(MLB_INVALID_ARGUMENT, "gemv_split: bad output");
    if (splits < 1 || splits > 65535 || k_per_cta <= 0 || k_per_cta % 32 != 0 || (long long)splits * k_per_cta < K)
        return fail(MLB_INVALID_ARGUMENT, "gemv_split: %d splits of %d do not cover K=%d in steps of 32", splits, k_per_cta, K);
    if (k_per_cta > mlb_gemv_fused_max_k()) return fail(MLB_UNSUPPORTED_SIZE, "gemv_split: a K range of %d per CTA is more than %d", k_per_cta, mlb_gemv_fused_max_k());
    const int nt = M <= 8 ? 1 : 2;
    SplitParams p{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, partial, ldx, ldw, M, N, K, k_per_cta, x_pitch(k_per_cta)};
    const size_t smem = (size_t)nt * 8 * p.x_stride * 2 + (size_t)SPLIT_WARPS * nt * 4 * 32 * sizeof(float);
    static size_t configured1_on[MAX_DEVICES] = {0}, configured2_on[MAX_DEVICES] = {0};   // per device, as the attribute is
    size_t& configured1 = configured1_on[device_index()];
    size_t& configured2 = configured2_on[device_index()];
    const dim3 grid((unsigned)((N + 15) / 16), (unsigned)splits);
    if (nt == 1) {
        status = reserve(gemv_split_kernel<1>, smem, configured1, "gemv_split");
        if (status != MLB_OK) return status;
        launch_kernel(gemv_split_kernel<1>, grid, SPLIT_WARPS * 32, smem, stream, p);
    } else {
        status = reserve(gemv_split_kernel<2>, smem, configured2, "gemv_split");
        if (status != MLB_OK) return status;
        launch_kernel(gemv_split_kernel<2>, grid, SPLIT_WARPS * 32, smem, stream, p);
    }
    return check_launch("gemv_split");
}
