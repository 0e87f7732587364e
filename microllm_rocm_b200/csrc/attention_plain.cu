// Plain attention over the paged cache: any mix of prompt portions and decoded tokens.
//
// One warp per (query token, query head).  The query at absolute position `pos` of its
// sequence sees keys lo..pos, lo = max(0, pos - window + 1) for a windowed layer and 0
// otherwise; keys beyond `pos` are never read (the reference computes no masked scores
// either: src/ops/ops.cpp:2343-2384).  Query head h uses kv head h / (NH/NKV)
// (ops.cpp:2357; consecutive query heads share one).  score = dot(q, k) * scale with the
// scale applied after the dot product (ops.cpp:2365-2369); softmax and the value sum are
// fp32 (ops.cpp:1624-1661 for the cached case).
//
// Keys are walked in tiles of 32 whose edges sit at multiples of 32 of the ABSOLUTE
// position, with a running maximum and sum.  The order of every addition therefore depends
// only on (pos, window), not on how the prompt was cut into steps, on the other requests of
// the batch, or on which physical pages hold the keys: in the fp32 path the same token gets
// bit-identical output however it is scheduled.  This kernel is the whole fp32 path's
// attention and the reference beside the tensor-core kernels.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

struct AttnParams {
    const void* q;           // [T, NH*D]
    const void* pages;       // [num_pages, 2, NKV, page_size, D]
    void* out;               // [T, NH*D]
    const int* positions;    // [T]
    const int* token_seq;    // [T]
    const int* block_table;  // [A, max_blocks]
    int max_blocks, num_pages, page_size;
    int tokens, num_heads, num_kv_heads, head_dim;
    int window;              // 0: all earlier keys
    float scale;
    int* error_flag;
};

template <typename QT, typename KVT, typename OutT>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_plain_kernel(AttnParams p) {
    pdl_prologue();
    __shared__ float q_s[WARPS][MAX_D];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)p.tokens * p.num_heads) return;     // whole warp leaves together
    const int t = (int)(item / p.num_heads), h = (int)(item % p.num_heads);
    const int D = p.head_dim;
    const int kvh = h / (p.num_heads / p.num_kv_heads);
    const int pos = p.positions[t];
    const int seq = p.token_seq[t];
    const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;

    const QT* qrow = (const QT*)p.q + ((size_t)t * p.num_heads + h) * D;
    for (int c = lane; c < D; c += 32) q_s[warp][c] = to_f32(qrow[c]);
    __syncwarp();

    constexpr int PER_LANE = MAX_D / 32;
    float acc[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    const size_t page_stride = (size_t)2 * p.num_kv_heads * p.page_size * D;
    const size_t v_offset = (size_t)p.num_kv_heads * p.page_size * D;
    const int* table = p.block_table + (size_t)seq * p.max_blocks;

    for (int base = (lo / 32) * 32; base <= pos; base += 32) {
        const int kp = base + lane;
        bool valid = kp >= lo && kp <= pos;
        long long k_off = -1;
        if (valid) {
            const int block = kp / p.page_size;
            const int page = block < p.max_blocks ? table[block] : -1;
            if (page < 0 || page >= p.num_pages) {
                if (p.error_flag) atomicExch(p.error_flag, 2);
                valid = false;
            } else {
                k_off = (long long)((size_t)page * page_stride + ((size_t)kvh * p.page_size + kp % p.page_size) * D);
            }
        }
        float s = -INFINITY;
        if (valid) {
            const KVT* krow = (const KVT*)p.pages + k_off;
            float dot = 0.0f;
            for (int c = 0; c < D; ++c) dot = fmaf(q_s[warp][c], to_f32(krow[c]), dot);
            s = dot * p.scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;                     // no readable key in this tile
        const float prob = valid ? expf(s - m_new) : 0.0f;
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + warp_sum(prob);
        m = m_new;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) acc[i] *= corr;
        const unsigned valid_mask = __ballot_sync(0xffffffffu, valid);
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, prob, j);
            const long long off_j = __shfl_sync(0xffffffffu, k_off, j);
            if (!((valid_mask >> j) & 1u)) continue;          // uniform over the warp
            const KVT* vrow = (const KVT*)p.pages + off_j + v_offset;
#pragma unroll
            for (int i = 0; i < PER_LANE; ++i) {
                const int c = lane + 32 * i;
                if (c < D) acc[i] = fmaf(pj, to_f32(vrow[c]), acc[i]);
            }
        }
    }
    OutT* orow = (OutT*)p.out + ((size_t)t * p.num_heads + h) * D;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const int c = lane + 32 * i;
        if (c < D) orow[c] = from_f32<OutT>(acc[i] * inv);
    }
}

}  // namespace

MLB_EXPORT int mlb_paged_attention_plain(const void* q, int q_dtype, const void* pages, int kv_dtype, void* out,
                                         int out_dtype, const int* positions, const int* token_seq,
                                         const int* block_table, int max_blocks, int num_pages, int page_size,
                                         int tokens, int num_heads, int num_kv_heads, int head_dim, int window,
                                         float scale, int* error_flag, cudaStream_t stream) {
    if (tokens < 0 || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_plain: bad head counts %d/%d", num_heads, num_kv_heads);
    if (head_dim <= 0 || head_dim > MAX_D)
        return fail(MLB_UNSUPPORTED_SIZE, "paged_attention_plain: head_dim %d not in 1..%d", head_dim, MAX_D);
    if (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0)
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_plain: bad cache geometry");
    if (tokens == 0) return MLB_OK;
    AttnParams p{q, pages, out, positions, token_seq, block_table, max_blocks, num_pages, page_size,
                 tokens, num_heads, num_kv_heads, head_dim, window, scale, error_flag};
    const long long items = (long long)tokens * num_heads;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    if (q_dtype == MLB_F32 && kv_dtype == MLB_F32 && out_dtype == MLB_F32)
        launch_kernel(paged_attention_plain_kernel<float, float, float>, blocks, WARPS * 32, 0, stream, p);
    else if (q_dtype == MLB_BF16 && kv_dtype == MLB_BF16 && out_dtype == MLB_BF16)
        launch_kernel(paged_attention_plain_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, blocks, WARPS * 32, 0, stream, p);
    else if (q_dtype == MLB_F32 && kv_dtype == MLB_BF16 && out_dtype == MLB_F32)
        launch_kernel(paged_attention_plain_kernel<float, __nv_bfloat16, float>, blocks, WARPS * 32, 0, stream, p);
    else if (q_dtype == MLB_BF16 && kv_dtype == MLB_BF16 && out_dtype == MLB_F32)
        launch_kernel(paged_attention_plain_kernel<__nv_bfloat16, __nv_bfloat16, float>, blocks, WARPS * 32, 0, stream, p);
    else
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_plain: unsupported dtypes %d/%d/%d", q_dtype, kv_dtype, out_dtype);
    return check_launch("paged_attention_plain");
}
