// Bias + rotary position encoding + key/value store, in one pass over the fused QKV
// projection output.
//
//   q' = rotate(q + bq, pos)            -> q_out[T, NH*D]            (fp32 or bf16)
//   k' = rotate(k + bk, pos), v + bv    -> pages[page, 0|1, kvh, slot, :] through the block table
//
// Rotation as the reference computes it (src/ops/ops.cpp:861-879, with bias :913-940, per
// row positions :1086-1115): for pair i, angle = float(pos) * base^(-2 i / D) in fp32,
// (a, b) -> (a cos - b sin, a sin + b cos); split-half pairs element i with i + D/2.  The
// inverse frequencies come in as a table (computed once with the same fp32 expression), so
// another rotary variant (partial width, interleaved pairs, scaled frequencies) is a
// different table and flag, not a different kernel.  Values and rotation stay fp32; only
// the store converts.  The reference keeps separate kernels for rotation, bias and cache
// store (basic_kernels.hip:456-592, 927-983) and copies K/V into a capacity-strided cache
// (src/model/model.cpp:129-164); here the cache is paged.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

struct RopeKvParams {
    const float* qkv;        // [T, ld]  columns: NH*D of q, NKV*D of k, NKV*D of v
    long long ld;
    int n_partials;          // the projection may arrive as partial results of a split product,
    long long partial_stride;  // `partial_stride` elements apart: they are added here, in order
    const float* bias;       // [(NH+2NKV)*D] or null
    const int* positions;    // [T] absolute position of each token
    const int* token_seq;    // [T] index of the token's sequence in this batch
    const int* block_table;  // [A, max_blocks] physical page of each logical block, -1 if none
    int max_blocks;
    const float* inv_freq;   // [rot_dim/2]
    int rot_dim;
    int interleaved;         // 0: pairs (i, i+rot/2); 1: pairs (2i, 2i+1)
    void* q_out;             // [T, NH*D]
    void* pages;             // [num_pages, 2, NKV, page_size, D] or null (read-only run)
    int num_pages, page_size;
    int tokens, num_heads, num_kv_heads, head_dim;
    int* error_flag;         // set to 1 when a token maps to no valid page
    const float2* cos_sin;   // [T, rot_dim/2] (cos, sin) of every token's angles, or null: computed here
};

template <typename QT, typename KVT>
__global__ void rope_kv_kernel(RopeKvParams p) {
    pdl_prologue();
    const int half = p.head_dim / 2;
    const int heads_all = p.num_heads + 2 * p.num_kv_heads;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)p.tokens * heads_all * half;
    if (idx >= total) return;
    const int i = (int)(idx % half);
    const int head = (int)((idx / half) % heads_all);
    const int t = (int)(idx / ((long long)half * heads_all));

    const bool is_q = head < p.num_heads;
    const bool is_k = !is_q && head < p.num_heads + p.num_kv_heads;
    const bool is_v = !is_q && !is_k;
    if (!is_q && p.pages == nullptr) return;

    // which two elements of the head this thread owns
    int e0, e1;
    bool rotate = false;
    const int rot_half = p.rot_dim / 2;
    if (!is_v && i < rot_half) {
        rotate = true;
        if (p.interleaved) { e0 = 2 * i; e1 = 2 * i + 1; }
        else               { e0 = i;     e1 = i + rot_half; }
    } else if (!is_v) {
        e0 = p.rot_dim + 2 * (i - rot_half); e1 = e0 + 1;
    } else {
        e0 = 2 * i; e1 = e0 + 1;
    }
    const size_t col = (size_t)head * p.head_dim;
    const float* src = p.qkv + (size_t)t * p.ld + col;
    float a = src[e0], b = src[e1];
    for (int k = 1; k < p.n_partials; ++k) {
        a += src[(size_t)k * p.partial_stride + e0];
        b += src[(size_t)k * p.partial_stride + e1];
    }
    if (p.bias) { a += p.bias[col + e0]; b += p.bias[col + e1]; }
    const int pos = p.positions[t];
    if (rotate) {
        const float angle = (float)pos * p.inv_freq[i];
        float s, c;
        sincosf(angle, &s, &c);
        const float ra = a * c - b * s;
        const float rb = a * s + b * c;
        a = ra; b = rb;
    }
    if (is_q) {
        QT* dst = (QT*)p.q_out + (size_t)t * p.num_heads * p.head_dim + col;
        dst[e0] = from_f32<QT>(a);
        dst[e1] = from_f32<QT>(b);
        return;
    }
    const int kvh = is_k ? head - p.num_heads : head - p.num_heads - p.num_kv_heads;
    const int block = pos / p.page_size, slot = pos % p.page_size;
    int page = -1;
    if (pos >= 0 && block < p.max_blocks) page = p.block_table[(size_t)p.token_seq[t] * p.max_blocks + block];
    if (page < 0 || page >= p.num_pages) {
        if (p.error_flag) atomicExch(p.error_flag, 1);
        return;                                   // never write outside the pool
    }
    KVT* dst = (KVT*)p.pages +
               ((((size_t)page * 2 + (is_v ? 1 : 0)) * p.num_kv_heads + kvh) * p.page_size + slot) * p.head_dim;
    dst[e0] = from_f32<KVT>(a);
    dst[e1] = from_f32<KVT>(b);
}

__device__ __forceinline__ void store4(float* dst, const float (&v)[4]) {
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* dst, const float (&v)[4]) {
    uint2 packed;
    *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(dst) = packed;
}

// Split-half rotation over the whole head (the model's own case), four pairs per thread:
// elements i..i+3 and i+D/2..i+D/2+3 travel as 16-byte pieces.  V heads copy eight elements.
template <typename QT, typename KVT>
__global__ void rope_kv_split_half_x4_kernel(RopeKvParams p) {
    // Everything that no kernel of this step writes is fetched and computed before the wait: the position, the
    // bias, the page of the cache, and the angles' sines and cosines when they are computed here.
    pdl_launch_dependents();
    const int half = p.head_dim / 2, quads = half / 4;
    const int heads_all = p.num_heads + 2 * p.num_kv_heads;
    // grid (tokens, blocks of a token's items): no 64-bit divisions on the way to (token, head, element)
    const int item = blockIdx.y * blockDim.x + threadIdx.x;
    const bool in_range = item < heads_all * quads;
    const int i = (item % quads) * 4;
    const int head = in_range ? item / quads : 0;
    const int t = blockIdx.x;
    const bool is_q = head < p.num_heads;
    const bool is_v = head >= p.num_heads + p.num_kv_heads;
    const bool working = in_range && (is_q || p.pages != nullptr);
    const size_t col = (size_t)head * p.head_dim;
    float4 ba = make_float4(0.f, 0.f, 0.f, 0.f), bb = ba;
    float sn[4] = {0.f, 0.f, 0.f, 0.f}, cs[4] = {1.f, 1.f, 1.f, 1.f};
    int pos = 0, page = -1;
    if (working) {
        if (p.bias) {
            ba = *reinterpret_cast<const float4*>(p.bias + col + i);
            bb = *reinterpret_cast<const float4*>(p.bias + col + i + half);
        }
        pos = p.positions[t];
        if (!is_v && !p.cos_sin) {
            const float4 f = *reinterpret_cast<const float4*>(p.inv_freq + i);
            const float fr[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) sincosf((float)pos * fr[k], &sn[k], &cs[k]);
        }
        if (!is_q) {
            const int block = pos / p.page_size;
            if (pos >= 0 && block < p.max_blocks) page = p.block_table[(size_t)p.token_seq[t] * p.max_blocks + block];
        }
    }
    pdl_wait();
    if (!working) return;
    if (!is_v && p.cos_sin) {
        // A step's table, made once for all layers and heads.  It is written by a kernel of THIS step (in the first
        // layer by the kernel launched just before this one), so it may only be read behind the wait: kernels
        // that sit in front of their waits can all be resident while the table's kernel has not run yet.
        const float4 u = *reinterpret_cast<const float4*>(p.cos_sin + (size_t)t * half + i);
        const float4 v = *reinterpret_cast<const float4*>(p.cos_sin + (size_t)t * half + i + 2);
        cs[0] = u.x; sn[0] = u.y; cs[1] = u.z; sn[1] = u.w; cs[2] = v.x; sn[2] = v.y; cs[3] = v.z; sn[3] = v.w;
    }
    const float* src = p.qkv + (size_t)t * p.ld + col;
    // V has nothing to rotate: its two pieces are simply elements i.. and i+half..
    float4 a = *reinterpret_cast<const float4*>(src + i), b = *reinterpret_cast<const float4*>(src + i + half);
    for (int k = 1; k < p.n_partials; ++k) {
        const float4 a2 = *reinterpret_cast<const float4*>(src + (size_t)k * p.partial_stride + i);
        const float4 b2 = *reinterpret_cast<const float4*>(src + (size_t)k * p.partial_stride + i + half);
        a.x += a2.x; a.y += a2.y; a.z += a2.z; a.w += a2.w;
        b.x += b2.x; b.y += b2.y; b.z += b2.z; b.w += b2.w;
    }
    a.x += ba.x; a.y += ba.y; a.z += ba.z; a.w += ba.w;
    b.x += bb.x; b.y += bb.y; b.z += bb.z; b.w += bb.w;
    float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
    if (!is_v) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float ra = av[k] * cs[k] - bv[k] * sn[k], rb = av[k] * sn[k] + bv[k] * cs[k];
            av[k] = ra; bv[k] = rb;
        }
    }
    if (is_q) {
        QT* dst = (QT*)p.q_out + (size_t)t * p.num_heads * p.head_dim + col;
        store4(dst + i, av);
        store4(dst + i + half, bv);
        return;
    }
    const int kvh = is_v ? head - p.num_heads - p.num_kv_heads : head - p.num_heads;
    const int slot = pos % p.page_size;
    if (page < 0 || page >= p.num_pages) {
        if (p.error_flag) atomicExch(p.error_flag, 1);
        return;
    }
    KVT* dst = (KVT*)p.pages +
               ((((size_t)page * 2 + (is_v ? 1 : 0)) * p.num_kv_heads + kvh) * p.page_size + slot) * p.head_dim;
    store4(dst + i, av);
    store4(dst + i + half, bv);
}

// (cos, sin) of position[t] * inv_freq[i]: the same fp32 expressions as in the rotation kernels
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cos_sin, int tokens, int half) {
    pdl_prologue();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)tokens * half) return;
    const int t = (int)(idx / half), i = (int)(idx % half);
    float s, c;
    sincosf((float)positions[t] * inv_freq[i], &s, &c);
    cos_sin[idx] = make_float2(c, s);
}

}  // namespace

// cos_sin[T, half] = (cos, sin)(positions[t] * inv_freq[i]): one table per step serves every layer's rotation
MLB_EXPORT int mlb_rope_table(const int* positions, const float* inv_freq, float* cos_sin, int tokens, int half,
                              cudaStream_t stream) {
    if (tokens < 0 || half <= 0) return fail(MLB_INVALID_ARGUMENT, "rope_table: bad sizes");
    if (tokens == 0) return MLB_OK;
    const long long total = (long long)tokens * half;
    launch_kernel(rope_table_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, positions, inv_freq, (float2*)cos_sin, tokens, half);
    return check_launch("rope_table");
}

MLB_EXPORT int mlb_rope_kv_write(const float* qkv, long long ld, int n_partials, long long partial_stride,
                                 const float* bias, const int* positions,
                                 const int* token_seq, const int* block_table, int max_blocks,
                                 const float* inv_freq, int rot_dim, int interleaved, void* q_out, int q_dtype,
                                 void* pages, int kv_dtype, int num_pages, int page_size, int tokens,
                                 int num_heads, int num_kv_heads, int head_dim, int* error_flag,
                                 const float* cos_sin, cudaStream_t stream) {
    if (tokens < 0 || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || head_dim % 2 != 0)
        return fail(MLB_INVALID_ARGUMENT, "rope_kv_write: bad head sizes");
    if (rot_dim < 0 || rot_dim > head_dim || rot_dim % 2 != 0)
        return fail(MLB_INVALID_ARGUMENT, "rope_kv_write: rot_dim %d must be even and <= head_dim %d", rot_dim, head_dim);
    if (ld < (long long)(num_heads + 2 * num_kv_heads) * head_dim)
        return fail(MLB_INVALID_ARGUMENT, "rope_kv_write: row pitch smaller than the fused width");
    if (pages && (page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || !block_table || !token_seq))
        return fail(MLB_INVALID_ARGUMENT, "rope_kv_write: cache geometry missing");
    if (tokens == 0) return MLB_OK;
    if (n_partials < 1) return fail(MLB_INVALID_ARGUMENT, "rope_kv_write: n_partials must be at least 1");
    RopeKvParams p{qkv, ld, n_partials, partial_stride, bias, positions, token_seq, block_table, max_blocks, inv_freq, rot_dim, interleaved,
                   q_out, pages, num_pages, page_size, tokens, num_heads, num_kv_heads, head_dim, error_flag, nullptr};
    const int key = q_dtype * 2 + kv_dtype;
    // the model's own case in 16-byte pieces: split-half over the whole head, eight-element alignment
    const bool wide = rot_dim == head_dim && !interleaved && head_dim % 8 == 0 && ld % 4 == 0 && partial_stride % 4 == 0 &&
                      (uintptr_t)q_out % 16 == 0 && (!pages || (uintptr_t)pages % 16 == 0) && (uintptr_t)qkv % 16 == 0 && (!bias || (uintptr_t)bias % 16 == 0) && (uintptr_t)inv_freq % 16 == 0;
    if (wide) {
        if (cos_sin && (uintptr_t)cos_sin % 16 == 0 && head_dim % 16 == 0) p.cos_sin = (const float2*)cos_sin;
        const int per_token = (num_heads + 2 * num_kv_heads) * (head_dim / 8);
        const int threads4 = per_token >= 256 ? 256 : ((per_token + 31) / 32) * 32;
        const dim3 blocks4((unsigned)tokens, (unsigned)((per_token + threads4 - 1) / threads4));
        switch (key) {
            case MLB_F32 * 2 + MLB_F32: launch_kernel(rope_kv_split_half_x4_kernel<float, float>, blocks4, threads4, 0, stream, p); break;
            case MLB_BF16 * 2 + MLB_BF16: launch_kernel(rope_kv_split_half_x4_kernel<__nv_bfloat16, __nv_bfloat16>, blocks4, threads4, 0, stream, p); break;
            case MLB_F32 * 2 + MLB_BF16: launch_kernel(rope_kv_split_half_x4_kernel<float, __nv_bfloat16>, blocks4, threads4, 0, stream, p); break;
            case MLB_BF16 * 2 + MLB_F32: launch_kernel(rope_kv_split_half_x4_kernel<__nv_bfloat16, float>, blocks4, threads4, 0, stream, p); break;
            default: return fail(MLB_INVALID_ARGUMENT, "rope_kv_write: unknown dtypes %d/%d", q_dtype, kv_dtype);
        }
        return check_launch("rope_kv_write");
    }
    const long long total = (long long)tokens * (num_heads + 2 * num_kv_heads) * (head_dim / 2);
    const unsigned blocks = (unsigned)((total + 255) / 256);
    switch (key) {
        case MLB_F32 * 2 + MLB_F32: launch_kernel(rope_kv_kernel<float, float>, blocks, 256, 0, stream, p); break;
        case MLB_BF16 * 2 + MLB_BF16: launch_kernel(rope_kv_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 256, 0, stream, p); break;
        case MLB_F32 * 2 + MLB_BF16: launch_kernel(rope_kv_kernel<float, __nv_bfloat16>, blocks, 256, 0, stream, p); break;
        case MLB_BF16 * 2 + MLB_F32: launch_kernel(rope_kv_kernel<__nv_bfloat16, float>, blocks, 256, 0, stream, p); break;
        default: return fail(MLB_INVALID_ARGUMENT, "rope_kv_write: unknown dtypes %d/%d", q_dtype, kv_dtype);
    }
    return check_launch("rope_kv_write");
}
