// The few-token weight-streaming kernel itself (see gemv_bf16.cu for the design); shared by
// the regular entry point and by the entry point that brings its own scratch memory.
#pragma once

#include "common.cuh"

namespace mlb_gemv {

using namespace mlb;


constexpr int WARPS = 4;
constexpr int ROWS_PER_CTA = WARPS * 16;
constexpr int BATCH = 4;                       // 32-wide K chunks per register set (two sets in flight)

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const __nv_bfloat16* p) {
    // weights are read once: do not let them push the activations out of L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float silu(float g) {
    // two-branch sigmoid, as the reference's activation (src/ops/ops.cpp:72-76)
    if (g >= 0.0f) return g / (1.0f + expf(-g));
    const float e = expf(g);
    return g * e / (1.0f + e);
}

struct GemvParams {
    const __nv_bfloat16* x;      // [M, ldx]
    const __nv_bfloat16* w;      // [rows, ldw]
    float* partial;              // [splits, M, N] fp32 (null when out is used)
    void* out;                   // dual: bf16 [M, ldo]
    const float* bias;           // [N] or null; added by split 0
    long long ldx, ldw, ldo;
    int M, N, K;
    int k_per_split;             // multiple of 32
    int x_stride;                // shared-memory row pitch of x in elements
    int up_offset;
};

// NT: 8-token column blocks (1: M <= 8, 2: M <= 16)
template <int NT, bool DUAL>
__global__ void __launch_bounds__(WARPS * 32) gemv_bf16_kernel(GemvParams p) {
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* x_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);       // [NT*8][x_stride]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int k_begin = blockIdx.y * p.k_per_split;
    const int k_end = min(p.K, k_begin + p.k_per_split);
    const int k_len = max(0, k_end - k_begin);
    const int chunks = k_len / 32;

    const int row0 = blockIdx.x * ROWS_PER_CTA + warp * 16;
    const bool active = row0 < p.N;
    // rows past the end read the last row (never stored)
    const int ra = min(row0 + g, p.N - 1), rb = min(row0 + g + 8, p.N - 1);
    const __nv_bfloat16* wa = p.w + (size_t)ra * p.ldw + k_begin + t * 8;
    const __nv_bfloat16* wb = p.w + (size_t)rb * p.ldw + k_begin + t * 8;
    const __nv_bfloat16* ua = DUAL ? wa + (size_t)p.up_offset * p.ldw : nullptr;
    const __nv_bfloat16* ub = DUAL ? wb + (size_t)p.up_offset * p.ldw : nullptr;
    const __nv_bfloat16* xs = x_s + (size_t)g * p.x_stride + t * 8;

    // Two register sets of BATCH chunks each: while one is multiplied the other is in flight.
    struct Batch { uint4 a[BATCH], b[BATCH], ua[DUAL ? BATCH : 1], ub[DUAL ? BATCH : 1]; };
    Batch set0, set1;
    auto load_batch = [&](Batch& s, int c0) {
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            if (c0 + u < chunks) {
                s.a[u] = ldg_stream(wa + (size_t)(c0 + u) * 32);
                s.b[u] = ldg_stream(wb + (size_t)(c0 + u) * 32);
                if (DUAL) {
                    s.ua[u] = ldg_stream(ua + (size_t)(c0 + u) * 32);
                    s.ub[u] = ldg_stream(ub + (size_t)(c0 + u) * 32);
                }
            }
        }
    };

    float acc[NT][4], acc_u[DUAL ? NT : 1][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[n][e] = 0.0f; if (DUAL) acc_u[n][e] = 0.0f; }
    auto mma_batch = [&](const Batch& s, int c0) {
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            if (c0 + u < chunks) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)n * 8 * p.x_stride + (c0 + u) * 32);
                    mma_bf16(acc[n], s.a[u].x, s.b[u].x, s.a[u].y, s.b[u].y, xv.x, xv.y);
                    mma_bf16(acc[n], s.a[u].z, s.b[u].z, s.a[u].w, s.b[u].w, xv.z, xv.w);
                    if (DUAL) {
                        mma_bf16(acc_u[n], s.ua[u].x, s.ub[u].x, s.ua[u].y, s.ub[u].y, xv.x, xv.y);
                        mma_bf16(acc_u[n], s.ua[u].z, s.ub[u].z, s.ua[u].w, s.ub[u].w, xv.z, xv.w);
                    }
                }
            }
        }
    };

    // The weights are never written by a kernel: the loads of both register sets go out before
    // this kernel waits for its predecessor, and before the activations are staged.
    if (active) { load_batch(set0, 0); load_batch(set1, BATCH); }
    pdl_wait();

    // stage this CTA's slice of the activations; rows beyond M are zero
    const int vec_per_row = k_len / 8;
    for (int i = threadIdx.x; i < NT * 8 * vec_per_row; i += WARPS * 32) {
        const int r = i / vec_per_row, c = (i % vec_per_row) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < p.M) v = *reinterpret_cast<const uint4*>(p.x + (size_t)r * p.ldx + k_begin + c);
        *reinterpret_cast<uint4*>(x_s + (size_t)r * p.x_stride + c) = v;
    }
    __syncthreads();
    if (!active) return;

    for (int c0 = 0; c0 < chunks; c0 += 2 * BATCH) {
        mma_batch(set0, c0);
        load_batch(set0, c0 + 2 * BATCH);
        mma_batch(set1, c0 + BATCH);
        load_batch(set1, c0 + 3 * BATCH);
    }

    // accumulator element e of column block n: row g (e < 2) or g+8, token n*8 + 2t + (e & 1)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = row0 + g + 8 * (e >> 1), tok = n * 8 + 2 * t + (e & 1);
            if (row >= p.N || tok >= p.M) continue;
            if (DUAL) {
                ((__nv_bfloat16*)p.out)[(size_t)tok * p.ldo + row] = __float2bfloat16_rn(silu(acc[n][e]) * acc_u[n][e]);
            } else {
                float v = acc[n][e];
                if (p.bias && blockIdx.y == 0) v += p.bias[row];
                p.partial[((size_t)blockIdx.y * p.M + tok) * p.N + row] = v;
            }
        }
}


}  // namespace mlb_gemv
