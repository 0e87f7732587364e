// Weight-streaming bf16 products for steps of up to 128 tokens on the fifth-generation tensor cores:
//     y[M, N] = x[M, K] * W[N, K]^T           1 <= M <= 128
//
// With so few tokens a product is bound by reading W once from HBM; the kernel is built around that stream.
// It is computed transposed: the 128-row side of tcgen05.mma is a tile of 128 WEIGHT rows, its N side the
// step's tokens (padded to a multiple of 16; the padding is zero-filled by TMA and never stored).  Per CTA:
//     warp 0      TMA producer (one thread): [64 x 64] boxes of W and one [tokens x 64] box of x per stage into
//                 a ring; the W boxes of the first ring-full are issued BEFORE the dependency wait, since no
//                 kernel of a step writes weights: they travel while the kernel in front still runs
//     warp 1      allocates tensor memory; one thread issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32 in
//                 TMEM), four K=16 steps per stage; tcgen05.commit hands the stage back to the producer
//     warps 2-5   epilogue: tcgen05.ld (lane = weight row, column = token), then one of
//                   PARTIAL   fp32 partial results [split, M, N] (bias in split 0): the K range of a product with
//                             few row tiles is cut over CTAs and the kernel that consumes the result adds the
//                             partial tiles in split order (no atomics: the sum never depends on timing)
//                   SILU      the tile stacks 64 gate rows on 64 up rows of a fused [gate; up] weight; the two
//                             halves meet through shared memory and silu(gate) * up is stored as bf16
// CTAs are persistent over work items (row tile, K split) with a double-buffered accumulator, so a product
// with more tiles than SMs (the LM head) drains one tile while the next one streams.
//
// The reference sends these products to the library whatever the token count (hipBLASLt,
// src/ops/optimized.cpp:349-403; bf16_qkv_projection :713-735, bf16_ffn_impl :644-692) and runs the
// activation (src/ops/optimized.cpp:676-683) as a kernel of its own.
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel raises the error flag, stops
// waiting, lets its copies in flight land, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>
#include <mutex>
#include <unordered_map>

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int BLOCK_W = 128;                 // weight rows per tile (MMA M)
constexpr int HALF_W = 64;                   // rows per TMA box of W
constexpr int BLOCK_K = 64;                  // bf16 per stage row: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BLOCK_W * BLOCK_K * 2;
constexpr int HALF_TILE_BYTES = HALF_W * BLOCK_K * 2;
constexpr int MAX_STAGES = 12;
constexpr int MAX_TOKENS = 128;
constexpr int THREADS = 192;
constexpr int SPIN_LIMIT = 1 << 22;          // polls of up to 1 us each
constexpr int XBUF_BYTES = 2 * 16 * HALF_W * 4;   // two exchange buffers of 16 tokens x 64 rows fp32
// Ring depth unless the caller asks for another.  Measured in whole decode steps of 12 to 128 tokens (the step's
// other kernels around it, started early behind it): six stages beat both a ring small enough to leave half of
// the SM's shared memory to the next kernel's CTAs (by 2 to 8 %) and the deepest ring that fits (by 1 to 12 %).
constexpr int USUAL_STAGES = 6;

enum Mode : int { MODE_PARTIAL = 0, MODE_SILU = 1 };

struct StreamParams {
    float* partial;            // PARTIAL: [splits, M, N] fp32
    const float* bias;         // PARTIAL: [N] or null, added in split 0
    __nv_bfloat16* out;        // SILU: [M, ldo] activations
    long long ldo;
    int* error_flag;
    int M, N, K;
    int tok_tile;              // tokens padded to a multiple of 16
    int k_blocks, k_blocks_per_split, splits;
    int n_tiles, items;
    int stages;
    int mode;
    int up_offset;             // SILU: first up row of the fused weight
    int tmem_cols;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One poll; the hint lets the hardware park the thread until the phase completes or the time (ns) is up.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
    return ok != 0;
}
// false when the bound was hit (the caller gives up and the flag tells the host)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
    for (int i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (error_flag) atomicExch(error_flag, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
// K-major operand tile, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);      // start address, 16-byte units
    d |= (uint64_t)1 << 16;                       // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset: next group of 8 rows
    d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
    return d;
}
// kind::f16 instruction descriptor: fp32 accumulator, bf16 A and B, both K-major, M = 128
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BLOCK_W >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 16 accumulator columns of this thread's lane, no wait: several may be in flight before tmem_wait()
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t addr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// the four epilogue warps among themselves
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ float silu(float g) {
    // g * sigmoid(g) (src/ops/ops.cpp:72-76, 760-785) in its one-branch form: for very negative g the
    // exponential overflows to +inf and the quotient is -0, which is the limit.  No branch and the fast
    // exponential and reciprocal: the epilogue of a one-tile CTA is not hidden behind anything, and the
    // result is rounded to bf16 right away.
    return __fdividef(g, 1.0f + __expf(-g));
}

// Where the 128 rows of work item `tile` come from: two boxes of 64 weight rows.
//   PARTIAL   rows [128 t, 128 t + 64) and [128 t + 64, 128 t + 128)
//   SILU      gate rows [64 t, 64 t + 64) and up rows up_offset + the same
__device__ __forceinline__ void tile_rows(const StreamParams& p, int tile, int& row_a, int& row_b) {
    if (p.mode == MODE_SILU) { row_a = tile * HALF_W; row_b = p.up_offset + tile * HALF_W; }
    else { row_a = tile * BLOCK_W; row_b = tile * BLOCK_W + HALF_W; }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, StreamParams p) {
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int epilogue_ok_s[2];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // operand ring, 1024-byte aligned as the swizzle pattern requires; the exchange buffers follow it
    const uint32_t ring = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t b_bytes = (uint32_t)p.tok_tile * BLOCK_K * 2;
    const uint32_t stage_bytes = (uint32_t)A_TILE_BYTES + b_bytes;
    float* xbuf = reinterpret_cast<float*>(smem_dyn + (ring - smem_u32(smem_dyn)) + (size_t)p.stages * stage_bytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 4);          // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            // cursor over this CTA's (item, k-block) sequence
            int item = blockIdx.x, kb = 0, kb_end = 0, row_a = 0, row_b = 0;
            auto open_item = [&]() {
                if (item >= p.items) return;
                const int split = item / p.n_tiles;
                kb = split * p.k_blocks_per_split;
                kb_end = min(p.k_blocks, kb + p.k_blocks_per_split);
                tile_rows(p, item % p.n_tiles, row_a, row_b);
            };
            auto advance = [&]() {
                if (++kb >= kb_end) { item += gridDim.x; open_item(); }
            };
            open_item();
            // the weights of the first ring-full: nothing of this step writes them, so they need not wait
            int issued = 0;
            {
                int item0 = item, kb0 = kb, kb_end0 = kb_end, ra0 = row_a, rb0 = row_b;
                while (issued < p.stages && item < p.items) {
                    const uint32_t dst = ring + (uint32_t)issued * stage_bytes, bar = smem_u32(&full_bar[issued]);
                    mbar_expect_tx(bar, stage_bytes);
                    tma_load_2d(dst, &map_w, kb * BLOCK_K, row_a, bar);
                    tma_load_2d(dst + HALF_TILE_BYTES, &map_w, kb * BLOCK_K, row_b, bar);
                    ++issued;
                    advance();
                }
                item = item0; kb = kb0; kb_end = kb_end0; row_a = ra0; row_b = rb0;
            }
            pdl_wait();                                   // the activations come from the kernel in front
            for (int i = 0; i < issued; ++i) {
                tma_load_2d(ring + (uint32_t)i * stage_bytes + A_TILE_BYTES, &map_x, kb * BLOCK_K, 0, smem_u32(&full_bar[i]));
                advance();
            }
            uint32_t it = (uint32_t)issued;
            bool ok = true;
            while (item < p.items) {
                lag_point();
                const int s = it % p.stages;
                const uint32_t round = it / p.stages;
                if (!mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, p.error_flag, 51)) { ok = false; break; }
                const uint32_t dst = ring + (uint32_t)s * stage_bytes, bar = smem_u32(&full_bar[s]);
                mbar_expect_tx(bar, stage_bytes);
                tma_load_2d(dst, &map_w, kb * BLOCK_K, row_a, bar);
                tma_load_2d(dst + HALF_TILE_BYTES, &map_w, kb * BLOCK_K, row_b, bar);
                tma_load_2d(dst + A_TILE_BYTES, &map_x, kb * BLOCK_K, 0, bar);
                ++it;
                advance();
            }
            if (!ok) {
                // given up: let the copies already issued land before the shared memory is handed back
                const uint32_t first = it > (uint32_t)p.stages ? it - p.stages : 0;
                for (uint32_t j = first; j < it; ++j)
                    mbar_wait(smem_u32(&full_bar[j % p.stages]), (j / p.stages) & 1, nullptr, 0);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(p.tok_tile);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++local) {
                const uint32_t buf = local & 1, use = local >> 1;
                const int split = item / p.n_tiles;
                const int kb_begin = split * p.k_blocks_per_split, kb_end = min(p.k_blocks, kb_begin + p.k_blocks_per_split);
                // the epilogue must have drained this buffer (the first use of each buffer passes at once)
                if (!mbar_wait(smem_u32(&acc_empty[buf]), (use & 1) ^ 1, p.error_flag, 52)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * (uint32_t)p.tok_tile;
                for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    lag_point();
                    const int s = it % p.stages;
                    if (!mbar_wait(smem_u32(&full_bar[s]), (it / p.stages) & 1, p.error_flag, 53)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = ring + (uint32_t)s * stage_bytes;
                    const uint64_t adesc = umma_desc(a_addr), bdesc = umma_desc(a_addr + A_TILE_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k)      // 16 elements of K = 32 bytes = 2 address units
                        umma(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb_begin || k > 0) ? 1u : 0u);
                    umma_commit(smem_u32(&empty_bar[s]));          // the stage is free once these MMAs have read it
                }
                if (ok) umma_commit(smem_u32(&acc_full[buf]));     // accumulator complete
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;                     // the TMEM lanes this warp may read
        uint32_t local = 0;
        bool ok = true;
        pdl_wait();                                       // nothing is stored while the kernel in front may still read it
        for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++local) {
            lag_point();
            const uint32_t buf = local & 1, use = local >> 1;
            const int tile = item % p.n_tiles, split = item / p.n_tiles;
            // ONE thread waits for the accumulator and tells the other 127: the four warps go on, or give up,
            // together (they meet at barriers below).  Two flags in turn: the next item's answer is written only
            // after everybody has read this one's and passed the following barrier.
            if (warp == 2 && lane == 0) epilogue_ok_s[local & 1] = mbar_wait(smem_u32(&acc_full[buf]), use & 1, p.error_flag, 54) ? 1 : 0;
            epilogue_sync();
            ok = epilogue_ok_s[local & 1] != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lane_addr = tmem_base + buf * (uint32_t)p.tok_tile + ((uint32_t)(quarter * 32) << 16);
            const int limit = min(p.tok_tile, (p.M + 15) / 16 * 16);       // columns that hold tokens
            if (p.mode == MODE_PARTIAL) {
                const int f = tile * BLOCK_W + quarter * 32 + lane;          // this thread's output feature
                const float bias = (p.bias && split == 0 && f < p.N) ? p.bias[f] : 0.0f;
                float* dst = p.partial + (size_t)split * p.M * p.N + f;
                // two 16-column loads in turn: the next one travels while this one is stored
                uint32_t a[16], b[16];
                tmem_ld16_nowait(lane_addr, a);
                tmem_wait();
                for (int c = 0; c < limit; c += 32) {
                    if (c + 16 < limit) tmem_ld16_nowait(lane_addr + (uint32_t)(c + 16), b);
                    if (f < p.N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c + j < p.M) dst[(size_t)(c + j) * p.N] = __uint_as_float(a[j]) + bias;
                    }
                    tmem_wait();
                    if (c + 16 >= limit) break;
                    if (c + 32 < limit) tmem_ld16_nowait(lane_addr + (uint32_t)(c + 32), a);
                    if (f < p.N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c + 16 + j < p.M) dst[(size_t)(c + 16 + j) * p.N] = __uint_as_float(b[j]) + bias;
                    }
                    tmem_wait();
                }
            } else if (p.mode == MODE_SILU) {
                // lanes 0-63 of the tile hold gate rows, lanes 64-127 the up rows of the same features.  Of every 16
                // tokens the gate side finishes the first 8 and the up side the last 8; each sends the other what
                // it needs through shared memory (token-major, so both sides touch consecutive words).
                const bool up_side = quarter >= 2;
                const int i = (quarter & 1) * 32 + lane;                  // row within the 64
                const int f = tile * HALF_W + i;
                auto finish = [&](const uint32_t (&raw)[16], int c, int chunk) {
                    float* xb = xbuf + (size_t)(chunk & 1) * 16 * HALF_W;
                    if (up_side) {                      // the gate side finishes tokens 0..7 of the chunk and needs their up values
#pragma unroll
                        for (int j = 0; j < 8; ++j) xb[j * HALF_W + i] = __uint_as_float(raw[j]);
                    } else {
#pragma unroll
                        for (int j = 8; j < 16; ++j) xb[j * HALF_W + i] = __uint_as_float(raw[j]);
                    }
                    epilogue_sync();
                    if (f >= p.N) return;
                    // all eight results first, without conditions, so that their exponentials and reciprocals overlap;
                    // then the stores
                    float res[8];
                    if (!up_side) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) res[j] = silu(__uint_as_float(raw[j])) * xb[j * HALF_W + i];
                    } else {
#pragma unroll
                        for (int j = 0; j < 8; ++j) res[j] = silu(xb[(8 + j) * HALF_W + i]) * __uint_as_float(raw[8 + j]);
                    }
                    __nv_bfloat16* dst = p.out + (size_t)(c + (up_side ? 8 : 0)) * p.ldo + f;
                    const int left = p.M - c - (up_side ? 8 : 0);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (j < left) dst[(size_t)j * p.ldo] = __float2bfloat16_rn(res[j]);
                };
                uint32_t a[16], b[16];
                tmem_ld16_nowait(lane_addr, a);
                tmem_wait();
                int chunk = 0;
                for (int c = 0; c < limit; c += 32, chunk += 2) {
                    if (c + 16 < limit) tmem_ld16_nowait(lane_addr + (uint32_t)(c + 16), b);
                    finish(a, c, chunk);
                    tmem_wait();
                    if (c + 16 >= limit) break;
                    if (c + 32 < limit) tmem_ld16_nowait(lane_addr + (uint32_t)(c + 32), a);
                    finish(b, c + 16, chunk + 1);
                    tmem_wait();
                }
                epilogue_sync();          // the exchange buffers are free for the next tile
            }
            // this warp is done reading the buffer: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    }
}

// --------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    return fn;
}

// Tensor maps are pure functions of (address, shape, pitch, box): weights and a step's scratch buffers keep
// their addresses, so the encoded maps are kept and a launch costs no driver call.
struct MapKey {
    const void* base; long long rows, cols, ld; int box_rows;
    bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.base;
        for (long long v : {k.rows, k.cols, k.ld, (long long)k.box_rows}) h = h * 1000003u ^ (size_t)v;
        return h;
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> map_cache;
std::mutex map_mutex;

// rows x cols bf16 matrix, row pitch `ld` elements; box = box_rows x 64 columns, 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    const MapKey key{base, rows, cols, ld, box_rows};
    {
        std::lock_guard<std::mutex> lock(map_mutex);
        auto found = map_cache.find(key);
        if (found != map_cache.end()) { *map = found->second; return MLB_OK; }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MLB_CUDA_ERROR, "gemm_stream: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MLB_CUDA_ERROR, "gemm_stream: cuTensorMapEncodeTiled failed with %d", (int)r);
    std::lock_guard<std::mutex> lock(map_mutex);
    if (map_cache.size() > 8192) map_cache.clear();
    map_cache.emplace(key, *map);
    return MLB_OK;
}

int check_operands(const void* x, long long ldx, const void* w, long long ldw, int M, int K) {
    if (M <= 0 || M > MAX_TOKENS || K <= 0) return fail(MLB_UNSUPPORTED_SIZE, "gemm_stream: M=%d must be 1..%d (K=%d)", M, MAX_TOKENS, K);
    if (!x || !w) return fail(MLB_INVALID_ARGUMENT, "gemm_stream: operands missing");
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K)
        return fail(MLB_UNSUPPORTED_SIZE, "gemm_stream: K=%d and the row pitches (%lld, %lld) must be multiples of 8 elements", K, ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(MLB_UNSUPPORTED_SIZE, "gemm_stream: operands must be 16-byte aligned");
    return MLB_OK;
}

int launch(StreamParams& p, const void* x, long long ldx, const void* w, long long ldw, int w_rows, int stages, cudaStream_t stream) {
    p.tok_tile = (p.M + 15) / 16 * 16;
    p.k_blocks = (p.K + BLOCK_K - 1) / BLOCK_K;
    if (p.splits < 1) p.splits = 1;
    if (p.splits > p.k_blocks) p.splits = p.k_blocks;
    p.k_blocks_per_split = (p.k_blocks + p.splits - 1) / p.splits;
    p.splits = (p.k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;      // no empty split
    p.items = p.n_tiles * p.splits;
    const int ctas = p.items < sm_count() ? p.items : sm_count();
    // a CTA with one work item needs one accumulator; with more, two, so that a tile drains while the next one runs
    p.tmem_cols = 32;
    while (p.tmem_cols < (p.items > ctas ? 2 : 1) * p.tok_tile) p.tmem_cols *= 2;
    const int stage_bytes = A_TILE_BYTES + p.tok_tile * BLOCK_K * 2;
    const int xbuf = p.mode == MODE_PARTIAL ? 0 : XBUF_BYTES;
    int most = (200 * 1024 - xbuf) / stage_bytes;
    if (most > MAX_STAGES) most = MAX_STAGES;
    int usual = USUAL_STAGES;
    if (p.items > ctas) usual = most;                 // a long stream (the head): as much in flight as fits
    if (usual > most) usual = most;
    p.stages = stages > 0 ? (stages < most ? stages : most) : usual;
    if (p.stages < 2) p.stages = 2;
    const size_t smem = (size_t)p.stages * stage_bytes + xbuf + 1024;

    CUtensorMap map_w, map_x;
    int status = make_map(&map_w, w, w_rows, p.K, ldw, HALF_W);
    if (status != MLB_OK) return status;
    status = make_map(&map_x, x, p.M, p.K, ldx, p.tok_tile);
    if (status != MLB_OK) return status;

    static bool configured_on[MAX_DEVICES] = {false};          // the attribute belongs to the device
    bool& configured = configured_on[device_index()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(220 * 1024));
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "gemm_stream: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    launch_kernel(gemm_stream_kernel, dim3(ctas), dim3(THREADS), smem, stream, map_w, map_x, p);
    return check_launch("gemm_stream");
}

}  // namespace

MLB_EXPORT int mlb_gemm_stream_max_tokens() { return MAX_TOKENS; }

// partial[splits', M, N] (fp32) = x[M, K] * W[:N, K]^T cut into K ranges of whole 64-element blocks (bias, if
// given, goes into split 0); splits' = mlb_gemm_stream_splits(K, splits) <= splits is what the kernel really
// uses (no empty range).  Their sum over the splits, taken in order by the consumer, is the product.
// x and W are bf16 with row pitches ldx, ldw (elements); K and the pitches must be multiples of 8 and the
// bases 16-byte aligned (TMA).  stages: 0 = the usual ring depth (six stages; as deep as fits for a product with more tiles than SMs).
MLB_EXPORT int mlb_gemm_stream_splits(int K, int splits) {
    const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    if (splits < 1) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    const int per = (k_blocks + splits - 1) / splits;
    return (k_blocks + per - 1) / per;
}

MLB_EXPORT int mlb_gemm_stream(const void* x, long long ldx, const void* w, long long ldw, int w_rows, const float* bias,
                               float* partial, int M, int N, int K, int splits, int stages, int* error_flag,
                               cudaStream_t stream) {
    int status = check_operands(x, ldx, w, ldw, M, K);
    if (status != MLB_OK) return status;
    if (N <= 0 || N > w_rows || !partial) return fail(MLB_INVALID_ARGUMENT, "gemm_stream: bad output (N=%d of %d weight rows)", N, w_rows);
    StreamParams p{};
    p.partial = partial; p.bias = bias; p.error_flag = error_flag; p.M = M; p.N = N; p.K = K;
    p.mode = MODE_PARTIAL; p.splits = splits;
    p.n_tiles = (N + BLOCK_W - 1) / BLOCK_W;
    return launch(p, x, ldx, w, ldw, w_rows, stages, stream);
}

// out[M, I] (bf16) = silu(x Wg^T) * (x Wu^T) with Wg = W rows [0, I) and Wu = W rows [up_offset, up_offset + I).
MLB_EXPORT int mlb_gemm_stream_silu(const void* x, long long ldx, const void* w, long long ldw, int w_rows, int up_offset,
                                    void* out, long long ldo, int M, int I, int K, int stages, int* error_flag,
                                    cudaStream_t stream) {
    int status = check_operands(x, ldx, w, ldw, M, K);
    if (status != MLB_OK) return status;
    if (I <= 0 || up_offset < I || up_offset + I > w_rows || ldo < I || !out)
        return fail(MLB_INVALID_ARGUMENT, "gemm_stream_silu: gate rows [0, %d) and up rows [%d, %d) must lie inside the weight's %d rows",
                    I, up_offset, up_offset + I, w_rows);
    StreamParams p{};
    p.out = (__nv_bfloat16*)out; p.ldo = ldo; p.error_flag = error_flag; p.M = M; p.N = I; p.K = K;
    p.mode = MODE_SILU; p.splits = 1; p.up_offset = up_offset;
    p.n_tiles = (I + HALF_W - 1) / HALF_W;
    return launch(p, x, ldx, w, ldw, w_rows, stages, stream);
}
