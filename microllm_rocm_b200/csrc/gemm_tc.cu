// bf16 matrix products on the fifth-generation tensor cores:  y[M,N] = x[M,K] * W[N,K]^T.
//
// Always computed transposed ("swap-AB"): the 128-row side of tcgen05.mma is a tile of 128
// WEIGHT rows (output features) and its N side is a tile of 16..256 TOKENS.  A decode step
// with 8 tokens and a prompt portion of 2,048 run the same kernel; only the token tile
// differs.  Per CTA:
//     warp 0   TMA producer: cp.async.bulk.tensor loads of a [128 x 64] weight tile and a
//              [tokens x 64] activation tile per stage, 128-byte swizzled, no multicast
//     warp 1   allocates tensor memory, then one elected thread issues tcgen05.mma
//              (kind::f16, bf16 x bf16 -> fp32 in TMEM), four K=16 steps per stage, and
//              tcgen05.commit hands the stage back to the producer
//     warps 2-5  epilogue: tcgen05.ld brings the accumulator back (lane = feature, column =
//              token), then bias / residual add / SiLU(gate)*up and the store
// The K range may be split over CTAs (blockIdx.z); partial tiles go to scratch memory and the
// CTA that finishes last adds them in split order, so the result does not depend on timing.
// With DUAL the CTA loads two weight tiles (gate rows n.. and up rows up_offset+n..) against
// the same activations into two accumulators and stores silu(gate)*up.
//
// This replaces the library product that the reference calls for its projections
// (hipBLASLt, src/ops/optimized.cpp:349-403, bf16 x bf16 with fp32 accumulation) and the
// separate bias, residual and activation kernels around it (src/model/model.cpp:332-335,
// src/ops/optimized.cpp:676-683).
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel raises the error
// flag, stops waiting, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>
#include <cstdlib>

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int BLOCK_W = 128;                 // weight rows per CTA (MMA M)
constexpr int BLOCK_K = 64;                  // bf16 per stage row: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BLOCK_W * BLOCK_K * 2;
constexpr int MAX_STAGES = 12;
constexpr int THREADS = 192;
constexpr int SPIN_LIMIT = 1 << 24;
constexpr int MAX_SPLITS = 32;

struct GemmParams {
    void* out;                 // [M, ldo] fp32 or bf16
    const float* bias;         // [N] or null
    float* partial;            // [splits, M, N] fp32 scratch (split-K)
    int* tickets;              // [n_tiles * m_tiles], zero between launches
    int* error_flag;
    long long ldo;
    int M, N, K;
    int tok_tile;              // tokens per CTA: multiple of 16, at most 256
    int k_blocks, k_blocks_per_split, splits;
    int stages;
    int out_bf16;              // 0: fp32, 1: bf16
    int accumulate;            // out += result (fp32 out only)
    int dual;                  // 1: silu(gate) * up; W rows n (gate) and up_offset + n (up); N counts gate rows
    int up_offset;
    int tmem_cols;
    int debug;                 // measurement aid: bit 0 skips the MMAs, bit 1 skips the loads (results are garbage)
    int reduce_here;           // split-K: 1 = the last CTA adds the partial tiles up; 0 = the caller's next kernel does
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
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
// kind::f16 instruction descriptor: fp32 accumulator, bf16 A and B, both K-major
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
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 accumulator columns of this thread's lane, no wait: several may be in flight before tmem_wait()
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float silu(float g) {
    // two-branch sigmoid, as the reference's activation (src/ops/ops.cpp:72-76)
    if (g >= 0.0f) return g / (1.0f + expf(-g));
    const float e = expf(g);
    return g * e / (1.0f + e);
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_bar[MAX_STAGES], empty_bar[MAX_STAGES], accum_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ int ticket_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BLOCK_W;                  // first feature (weight row) of the tile
    const int tok0 = blockIdx.y * p.tok_tile;             // first token of the tile
    const int kb_begin = blockIdx.z * p.k_blocks_per_split;
    const int kb_end = min(p.k_blocks, kb_begin + p.k_blocks_per_split);
    const int num_kb = max(0, kb_end - kb_begin);

    // operand ring, 1024-byte aligned as the swizzle pattern requires
    const uint32_t ring = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t b_bytes = (uint32_t)p.tok_tile * BLOCK_K * 2;
    const uint32_t a_bytes = p.dual ? 2u * A_TILE_BYTES : (uint32_t)A_TILE_BYTES;
    const uint32_t stage_bytes = a_bytes + b_bytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&accum_bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {                                      // tensor memory for the accumulator(s)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();                  // barriers and tensor memory were set up while the previous kernel ran

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            for (int i = 0; i < num_kb; ++i) {
                const int s = i % p.stages;
                const uint32_t round = (uint32_t)(i / p.stages);
                if (i >= p.stages && !mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, p.error_flag, 11)) break;
                const uint32_t dst = ring + (uint32_t)s * stage_bytes;
                const uint32_t bar = smem_u32(&full_bar[s]);
                const int k = (kb_begin + i) * BLOCK_K;
                if (p.debug & 2) {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
                    continue;
                }
                mbar_expect_tx(bar, stage_bytes);
                tma_load_2d(dst, &map_w, k, n0, bar);
                if (p.dual) tma_load_2d(dst + A_TILE_BYTES, &map_w, k, p.up_offset + n0, bar);
                tma_load_2d(dst + a_bytes, &map_x, k, tok0, bar);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(p.tok_tile);
            bool ok = true;
            for (int i = 0; i < num_kb && ok; ++i) {
                const int s = i % p.stages;
                ok = mbar_wait(smem_u32(&full_bar[s]), (uint32_t)(i / p.stages) & 1, p.error_flag, 12);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = ring + (uint32_t)s * stage_bytes;
                const uint32_t b_addr = a_addr + a_bytes;
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    if (p.debug & 1) break;
                    const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    const uint64_t bdesc = umma_desc(b_addr + k * UMMA_K * 2);
                    umma(tmem_base, umma_desc(a_addr + k * UMMA_K * 2), bdesc, idesc, acc);
                    if (p.dual)
                        umma(tmem_base + (uint32_t)p.tok_tile, umma_desc(a_addr + A_TILE_BYTES + k * UMMA_K * 2), bdesc, idesc, acc);
                }
                umma_commit(smem_u32(&empty_bar[s]));     // the stage is free once these MMAs have read it
            }
            umma_commit(smem_u32(&accum_bar));            // accumulator complete
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;                     // the TMEM lanes this warp may read
        const int f = n0 + quarter * 32 + lane;           // this thread's output feature
        bool ok = true;
        if (num_kb > 0) ok = mbar_wait(smem_u32(&accum_bar), 0, p.error_flag, 13);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const float bias = (p.bias && f < p.N) ? p.bias[f] : 0.0f;
        for (int c = 0; c < p.tok_tile && ok; c += 16) {
            if (tok0 + c >= p.M) break;                   // uniform over the warp
            float v[16];
            if (num_kb > 0) {
                tmem_ld16(lane_addr + (uint32_t)c, v);
                if (p.dual) {
                    float u[16];
                    tmem_ld16(lane_addr + (uint32_t)(p.tok_tile + c), u);
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = silu(v[j]) * u[j];
                }
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            }
            if (f >= p.N) continue;
            if (p.splits > 1) {
                float* dst = p.partial + ((size_t)blockIdx.z * p.M + tok0 + c) * p.N + f;
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (tok0 + c + j < p.M) dst[(size_t)j * p.N] = v[j];
                continue;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int tok = tok0 + c + j;
                if (tok >= p.M) break;
                const float r = v[j] + bias;
                if (p.out_bf16) ((__nv_bfloat16*)p.out)[(size_t)tok * p.ldo + f] = __float2bfloat16_rn(r);
                else {
                    float* o = (float*)p.out + (size_t)tok * p.ldo + f;
                    *o = p.accumulate ? *o + r : r;
                }
            }
        }
    }

    // ---------------------------------------------------------------- split-K: the last CTA adds up
    if (p.splits > 1 && p.reduce_here) {
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) ticket_s = atomicAdd(p.tickets + blockIdx.y * gridDim.x + blockIdx.x, 1);
        __syncthreads();
        if (ticket_s == p.splits - 1) {
            __threadfence();
            if (threadIdx.x == 0) p.tickets[blockIdx.y * gridDim.x + blockIdx.x] = 0;
            const int rows = min(p.tok_tile, p.M - tok0), cols = min(BLOCK_W, p.N - n0);
            for (int i = threadIdx.x; i < rows * cols; i += THREADS) {
                const int tok = tok0 + i / cols, f = n0 + i % cols;
                const float* src = p.partial + (size_t)tok * p.N + f;
                const size_t step = (size_t)p.M * p.N;
                float acc = 0.0f;
                for (int s0 = 0; s0 < p.splits; s0 += 8) {      // eight loads in flight; the sum keeps split order
                    float part[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) part[k] = s0 + k < p.splits ? __ldcg(src + (size_t)(s0 + k) * step) : 0.0f;
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc += part[k];
                }
                if (p.bias) acc += p.bias[f];
                if (p.out_bf16) ((__nv_bfloat16*)p.out)[(size_t)tok * p.ldo + f] = __float2bfloat16_rn(acc);
                else {
                    float* o = (float*)p.out + (size_t)tok * p.ldo + f;
                    *o = p.accumulate ? *o + acc : acc;
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
    }
}

// --------------------------------------------------------------------------------- persistent variant
// For products with many output tiles (prompt portions): each CTA stays on its SM and walks
// tiles blockIdx.x, blockIdx.x + gridDim.x, ...  The accumulator is DOUBLE-BUFFERED in tensor
// memory, so while the four epilogue warps drain tile i (tcgen05.ld, activation, stores) the
// MMA warp already runs tile i+1, and the TMA warp runs ahead of both across tile borders.
// Consecutive tiles share a weight tile and differ in the token tile, so the weights of a
// wave come from L2.  No split over K here (there are tiles enough).
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          GemmParams p, int n_tiles, int m_tiles) {
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = n_tiles * m_tiles;
    const uint32_t ring = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    const uint32_t b_bytes = (uint32_t)p.tok_tile * BLOCK_K * 2;
    const uint32_t a_bytes = p.dual ? 2u * A_TILE_BYTES : (uint32_t)A_TILE_BYTES;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    const uint32_t acc_cols = (uint32_t)(p.dual ? 2 * p.tok_tile : p.tok_tile);     // columns of one accumulator buffer

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
    pdl_wait();

    if (warp == 0) {
        // ---------------------------------------------------------------- producer
        if (lane == 0) {
            uint32_t it = 0;                                  // k-blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int n0 = (tile / m_tiles) * BLOCK_W, tok0 = (tile % m_tiles) * p.tok_tile;
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const int s = it % p.stages;
                    const uint32_t round = it / p.stages;
                    if (round > 0 && !mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, p.error_flag, 21)) { ok = false; break; }
                    const uint32_t dst = ring + (uint32_t)s * stage_bytes;
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    mbar_expect_tx(bar, stage_bytes);
                    const int k = kb * BLOCK_K;
                    tma_load_2d(dst, &map_w, k, n0, bar);
                    if (p.dual) tma_load_2d(dst + A_TILE_BYTES, &map_w, k, p.up_offset + n0, bar);
                    tma_load_2d(dst + a_bytes, &map_x, k, tok0, bar);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(p.tok_tile);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const uint32_t buf = local & 1, use = local >> 1;
                // the epilogue must have drained this buffer (first use of each buffer passes at once)
                if (!mbar_wait(smem_u32(&acc_empty[buf]), (use & 1) ^ 1, p.error_flag, 22)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * acc_cols;
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const int s = it % p.stages;
                    if (!mbar_wait(smem_u32(&full_bar[s]), (it / p.stages) & 1, p.error_flag, 23)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = ring + (uint32_t)s * stage_bytes;
                    const uint32_t b_addr = a_addr + a_bytes;
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        const uint64_t bdesc = umma_desc(b_addr + k * UMMA_K * 2);
                        umma(acc, umma_desc(a_addr + k * UMMA_K * 2), bdesc, idesc, accumulate);
                        if (p.dual)
                            umma(acc + (uint32_t)p.tok_tile, umma_desc(a_addr + A_TILE_BYTES + k * UMMA_K * 2), bdesc, idesc, accumulate);
                    }
                    umma_commit(smem_u32(&empty_bar[s]));
                }
                if (ok) umma_commit(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const uint32_t buf = local & 1, use = local >> 1;
            const int n0 = (tile / m_tiles) * BLOCK_W, tok0 = (tile % m_tiles) * p.tok_tile;
            const int f = n0 + quarter * 32 + lane;
            ok = mbar_wait(smem_u32(&acc_full[buf]), use & 1, p.error_flag, 24);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lane_addr = tmem_base + buf * acc_cols + ((uint32_t)(quarter * 32) << 16);
            const float bias = (p.bias && f < p.N) ? p.bias[f] : 0.0f;
            for (int c = 0; c < p.tok_tile; c += 32) {
                if (tok0 + c >= p.M) break;
                uint32_t raw[32], raw_u[32];
                tmem_ld32_nowait(lane_addr + (uint32_t)c, raw);
                if (p.dual) tmem_ld32_nowait(lane_addr + (uint32_t)(p.tok_tile + c), raw_u);
                tmem_wait();
                if (f >= p.N) continue;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int tok = tok0 + c + j;
                    if (tok >= p.M || c + j >= p.tok_tile) break;
                    float r = __uint_as_float(raw[j]);
                    if (p.dual) r = silu(r) * __uint_as_float(raw_u[j]);
                    r += bias;
                    if (p.out_bf16) ((__nv_bfloat16*)p.out)[(size_t)tok * p.ldo + f] = __float2bfloat16_rn(r);
                    else {
                        float* o = (float*)p.out + (size_t)tok * p.ldo + f;
                        *o = p.accumulate ? *o + r : r;
                    }
                }
            }
            // this warp is done reading the buffer: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[buf])) : "memory");
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

// rows x cols bf16 matrix, row pitch `ld` elements; box = box_rows x 64 columns, 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MLB_CUDA_ERROR, "gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MLB_CUDA_ERROR, "gemm_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
    return MLB_OK;
}

}  // namespace

// Scratch for a split product: `splits * M * N` floats and one int per output tile.
MLB_EXPORT int mlb_gemm_tc_max_splits() { return MAX_SPLITS; }

// y[M, N] = x[M, K] * W[N, K]^T (+ bias) (+ y when accumulate), or, with dual,
// y[M, N] = silu(x Wg^T) * (x Wu^T) where Wg = W rows [0, N) and Wu = W rows [up_offset, up_offset + N).
// x and W are bf16 with row pitches ldx, ldw (elements); K and the pitches must be multiples of 8
// and the bases 16-byte aligned (TMA).  tok_tile: tokens per CTA, a multiple of 16 up to 256
// (128 with dual).  splits > 1 cuts K over CTAs into `partial` [splits, M, N]; with reduce_here the
// last CTA of a tile adds them into `out` (needs zeroed `tickets`), without it `out` is not
// written and the caller's next kernel sums the partial tiles in split order.
MLB_EXPORT int mlb_gemm_tc(const void* x, long long ldx, const void* w, long long ldw, int w_rows, const float* bias,
                           void* out, long long ldo, int out_bf16, int accumulate, int dual, int up_offset, int M, int N,
                           int K, int tok_tile, int splits, int reduce_here, int stages, float* partial, int* tickets,
                           int* error_flag, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0) return fail(MLB_INVALID_ARGUMENT, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K)
        return fail(MLB_UNSUPPORTED_SIZE, "gemm_tc: K=%d and the row pitches (%lld, %lld) must be multiples of 8 elements", K, ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        return fail(MLB_UNSUPPORTED_SIZE, "gemm_tc: operands must be 16-byte aligned");
    if (tok_tile < 16 || tok_tile % 16 != 0 || tok_tile > (dual ? 128 : 256))
        return fail(MLB_UNSUPPORTED_SIZE, "gemm_tc: token tile %d must be a multiple of 16 up to %d", tok_tile, dual ? 128 : 256);
    if (accumulate && out_bf16) return fail(MLB_INVALID_ARGUMENT, "gemm_tc: accumulation needs an fp32 output");
    if (dual && (up_offset < 0 || up_offset + N > w_rows)) return fail(MLB_INVALID_ARGUMENT, "gemm_tc: up rows outside the weight");
    if (dual && splits > 1) return fail(MLB_INVALID_ARGUMENT, "gemm_tc: the activation is not linear, a dual product cannot be split over K");
    if (splits < 1 || splits > MAX_SPLITS || (splits > 1 && (!partial || (reduce_here && !tickets))))
        return fail(MLB_INVALID_ARGUMENT, "gemm_tc: bad split arguments (1..%d, scratch required)", MAX_SPLITS);
    if (M == 0) return MLB_OK;

    CUtensorMap map_w, map_x;
    int status = make_map(&map_w, w, w_rows, K, ldw, BLOCK_W);
    if (status != MLB_OK) return status;
    status = make_map(&map_x, x, M, K, ldx, tok_tile);
    if (status != MLB_OK) return status;

    GemmParams p{};
    p.out = out; p.bias = bias; p.partial = partial; p.tickets = tickets; p.error_flag = error_flag; p.ldo = ldo;
    p.M = M; p.N = N; p.K = K; p.tok_tile = tok_tile;
    p.k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    p.k_blocks_per_split = (p.k_blocks + splits - 1) / splits;
    p.splits = splits;
    {
        static int debug = -1;
        if (debug < 0) { const char* e = getenv("MLB_GEMM_DEBUG"); debug = e ? atoi(e) : 0; }
        p.debug = debug;
    }
    p.out_bf16 = out_bf16; p.accumulate = accumulate; p.dual = dual; p.up_offset = up_offset; p.reduce_here = reduce_here;
    int cols = dual ? 2 * tok_tile : tok_tile;
    p.tmem_cols = 32;
    while (p.tmem_cols < cols) p.tmem_cols *= 2;
    const int stage_bytes = (dual ? 2 : 1) * A_TILE_BYTES + tok_tile * BLOCK_K * 2;
    // small token tiles (weight streaming): several CTAs share an SM, so that one streams while
    // another sets up or stores; large ones take the whole SM for a deeper ring
    // With more CTAs than SMs, several share an SM (one streams while another sets up or
    // stores) and each gets a third of the shared memory; a grid of at most one CTA per SM gives
    // each the whole SM for a deeper ring.  `stages` > 0 overrides the choice.
    const long long ctas = (long long)((N + BLOCK_W - 1) / BLOCK_W) * ((M + tok_tile - 1) / tok_tile) * splits;
    const int budget = (ctas > 148 && tok_tile <= 128) ? 72 * 1024 : 200 * 1024;
    p.stages = stages > 0 ? stages : budget / stage_bytes;
    if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
    if (p.stages < 2) p.stages = 2;
    if ((size_t)p.stages * stage_bytes > 216 * 1024) p.stages = (216 * 1024) / stage_bytes;
    if (p.stages > p.k_blocks_per_split) p.stages = p.k_blocks_per_split < 1 ? 1 : p.k_blocks_per_split;
    const size_t smem = (size_t)p.stages * stage_bytes + 1024;

    static size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(220 * 1024));
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "gemm_tc: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured = 220 * 1024;
    }
    const int n_tiles = (N + BLOCK_W - 1) / BLOCK_W, m_tiles = (M + tok_tile - 1) / tok_tile;
    if (m_tiles > 65535) return fail(MLB_UNSUPPORTED_SIZE, "gemm_tc: too many token tiles (%d)", m_tiles);
    if (splits == 1 && (long long)n_tiles * m_tiles > 148 && tok_tile % 32 == 0) {
        // many tiles: persistent CTAs with a double-buffered accumulator
        int acc_cols = 2 * cols;
        p.tmem_cols = 32;
        while (p.tmem_cols < acc_cols) p.tmem_cols *= 2;
        p.stages = stages > 0 ? stages : (int)((200 * 1024) / stage_bytes);
        if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
        if (p.stages < 2) p.stages = 2;
        const size_t smem_p = (size_t)p.stages * stage_bytes + 1024;
        static bool configured_p = false;
        if (!configured_p) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(220 * 1024));
            if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "gemm_tc: cannot reserve shared memory: %s", cudaGetErrorString(e));
            configured_p = true;
        }
        launch_kernel(gemm_tc_persistent_kernel, dim3(148), dim3(THREADS), smem_p, stream, map_w, map_x, p, n_tiles, m_tiles);
        return check_launch("gemm_tc_persistent");
    }
    dim3 grid(n_tiles, m_tiles, splits);
    launch_kernel(gemm_tc_kernel, grid, THREADS, smem, stream, map_w, map_x, p);
    return check_launch("gemm_tc");
}
