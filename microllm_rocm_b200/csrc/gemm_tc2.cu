// Prompt-sized bf16 products on the fifth-generation tensor cores with CTA PAIRS:
//     y[M, N] = x[M, K] * W[N, K]^T   (+ bias), or   y[M, I] = silu(x Wg^T) * (x Wu^T).
//
// Computed transposed, like gemm_stream.cu: the 256-row side of the instruction is a tile of 256
// WEIGHT rows, its N side a tile of 128 or 256 TOKENS.  A thread-block cluster of two CTAs (one
// per SM of a TPC) shares every tile through tcgen05.mma.cta_group::2: each CTA stages HALF of
// both operands (its 128 weight rows, its half of the tokens) and keeps its 128 accumulator
// rows in its own tensor memory.  Against one CTA per 128 x 256 tile this halves the shared-memory
// traffic per flop, which is what bounds the single-CTA kernel.
//
// Persistent: 74 pairs walk the output tiles; per CTA
//     warp 0   TMA producer: its halves of the operands into a ring of stages; the transaction
//              bytes of BOTH CTAs are counted on the leader's (rank 0) mbarrier
//              (cp.async.bulk.tensor ... .cta_group::2, no multicast)
//     warp 1   rank 0 only: one thread issues the pair's tcgen05.mma; tcgen05.commit with
//              multicast hands a stage back to both producers and an accumulator to both epilogues
//     warps 2-5  epilogue of the CTA's own 128 rows: tcgen05.ld, bias / SiLU*up, stores; the
//              accumulator is double-buffered so that the next tile's products run meanwhile
//
// Every mbarrier wait is bounded (error flag, then everybody falls through to the common end);
// the two cluster barriers (after set-up, before exit) are reached on every path.
//
// Replaces the library product the reference calls for its projections (hipBLASLt,
// src/ops/optimized.cpp:349-403) and the separate activation kernel (src/ops/optimized.cpp:676-683).
#include "common.cuh"

#include <cooperative_groups.h>
#include <cuda.h>
#include <cstdlib>

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int BLOCK_W = 128;                 // weight rows per CTA
constexpr int PAIR_W = 256;                  // weight rows per pair (MMA M)
constexpr int BLOCK_K = 64;                  // bf16 per stage row: 128 bytes, one swizzle span
constexpr int UMMA_K = 16;
constexpr int A_TILE_BYTES = BLOCK_W * BLOCK_K * 2;
constexpr int MAX_STAGES = 8;
constexpr int THREADS = 192;
constexpr int SPIN_LIMIT = 1 << 21;          // polls of up to 2 us each
constexpr int TMEM_COLS = 512;
#ifndef WAIT_HINT_NS
#define WAIT_HINT_NS 2000
#endif

struct PairParams {
    void* out;                 // [M, ldo] fp32 or bf16
    const float* bias;         // [N] or null
    int* error_flag;
    long long ldo;
    int M, N, K;
    int tok_tile;              // tokens per pair tile: 256, or 128 with dual
    int k_blocks, stages;
    int out_bf16;
    int accumulate;            // out += result (fp32 out only)
    int dual;                  // 1: silu(gate) * up; W rows n (gate) and up_offset + n (up); N counts gate rows
    int up_offset;
    int n_tiles, m_tiles;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// the address, in the cluster's shared window, of `addr` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t cluster_addr(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// One poll.  The hint lets the hardware park the thread until the phase completes or the time (ns) is up,
// so that waiting threads do not hammer shared memory while the tensor core reads its operands from it.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"((uint32_t)WAIT_HINT_NS) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
    for (int i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (error_flag) atomicExch(error_flag, code);
    return false;
}
// a whole warp waits: one lane polls, the others sleep at the warp barrier
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int* error_flag, int code) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, error_flag, code);
    return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}
// true in exactly one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}
// this CTA's half of an operand tile; the bytes are counted on `cluster_bar`, which may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t cluster_bar) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar) : "memory");
}
// K-major operand tile, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16: fp32 accumulator, bf16 A and B, both K-major, M = 256 over the pair
__device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(PAIR_W >> 4) << 24);
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the pair's MMAs so far have completed, on the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
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
    // g * sigmoid(g) (src/ops/ops.cpp:72-76, 760-785) in its one-branch form: for very negative g the
    // exponential overflows to +inf and the quotient is -0, which is the limit; no branch, so that the
    // 32 elements a thread holds can be evaluated side by side
    return __fdividef(g, 1.0f + __expf(-g));
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, PairParams p) {
    pdl_launch_dependents();
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster.block_rank();                       // 0: leader (issues the MMAs)
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int num_tiles = p.n_tiles * p.m_tiles;
    const int half_tok = p.tok_tile / 2;
    const uint32_t ring = (smem_u32(smem_dyn) + 1023u) & ~1023u;      // same offset in both CTAs
    const uint32_t a_bytes = p.dual ? 2u * A_TILE_BYTES : (uint32_t)A_TILE_BYTES;
    const uint32_t b_bytes = (uint32_t)half_tok * BLOCK_K * 2;
    const uint32_t stage_bytes = a_bytes + b_bytes;
    const uint32_t acc_cols = (uint32_t)(p.dual ? 2 * p.tok_tile : p.tok_tile);

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);             // the leader's expect_tx arrival
            mbar_init(smem_u32(&empty_bar[s]), 1);            // the leader's multicast commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);             // multicast commit
            mbar_init(smem_u32(&acc_empty[b]), 8);            // leader's copy: 4 epilogue warps of each CTA
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {                                          // the same warp of both CTAs allocates for the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster.sync();                                           // both CTAs' barriers exist before anything is signalled
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (both CTAs)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int n0 = (tile / p.m_tiles) * PAIR_W + (int)rank * BLOCK_W;
                const int tok0 = (tile % p.m_tiles) * p.tok_tile + (int)rank * half_tok;
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    lag_point();
                    const int s = it % p.stages;
                    const uint32_t round = it / p.stages;
                    if (round > 0 && !mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1, p.error_flag, 41)) { ok = false; break; }
                    const uint32_t dst = ring + (uint32_t)s * stage_bytes;
                    const uint32_t leader_full = cluster_addr(smem_u32(&full_bar[s]), 0);
                    if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * stage_bytes);
                    const int k = kb * BLOCK_K;
                    tma_load_2d_pair(dst, &map_w, k, n0, leader_full);
                    if (p.dual) tma_load_2d_pair(dst + A_TILE_BYTES, &map_w, k, p.up_offset + n0, leader_full);
                    tma_load_2d_pair(dst + a_bytes, &map_x, k, tok0, leader_full);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue (leader only)
        // The whole warp walks the loop converged (its waits park 31 lanes at a warp barrier) and ONE elected lane
        // issues: descriptors and addresses are then warp-uniform values, as the instruction wants them.
        if (rank == 0) {
            const uint32_t idesc = umma_idesc(p.tok_tile);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
                const uint32_t buf = local & 1, use = local >> 1;
                // both epilogues must have drained this buffer (the first use of each buffer passes at once)
                if (!mbar_wait_warp(smem_u32(&acc_empty[buf]), (use & 1) ^ 1, p.error_flag, 42)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + buf * acc_cols;
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    lag_point();
                    const int s = it % p.stages;
                    // every lane polls (one broadcast read each time): no shuffle between the barrier and the issue.
                    // No tcgen05 fence here: the copies and the MMAs that read them are ordered by the mbarrier itself.
                    if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s]), (it / p.stages) & 1, p.error_flag, 43))) { ok = false; break; }
                    const uint32_t a_addr = ring + (uint32_t)s * stage_bytes;
                    // descriptors of the stage; a K step of 16 elements moves the start address (16-byte units) by 2
                    const uint64_t adesc = umma_desc(a_addr), bdesc = umma_desc(a_addr + a_bytes), udesc = umma_desc(a_addr + A_TILE_BYTES);
                    if (elect_one()) {
                        umma_pair(acc, adesc, bdesc, idesc, kb > 0 ? 1u : 0u);
                        if (p.dual) umma_pair(acc + (uint32_t)p.tok_tile, udesc, bdesc, idesc, kb > 0 ? 1u : 0u);
#pragma unroll
                        for (int k = 1; k < BLOCK_K / UMMA_K; ++k) {
                            umma_pair(acc, adesc + 2 * k, bdesc + 2 * k, idesc, 1u);
                            if (p.dual) umma_pair(acc + (uint32_t)p.tok_tile, udesc + 2 * k, bdesc + 2 * k, idesc, 1u);
                        }
                        umma_commit_pair(smem_u32(&empty_bar[s]));  // the stage is free in both CTAs once these MMAs have read it
                    }
                    __syncwarp();
                }
                if (ok && elect_one()) umma_commit_pair(smem_u32(&acc_full[buf]));
                __syncwarp();
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
        const int quarter = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
            lag_point();
            const uint32_t buf = local & 1, use = local >> 1;
            const int n0 = (tile / p.m_tiles) * PAIR_W + (int)rank * BLOCK_W, tok0 = (tile % p.m_tiles) * p.tok_tile;
            const int f = n0 + quarter * 32 + lane;
            ok = mbar_wait_warp(smem_u32(&acc_full[buf]), use & 1, p.error_flag, 44);
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
                    if (tok >= p.M) break;
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
            // this warp is done reading the buffer: tell the leader's MMA thread
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_addr(smem_u32(&acc_empty[buf]), 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster.sync();                      // nobody leaves while the peer may still signal its barriers or read its operands
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
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

int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MLB_CUDA_ERROR, "gemm_pair: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MLB_CUDA_ERROR, "gemm_pair: cuTensorMapEncodeTiled failed with %d", (int)r);
    return MLB_OK;
}

}  // namespace

// y[M, N] = x[M, K] * W[N, K]^T (+ bias) (+ y when accumulate), or, with dual,
// y[M, N] = silu(x Wg^T) * (x Wu^T) where Wg = W rows [0, N) and Wu = W rows [up_offset, up_offset + N).
// x and W are bf16 with row pitches ldx, ldw (elements); K and the pitches must be multiples of 8 and the
// bases 16-byte aligned (TMA).  sm_count: SMs to use (an even number; CTAs come in pairs).
MLB_EXPORT int mlb_gemm_pair(const void* x, long long ldx, const void* w, long long ldw, int w_rows, const float* bias,
                             void* out, long long ldo, int out_bf16, int accumulate, int dual, int up_offset, int M, int N,
                             int K, int stages, int sm_count, int* error_flag, cudaStream_t stream) {
    if (M < 0 || N <= 0 || K <= 0) return fail(MLB_INVALID_ARGUMENT, "gemm_pair: bad sizes M=%d N=%d K=%d", M, N, K);
    if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K)
        return fail(MLB_UNSUPPORTED_SIZE, "gemm_pair: K=%d and the row pitches (%lld, %lld) must be multiples of 8 elements", K, ldx, ldw);
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(MLB_UNSUPPORTED_SIZE, "gemm_pair: operands must be 16-byte aligned");
    if (accumulate && out_bf16) return fail(MLB_INVALID_ARGUMENT, "gemm_pair: accumulation needs an fp32 output");
    if (dual && (up_offset < 0 || up_offset + N > w_rows)) return fail(MLB_INVALID_ARGUMENT, "gemm_pair: up rows outside the weight");
    if (!dual && N > w_rows) return fail(MLB_INVALID_ARGUMENT, "gemm_pair: more outputs than weight rows");
    if (sm_count < 2 || sm_count % 2 != 0) return fail(MLB_INVALID_ARGUMENT, "gemm_pair: sm_count %d must be even", sm_count);
    if (M == 0) return MLB_OK;

    PairParams p{};
    p.out = out; p.bias = bias; p.error_flag = error_flag; p.ldo = ldo; p.M = M; p.N = N; p.K = K;
    p.tok_tile = dual ? 128 : 256;
    p.k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
    p.out_bf16 = out_bf16; p.accumulate = accumulate; p.dual = dual; p.up_offset = up_offset;
    p.n_tiles = (N + PAIR_W - 1) / PAIR_W;
    p.m_tiles = (M + p.tok_tile - 1) / p.tok_tile;
    const int stage_bytes = (dual ? 2 : 1) * A_TILE_BYTES + (p.tok_tile / 2) * BLOCK_K * 2;
    p.stages = stages > 0 ? stages : (200 * 1024) / stage_bytes;
    if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
    if (p.stages < 2) p.stages = 2;
    const size_t smem = (size_t)p.stages * stage_bytes + 1024;

    CUtensorMap map_w, map_x;
    int status = make_map(&map_w, w, w_rows, K, ldw, BLOCK_W);
    if (status != MLB_OK) return status;
    status = make_map(&map_x, x, M, K, ldx, p.tok_tile / 2);
    if (status != MLB_OK) return status;

    static bool configured_on[MAX_DEVICES] = {false};         // the attribute belongs to the device
    bool& configured = configured_on[device_index()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(220 * 1024));
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "gemm_pair: cannot reserve shared memory: %s", cudaGetErrorString(e));
        configured = true;
    }
    const long long tiles = (long long)p.n_tiles * p.m_tiles;
    int ctas = sm_count;
    if (tiles * 2 < ctas) ctas = (int)tiles * 2;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(ctas);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    // No programmatic early start: a CTA of this kernel holds a whole SM and all of its tensor memory, so it becomes
    // resident only where a CTA of the kernel in front has left; started early, 2,048-token steps of three model
    // shapes take the same time within +-1 %.
    cudaLaunchAttribute attributes[1];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    config.attrs = attributes;
    config.numAttrs = 1;
    cudaLaunchKernelEx(&config, gemm_pair_kernel, map_w, map_x, p);
    return check_launch("gemm_pair");
}
