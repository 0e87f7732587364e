// Prompt attention on the fifth-generation tensor cores: causal (optionally windowed)
// grouped-query attention of prompt portions over the paged bf16 cache.  Compiled per head
// size (-DHEAD_DIM=64 or 128).
//
// One CTA owns 128 consecutive new tokens of one (sequence, query head) and walks the keys
// lo..hi that any of them may see in tiles of 128 keys, whose edges sit at multiples of 128
// of the absolute position.  Six warps:
//     warp 0     TMA producer.  The Q tile once; then the K and V tiles in the order the tensor
//                core needs them (K0 K1 V0 K2 V1 ...) into one ring of 32 KB slots (six at head
//                size 128), so that loads run two to three key tiles ahead.  Lane g looks up page g of a tile in
//                the block table (one tile ahead of use) and issues that page's
//                cp.async.bulk.tensor copies, one per 64-element column span, 128-byte swizzled.
//     warp 1     one thread issues tcgen05.mma (kind::f16, bf16 in, fp32 in tensor memory):
//                S = Q K^T into one of two score buffers, O += P V into the output accumulator,
//                with P read from tensor memory (the A operand may live there) and V from the ring.
//                S of tile j+1 is issued before P V of tile j, so the tensor pipe works on
//                the next scores while the softmax warps turn the current ones into P.
//     warps 2-5  softmax, one thread per query row: tcgen05.ld brings the row's 128 scores,
//                mask (only in tiles that touch the causal or window edge), running maximum and
//                sum in fp32 with base-2 exponentials, P rounded to bf16 and written back to
//                tensor memory (tcgen05.st, two buffers, two keys per column): it never touches
//                shared memory.  The accumulator in tensor memory is rescaled
//                only when a row's maximum has grown by more than 2^8 since the last rescale:
//                P and the row sum use the same (stale) reference, so the quotient is exact.
//                V rows of keys that no row of the tile may see are cleared in shared memory, so
//                that whatever an unused slot of a page holds cannot reach the output.
// V is used as stored, [key, head element]: it is the MN-major B operand of P V.
//
// Formulas as the plain kernel's (attention_plain.cu; src/ops/ops.cpp:2343-2384 in the
// reference: key range, head grouping, scale after the dot product, fp32 softmax).
//
// Every wait on an mbarrier is bounded; when a bound is hit the error flag is raised, the CTA
// waits (bounded) for the copies it still has in flight, frees its tensor memory and returns.
#include "common.cuh"

#include <cuda.h>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=64 or 128"
#endif

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int D = HEAD_DIM;
static_assert(D == 64 || D == 128, "HEAD_DIM must be 64 or 128");
constexpr int BM = 128;                      // query rows per CTA (MMA M)
constexpr int BN = 128;                      // keys per tile
constexpr int SPANS = D / 64;                // 64-element (128-byte) column spans of a Q/K/V row
constexpr int ROW_BYTES = 128;               // one swizzle span
constexpr int Q_BYTES = SPANS * BM * ROW_BYTES;
constexpr int KV_BYTES = SPANS * BN * ROW_BYTES;
constexpr int RING_BUDGET = 226 * 1024 - 1024 - Q_BYTES;
constexpr int SLOTS = RING_BUDGET / KV_BYTES > 8 ? 8 : RING_BUDGET / KV_BYTES;
constexpr int SMEM_BYTES = Q_BYTES + SLOTS * KV_BYTES + 1024;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;               // S0 [0,128)  S1 [128,256)  O [256, 256+D)  P0 [384,448)  P1 [448,512)
constexpr int O_COL = 2 * BN;
constexpr int P_COL = 384;                   // P as bf16 pairs: 64 columns per buffer, two buffers
static_assert(O_COL + D <= P_COL, "the accumulator must end before the P buffers");
constexpr int SPIN_LIMIT = 1 << 21;          // polls of up to 2 us each
constexpr int MAX_PAGES_PER_TILE = 16;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_STEP = 8.0f;         // rescale the accumulator when the maximum grew by 2^8

struct TcParams {
    __nv_bfloat16* out;             // [T, ldo]
    long long ldo;
    const int* seq_starts;          // [A+1]
    const int* seq_pos0;            // [A]
    const int* block_table;         // [A, max_blocks]
    const int* work;                // [num_work, 2] (sequence, 128-row tile of its new tokens)
    int max_blocks, num_pages, page_size, pages_per_tile;
    int num_heads, num_kv_heads, group, window;
    float scale_log2;
    int* error_flag;
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
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    // the hint (ns) lets the hardware park the thread until the phase completes instead of spinning on shared memory
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(2000u) : "memory");
    return ok != 0;
}
// false when the bound was hit (the caller gives up and the flag tells the host)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
    for (int i = 0; i < SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (error_flag) atomicCAS(error_flag, 0, code);          // the first failure is the one worth reporting
    return false;
}
// true in exactly one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// Shared-memory operand descriptors, 128-byte swizzle.  Rows are 128 bytes, groups of 8 rows
// 1024 bytes apart (the stride byte offset).  K-major: a row is an M/N index and holds 64
// contraction elements.  MN-major: a row is a contraction index and holds 64 M/N elements; the
// next 64 M/N elements are `lead_bytes` further on.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lead_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lead_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor: fp32 accumulator, bf16 A (K-major) and B
__device__ __forceinline__ uint32_t idesc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(id), "r"(accumulate) : "memory");
}
// the same with the A operand in tensor memory (lane = row, a 32-bit column = two neighbouring bf16 of the contraction)
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(id), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(THREADS, 1)
fa_tc_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, TcParams p) {
    pdl_launch_dependents();
    extern __shared__ unsigned char smem_dyn[];
    __shared__ __align__(8) unsigned long long q_full, slot_full[SLOTS], slot_empty[SLOTS], s_full[2], s_empty[2], p_full[2], pv_done[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;     // the swizzle pattern wants 1024-byte alignment
    const uint32_t q_s = base;
    const uint32_t ring_s = q_s + Q_BYTES;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&q_full), 1);
        for (int s = 0; s < SLOTS; ++s) {
            mbar_init(smem_u32(&slot_full[s]), 1);
            mbar_init(smem_u32(&slot_empty[s]), 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(smem_u32(&s_full[s]), 1);
            mbar_init(smem_u32(&s_empty[s]), 4);          // one arrival per softmax warp
        }
        // One barrier per P buffer.  A softmax warp may be a whole tile ahead of another (tile j + 1's scores exist
        // before P V of tile j is issued): with a single barrier its arrival for tile j + 1 would complete tile j's
        // phase in place of the slow warp's, and P V would read rows of P that were not written yet.
        mbar_init(smem_u32(&p_full[0]), 4);
        mbar_init(smem_u32(&p_full[1]), 4);
        mbar_init(smem_u32(&pv_done[0]), 1);        // P V of the even tiles, and of the odd ones: one per P buffer
        mbar_init(smem_u32(&pv_done[1]), 1);
        failed_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_s)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();                  // queries and this step's keys were written by the kernel before

    // ---- the tile's geometry (uniform over the CTA)
    const int head = blockIdx.x, item = blockIdx.y;
    const int seq = p.work[2 * item], q_tile = p.work[2 * item + 1];
    const int token0 = p.seq_starts[seq];
    const int n_new = p.seq_starts[seq + 1] - token0;
    const int pos0 = p.seq_pos0[seq];
    const int row_first = q_tile * BM;
    const int rows = min(BM, n_new - row_first);
    const int qpos_first = pos0 + row_first, qpos_last = qpos_first + rows - 1;
    const int lo = (p.window > 0 && qpos_first - p.window + 1 > 0) ? qpos_first - p.window + 1 : 0;
    const int kt_begin = lo / BN;
    const int n_tiles = qpos_last / BN + 1 - kt_begin;
    const int kvh = head / p.group;

    // Ring items in order of need: K0, then for every tile j: K(j+1) if there is one, V(j).
    //   item of K(j) = 0 for j = 0, 2j - 1 otherwise;   item of V(j) = 2j + 2, or 2j + 1 for the last tile.
    const int n_items = 2 * n_tiles;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer (whole warp)
        if (lane == 0) {
            mbar_expect_tx(smem_u32(&q_full), Q_BYTES);
#pragma unroll
            for (int s = 0; s < SPANS; ++s)
                tma_load_2d(q_s + s * BM * ROW_BYTES, &map_q, head * D + s * 64, token0 + row_first, smem_u32(&q_full));
        }
        const int* table = p.block_table + (size_t)seq * p.max_blocks;
        auto tile_of = [&](int i, int& is_v) {            // item -> key tile, and whether it is the V half
            if (i == 0) { is_v = 0; return 0; }
            if (i == n_items - 1) { is_v = 1; return n_tiles - 1; }
            is_v = (i & 1) ? 0 : 1;
            return is_v ? (i - 2) / 2 : (i + 1) / 2;
        };
        auto lookup = [&](int i) {                        // lane g: the page of block g of item i's tile
            int is_v;
            const int block = (kt_begin + tile_of(i, is_v)) * p.pages_per_tile + lane;
            return (lane < p.pages_per_tile && block < p.max_blocks) ? __ldg(table + block) : -1;
        };
        bool ok = true;
        int issued = 0;
        int page_next = lookup(0);
        for (int i = 0; i < n_items; ++i) {
            lag_point();
            int page = page_next;
            if (i + 1 < n_items) page_next = lookup(i + 1);          // in flight while this item waits and issues
            const int slot = i % SLOTS;
            if (i >= SLOTS) ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&slot_empty[slot]), ((i / SLOTS) - 1) & 1, p.error_flag, 21)) != 0;
            if (!ok) break;
            int is_v;
            const int tile = tile_of(i, is_v);
            const uint32_t bar = smem_u32(&slot_full[slot]);
            if (lane == 0) mbar_expect_tx(bar, KV_BYTES);
            __syncwarp();
            if (lane < p.pages_per_tile) {
                const int block = (kt_begin + tile) * p.pages_per_tile + lane;
                if (page < 0 || page >= p.num_pages) {
                    // a page that holds a key some row must see has to exist; the others are masked
                    const int first_key = block * p.page_size;
                    if (first_key <= qpos_last && first_key + p.page_size - 1 >= lo && p.error_flag) atomicExch(p.error_flag, 2);
                    page = 0;
                }
                const int row = ((page * 2 + is_v) * p.num_kv_heads + kvh) * p.page_size;
                const uint32_t dst = ring_s + slot * KV_BYTES + lane * p.page_size * ROW_BYTES;
#pragma unroll
                for (int s = 0; s < SPANS; ++s) tma_load_2d(dst + s * BN * ROW_BYTES, &map_kv, s * 64, row, bar);
            }
            issued = i + 1;
        }
        if (lane == 0 && (!ok || failed_s)) {
            // give the copies in flight a bounded chance to land before the CTA's memory goes away
            for (int i = max(0, issued - SLOTS); i < issued; ++i)
                mbar_wait(smem_u32(&slot_full[i % SLOTS]), (i / SLOTS) & 1, nullptr, 0);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issue
        // The whole warp walks the loop converged and ONE elected lane issues, so that descriptors and
        // addresses are warp-uniform values; every lane polls the barriers (one broadcast read per poll).
        {
            const uint32_t idesc_qk = idesc(BN, false), idesc_pv = idesc(D, true);
            auto wait_warp = [&](unsigned long long* bar, uint32_t parity, int code) {
                return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, p.error_flag, code)) != 0;
            };
            bool ok = wait_warp(&q_full, 0, 23);
            int item = 0;                                  // ring items are consumed in the order they were loaded
            auto issue_qk = [&](int j) {
                const int slot = item % SLOTS;
                if (!wait_warp(&slot_full[slot], (item / SLOTS) & 1, 24)) return false;
                const uint32_t kb = ring_s + slot * KV_BYTES;
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) {
                        const uint32_t off = (ks / 4) * (BM * ROW_BYTES) + (ks % 4) * 32;
                        umma(tmem_base + (uint32_t)((j & 1) * BN), desc_k_major(q_s + off), desc_k_major(kb + off), idesc_qk, ks > 0);
                    }
                    umma_commit(smem_u32(&slot_empty[slot]));
                    umma_commit(smem_u32(&s_full[j & 1]));
                }
                __syncwarp();
                ++item;
                return true;
            };
            for (int j = 0; j < 2 && j < n_tiles && ok; ++j) ok = issue_qk(j);
            for (int j = 0; j < n_tiles && ok; ++j) {
                lag_point();
                ok = wait_warp(&p_full[j & 1], (j >> 1) & 1, 25);
                if (!ok) break;
                const int slot = item % SLOTS;
                ok = wait_warp(&slot_full[slot], (item / SLOTS) & 1, 26);
                if (!ok) break;
                tc_fence_after();                          // P and the rescaled accumulator were written by the softmax warps
                const uint32_t vb = ring_s + slot * KV_BYTES;
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < BN / 16; ++ks)          // 16 keys = 8 columns of P
                        umma_ts(tmem_base + O_COL, tmem_base + (uint32_t)(P_COL + (j & 1) * (BN / 2) + ks * 8),
                                desc_mn_major(vb + ks * 16 * ROW_BYTES, BN * ROW_BYTES), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    umma_commit(smem_u32(&slot_empty[slot]));
                    umma_commit(smem_u32(&pv_done[j & 1]));
                }
                __syncwarp();
                ++item;
                if (j + 2 < n_tiles) {
                    ok = wait_warp(&s_empty[j & 1], (j >> 1) & 1, 27);
                    if (!ok) break;
                    tc_fence_after();                      // the softmax warps have read this score buffer
                    ok = issue_qk(j + 2);
                }
            }
            if (!ok && lane == 0) failed_s = 1;
        }
    } else {
        // ------------------------------------------------------------------ softmax, one thread per row
        const int quarter = warp & 3;                     // the tensor-memory lanes this warp may touch
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const int qpos = qpos_first + r;
        const int lo_r = p.window > 0 ? qpos - p.window + 1 : -0x40000000;
        float m_used = -INFINITY, l = 0.0f;
        bool ok = true;
        // the tensor-memory instructions below are warp-wide: a wait gives up for the whole warp or not at all
        auto wait_all = [&](unsigned long long* bar, uint32_t parity, int code) {
            return __all_sync(0xffffffffu, mbar_wait(smem_u32(bar), parity, p.error_flag, code)) != 0;
        };
        for (int j = 0; j < n_tiles; ++j) {
            const int buf = j & 1;
            lag_point();
            ok = wait_all(&s_full[buf], (j >> 1) & 1, 28);
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[BN];
#pragma unroll
            for (int c = 0; c < BN / 32; ++c) tmem_ld32(lane_base + (uint32_t)(buf * BN + c * 32), sr + c * 32);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&s_empty[buf]));

            const int kbase = (kt_begin + j) * BN;
            const bool edge = (kbase + BN - 1 > qpos_first) || (p.window > 0 && kbase < qpos_last - p.window + 1);
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};       // four chains: no 128-long dependence
            if (edge) {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const int kpos = kbase + c;
                    const float s = (kpos <= qpos && kpos >= lo_r) ? __uint_as_float(sr[c]) : -INFINITY;
                    sr[c] = __float_as_uint(s);
                    mx4[c & 3] = fmaxf(mx4[c & 3], s);
                }
            } else {
#pragma unroll
                for (int c = 0; c < BN; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c]));
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            const float m_new = fmaxf(m_used, mx * p.scale_log2);
            const bool grow = m_new > m_used + RESCALE_STEP;          // also true for the first finite maximum
            const float alpha = grow ? (m_used == -INFINITY ? 0.0f : fast_exp2(m_used - m_new)) : 1.0f;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                ok = wait_all(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, 29);      // O holds tiles 0..j-1
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + (uint32_t)(O_COL + c * 32), o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_base + (uint32_t)(O_COL + c * 32), o);
                }
                tmem_wait_st();
            }
            if (grow) { l *= alpha; m_used = m_new; }
            const float m_ref = m_used == -INFINITY ? 0.0f : m_used;
            // P = 2^(s * scale - m), rounded to bf16 for the tensor core; the sum keeps fp32 terms
            float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            uint32_t packed[BN / 2];
#pragma unroll
            for (int c = 0; c < BN; c += 2) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(sr[c]), p.scale_log2, -m_ref));
                const float p1 = fast_exp2(fmaf(__uint_as_float(sr[c + 1]), p.scale_log2, -m_ref));
                sum4[(c >> 1) & 3] += p0 + p1;
                packed[c / 2] = pack_bf16(p0, p1);
            }
            const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
            l += sum;
            if (j > 1) {                                  // this P buffer is free once P V of the tile before the last is done
                ok = wait_all(&pv_done[j & 1], ((j - 2) >> 1) & 1, 30);
                if (!ok) break;
            }
            // Keys outside lo..hi of the whole tile have P = 0, but 0 * V must not be NaN whatever an unused
            // slot of a page holds: their V rows are cleared before the tensor core reads them.
            const int keep_from = max(0, lo - kbase), keep_to = min(BN, qpos_last + 1 - kbase);
            if (keep_from > 0 || keep_to < BN) {
                const int v_item = (j + 1 < n_tiles) ? 2 * j + 2 : 2 * j + 1;
                ok = wait_all(&slot_full[v_item % SLOTS], (v_item / SLOTS) & 1, 32);
                if (!ok) break;
                const uint32_t vb = ring_s + (v_item % SLOTS) * KV_BYTES;
                const int cleared = keep_from + (BN - keep_to);
                for (int i = r; i < cleared * SPANS * 8; i += BM) {
                    const int row_i = i / (SPANS * 8), rest = i % (SPANS * 8);
                    const int key = row_i < keep_from ? row_i : keep_to + (row_i - keep_from);
                    const uint32_t addr = vb + (rest / 8) * (BN * ROW_BYTES) + key * ROW_BYTES + (rest % 8) * 16;
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
                }
            }
            // row r of P goes to tensor memory, where the second product reads it as its A operand
            // (lane = row, a column = two neighbouring keys as bf16): no shared memory, no swizzle, no proxy fence
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tmem_st32(lane_base + (uint32_t)(P_COL + buf * (BN / 2) + c * 32), packed + c * 32);
            tmem_wait_st();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the cleared V rows, for the tensor core
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&p_full[buf]));
        }
        if (ok && n_tiles > 0) ok = wait_all(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, 31);
        if (ok && n_tiles > 0) {
            tc_fence_after();
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            __nv_bfloat16* orow = p.out + (size_t)(token0 + row_first + r) * p.ldo + (size_t)head * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(lane_base + (uint32_t)(O_COL + c * 32), o);
                tmem_wait_ld();
                if (r < rows) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 v;
                        v.x = pack_bf16(__uint_as_float(o[i + 0]) * inv, __uint_as_float(o[i + 1]) * inv);
                        v.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                        v.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                        v.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + i) = v;
                    }
                }
            }
        }
        if (!ok) failed_s = 1;
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
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

// rows x cols bf16 matrix with row pitch `ld` elements; box = box_rows x 64 columns, 128-byte swizzle,
// rows outside the matrix read as zero
int make_map(CUtensorMap* map, const void* base_ptr, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(MLB_CUDA_ERROR, "attention_tc: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base_ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MLB_CUDA_ERROR, "attention_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
    return MLB_OK;
}

}  // namespace

MLB_EXPORT int mlb_fa_tc_head_dim() { return D; }
MLB_EXPORT int mlb_fa_tc_rows_per_tile() { return BM; }

// 1 when the kernel takes this cache geometry, 0 (with the reason in mlb_last_error) when not
MLB_EXPORT int mlb_fa_tc_supported(int page_size, float scale) {
    if (page_size < 8 || page_size % 8 != 0 || BN % page_size != 0 || BN / page_size > MAX_PAGES_PER_TILE) {
        fail(MLB_UNSUPPORTED_SIZE, "attention_tc: page_size %d must be a multiple of 8 that divides %d", page_size, BN);
        return 0;
    }
    if (!(scale > 0.0f)) {
        fail(MLB_UNSUPPORTED_SIZE, "attention_tc: the softmax scale must be positive");
        return 0;
    }
    return 1;
}

// q [tokens, ldq] and out [tokens, ldo] bf16 with heads side by side; pages [num_pages, 2, NKV, page_size, D].
// work: num_work pairs (sequence, tile of 128 new tokens); one CTA per pair and query head.
MLB_EXPORT int mlb_paged_attention_tc(const void* q, long long ldq, const void* pages, void* out, long long ldo, int tokens,
                                      const int* seq_starts, const int* seq_pos0, const int* block_table, const int* work,
                                      int num_work, int max_blocks, int num_pages, int page_size, int num_heads,
                                      int num_kv_heads, int window, float scale, int* error_flag, cudaStream_t stream) {
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail(MLB_INVALID_ARGUMENT, "attention_tc: bad head counts %d/%d", num_heads, num_kv_heads);
    if (!mlb_fa_tc_supported(page_size, scale)) return MLB_UNSUPPORTED_SIZE;
    if (num_pages <= 0 || max_blocks <= 0 || window < 0 || num_work < 0 || tokens < 0)
        return fail(MLB_INVALID_ARGUMENT, "attention_tc: bad cache geometry");
    if (ldq < (long long)num_heads * D || ldo < (long long)num_heads * D || ldq % 8 != 0 || ldo % 8 != 0 ||
        ((uintptr_t)q & 15) || ((uintptr_t)out & 15) || ((uintptr_t)pages & 15))
        return fail(MLB_UNSUPPORTED_SIZE, "attention_tc: q, out and the pages must be 16-byte aligned with pitches that are multiples of 8");
    const long long kv_rows = (long long)num_pages * 2 * num_kv_heads * page_size;
    if (kv_rows >= (1ll << 31)) return fail(MLB_UNSUPPORTED_SIZE, "attention_tc: the cache has too many rows (%lld)", kv_rows);
    if (num_work > 65535) return fail(MLB_UNSUPPORTED_SIZE, "attention_tc: too many row tiles (%d)", num_work);
    if (num_work == 0 || tokens == 0) return MLB_OK;

    CUtensorMap map_q, map_kv;
    int status = make_map(&map_q, q, tokens, (long long)num_heads * D, ldq, BM);
    if (status != MLB_OK) return status;
    status = make_map(&map_kv, pages, kv_rows, D, D, page_size);
    if (status != MLB_OK) return status;

    TcParams p{(__nv_bfloat16*)out, ldo, seq_starts, seq_pos0, block_table, work, max_blocks, num_pages, page_size,
               BN / page_size, num_heads, num_kv_heads, num_heads / num_kv_heads, window, scale * LOG2E, error_flag};
    static bool configured_on[MAX_DEVICES] = {false};         // the attribute belongs to the device
    bool& configured = configured_on[device_index()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(fa_tc_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "attention_tc: cannot reserve %d bytes of shared memory: %s",
                                          (int)SMEM_BYTES, cudaGetErrorString(e));
        configured = true;
    }
    // Launched without programmatic early start.  Started early it gains nothing that could be measured (2,048-token
    // steps of three model shapes: within +-1 %): a CTA takes a whole SM (225 KB of shared memory, all of the tensor
    // memory), so it becomes resident only where a CTA of the kernel in front has left.  (Bounded waits that once ran
    // out when this kernel was started early, with the host far ahead of the GPU, were the single P barrier's fault,
    // see p_full in the kernel: with one barrier per P buffer the same commands run with or without early start.)
    fa_tc_prefill_kernel<<<dim3(num_heads, num_work, 1), THREADS, SMEM_BYTES, stream>>>(map_q, map_kv, p);
    return check_launch("fa_tc_prefill");
}
