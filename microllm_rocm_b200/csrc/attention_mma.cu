// Tensor-core attention over the paged bf16 cache, for prompt portions and decoded tokens
// alike.  Compiled per head size (-DHEAD_DIM=...).
//
// The unit of work is a ROW TILE: 16 rows of one (sequence, kv head), a row being one
// (new token, query head of the group).  A decoded token contributes G = NH/NKV rows, a
// prompt portion n*G; every row carries its own position, so one causal/window rule covers
// both.  A warp walks the keys lo..hi of its tile 16 at a time:
//     S = Q K^T   (mma.sync m16n8k16, bf16 in, fp32 out; Q from shared memory, K straight
//                  from the page into registers with 16-byte loads)
//     online softmax in fp32 (running max and sum per row, base-2 exponentials)
//     O += P V    (P rounded to bf16 as the tensor-core operand; V straight from the page)
// K/V are read once per row tile and shared by all query heads of the group; the reference
// re-reads them per query head and keeps every score in shared memory
// (src/ops/hip/basic_kernels.hip:1035-1083, limit 4096 keys at src/ops/ops.cpp:1592).
//
// Two launch shapes:
//   prefill  one CTA = 4 warps = 4 consecutive row tiles; K/V tiles of 64 keys staged once per
//            CTA in shared memory (cp.async, two stages), fragments by ldmatrix; no key split
//   decode   one CTA = one row tile, its 4 warps take every 4th key tile and are merged in
//            shared memory; the keys are further split over a thread-block cluster whose CTAs
//            combine their results through distributed shared memory, in rank order.
//
// Operand layout trick: mma.sync only needs A and B to agree on which contraction index a
// register holds.  Thread t of a quad therefore loads 8 CONSECUTIVE head elements of a key
// (one 16-byte load) and uses them as the fragments of two k-steps; Q is read from shared
// memory with the same permutation.  For V the output columns are permuted instead.
#include "common.cuh"

#include <cooperative_groups.h>
#include <cuda.h>
#include <mutex>
#include <unordered_map>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<multiple of 32, at most 256>"
#endif

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int D = HEAD_DIM;
static_assert(D % 32 == 0 && D >= 32 && D <= 256, "HEAD_DIM must be a multiple of 32 in 32..256");
constexpr int KCHUNKS = D / 32;             // 32 head elements per chunk of the QK^T contraction
constexpr int VBLOCKS = (D + 63) / 64;      // 64 output elements per block of PV
constexpr int NB_O = VBLOCKS * 8;           // 8-wide output column blocks
constexpr int WARPS = 4;
constexpr int Q_STRIDE = D + 32;            // bf16 elements; +64 bytes keeps 16-byte row loads conflict free
constexpr float LOG2E = 1.4426950408889634f;

struct FaParams {
    const __nv_bfloat16* q;         // [T, NH*D]
    const __nv_bfloat16* pages;     // [num_pages, 2, NKV, page_size, D]
    __nv_bfloat16* out;             // [T, NH*D]
    const int* seq_starts;          // [A+1] first flat token of each sequence
    const int* seq_pos0;            // [A]   tokens cached before this step
    const int* block_table;         // [A, max_blocks]
    const int* work;                // [num_work, 2] (sequence, first row tile)
    int max_blocks, num_pages, page_size;
    int num_heads, num_kv_heads, group;
    int window;
    float scale_log2;               // softmax scale * log2(e)
    int page_shift;                 // log2(page_size) when it is a power of two, else -1
    int* error_flag;
    int listed;                     // decode shape: 1 = work item i is sequence work[i] (a step that also holds prompt
                                    // portions), 0 = work item i is sequence i and token i (every sequence brings one token)
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

constexpr float RESCALE_STEP = 8.0f;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint4 load16(const __nv_bfloat16* p) {
    // keys and values are read once per step: they need no line in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

struct RowState {
    float m[2];            // running maximum (base-2 scaled) of rows g and g+8
    float l[2];            // this thread's share of the running sum
    float o[NB_O][4];      // output accumulators; column permutation: see out_dim()
};

// Rows of a tile: row r (0..15) is flat row row0 + r of the (sequence, kv head) row space,
// token = row / group, head-in-group = row % group.
struct TileGeometry {
    int seq, kvh, row0, n_new, pos0, token0;   // token0: flat index of the sequence's first new token
    __device__ __forceinline__ int token_of(int r, int group) const { return (row0 + r) / group; }
};

// The block-table entries a CTA will need, fetched once into shared memory: a lookup in the
// key loop must not cost a trip to global memory, because the loads of a tile cannot issue
// before its page is known.  Blocks outside the cached span fall back to global memory.
constexpr int TABLE_SPAN = 1024;
struct PageTable {
    const int* global;       // this sequence's row of the block table
    const int* cached;       // shared-memory copy of blocks [first, first + count)
    int first, count, max_blocks;
    __device__ __forceinline__ int page_of(int block) const {
        if (block >= max_blocks) return -1;
        const int i = block - first;
        return (i >= 0 && i < count) ? cached[i] : __ldg(global + block);
    }
};

__device__ __forceinline__ void fill_page_table(PageTable& pt, int* table_s, const int* row, int max_blocks,
                                                int first_block, int last_block, int tid, int threads) {
    pt.global = row;
    pt.cached = table_s;
    pt.max_blocks = max_blocks;
    pt.first = first_block;
    pt.count = max(0, min(min(last_block, max_blocks - 1) - first_block + 1, TABLE_SPAN));
    for (int i = tid; i < pt.count; i += threads) table_s[i] = __ldg(row + first_block + i);
}

// The K and V of 16 keys as this thread holds them for the tensor cores.
struct KeyTile {
    uint4 k[2][KCHUNKS];
    uint4 v[VBLOCKS][4];
    int base;              // first key position; -1: nothing loaded
};

// Issue every load of one 16-key tile (nothing waits here).  hi_tile: last position any row
// of the row tile may see; slots behind it were never written by this sequence, so their V
// stays zero (their probability is zero, and zero times stale memory must stay zero).
__device__ __forceinline__ void load_keys(const FaParams& p, const TileGeometry& geo, const PageTable& pt, int kt,
                                          int hi_tile, KeyTile& kv) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int base = kt * 16;
    const int block = p.page_shift >= 0 ? base >> p.page_shift : base / p.page_size;
    const int slot = p.page_shift >= 0 ? base & (p.page_size - 1) : base % p.page_size;
    const int page = pt.page_of(block);
    if (page < 0 || page >= p.num_pages) {
        if (lane == 0 && p.error_flag) atomicExch(p.error_flag, 3);
        kv.base = -1;
        return;
    }
    kv.base = base;
    const size_t page_stride = (size_t)2 * p.num_kv_heads * p.page_size * D;
    const __nv_bfloat16* kbase = p.pages + (size_t)page * page_stride + ((size_t)geo.kvh * p.page_size + slot) * D;
    const __nv_bfloat16* vbase = kbase + (size_t)p.num_kv_heads * p.page_size * D;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int c = 0; c < KCHUNKS; ++c) kv.k[nb][c] = load16(kbase + (size_t)(nb * 8 + g) * D + c * 32 + t * 8);
    if (base + 15 <= hi_tile) {                        // every key of the tile was written: no predicates
#pragma unroll
        for (int vb = 0; vb < VBLOCKS; ++vb) {
            const int col = vb * 64 + g * 8;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int key = 2 * t + (r & 1) + 8 * (r >> 1);   // this thread's keys: 2t, 2t+1, 2t+8, 2t+9
                kv.v[vb][r] = (D % 64 == 0 || col < D) ? load16(vbase + (size_t)key * D + col) : make_uint4(0, 0, 0, 0);
            }
        }
        return;
    }
#pragma unroll
    for (int vb = 0; vb < VBLOCKS; ++vb) {
        const int col = vb * 64 + g * 8;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int key = 2 * t + (r & 1) + 8 * (r >> 1);
            kv.v[vb][r] = (col < D && base + key <= hi_tile) ? load16(vbase + (size_t)key * D + col) : make_uint4(0, 0, 0, 0);
        }
    }
}

// One 16-key tile through scores, running softmax and the value product.
// first_pos: the smallest position of any real row of the row tile; last_lo: the largest window start.
__device__ __forceinline__ void consume_keys(const FaParams& p, const __nv_bfloat16* q_s, const KeyTile& kv,
                                             const int (&pos_row)[2], const int (&lo_row)[2], int first_pos, int last_lo,
                                             RowState& st) {
    if (kv.base < 0) return;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    float s[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nb][e] = 0.0f;
#pragma unroll
    for (int c = 0; c < KCHUNKS; ++c) {
        const uint4 qa = *reinterpret_cast<const uint4*>(q_s + g * Q_STRIDE + c * 32 + t * 8);
        const uint4 qb = *reinterpret_cast<const uint4*>(q_s + (g + 8) * Q_STRIDE + c * 32 + t * 8);
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            mma_bf16(s[nb], qa.x, qb.x, qa.y, qb.y, kv.k[nb][c].x, kv.k[nb][c].y);
            mma_bf16(s[nb], qa.z, qb.z, qa.w, qb.w, kv.k[nb][c].z, kv.k[nb][c].w);
        }
    }
    // Masks only where the tile touches an edge (the newest key, the window's start); a padding row
    // (position -1) of an interior tile keeps finite scores that are never stored.
    const bool edge = kv.base + 15 > first_pos || kv.base < last_lo;           // uniform over the warp
    float mx[2] = {-INFINITY, -INFINITY};
    if (edge) {
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = e >> 1;
                const int key = kv.base + nb * 8 + 2 * t + (e & 1);
                const bool ok = key >= lo_row[i] && key <= pos_row[i];
                s[nb][e] = ok ? s[nb][e] * p.scale_log2 : -INFINITY;
                mx[i] = fmaxf(mx[i], s[nb][e]);
            }
    } else {
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[nb][e] *= p.scale_log2;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
            }
    }
    // The reference maximum of a row moves only when the true maximum has grown by more than 2^8 beyond
    // it (P, the running sum and the accumulator all use the same reference, so the result is exact):
    // after the first tiles the accumulator is hardly ever rescaled.
    float corr[2];
    bool grow = false;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const bool g_i = mx[i] > st.m[i] + RESCALE_STEP;          // true as well for the first finite maximum
        corr[i] = g_i ? (st.m[i] == -INFINITY ? 0.0f : fast_exp2(st.m[i] - mx[i])) : 1.0f;
        st.m[i] = g_i ? mx[i] : st.m[i];
        grow |= g_i;
    }
    float rowsum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float ref = st.m[i] == -INFINITY ? 0.0f : st.m[i];
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e2 = 0; e2 < 2; ++e2) {
                const float pv = fast_exp2(s[nb][2 * i + e2] - ref);      // 2^(-inf) = 0 for masked keys
                s[nb][2 * i + e2] = pv;
                rowsum[i] += pv;
            }
    }
    if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
        for (int i = 0; i < 2; ++i) st.l[i] *= corr[i];
#pragma unroll
        for (int nbo = 0; nbo < NB_O; ++nbo) {
            st.o[nbo][0] *= corr[0]; st.o[nbo][1] *= corr[0];
            st.o[nbo][2] *= corr[1]; st.o[nbo][3] *= corr[1];
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) st.l[i] += rowsum[i];
    const unsigned pa0 = pack_bf16(s[0][0], s[0][1]);     // row g,   keys 2t, 2t+1
    const unsigned pa1 = pack_bf16(s[0][2], s[0][3]);     // row g+8
    const unsigned pa2 = pack_bf16(s[1][0], s[1][1]);     // row g,   keys 8+2t, 9+2t
    const unsigned pa3 = pack_bf16(s[1][2], s[1][3]);     // row g+8
#pragma unroll
    for (int vb = 0; vb < VBLOCKS; ++vb) {
        const unsigned* v0 = reinterpret_cast<const unsigned*>(&kv.v[vb][0]);
        const unsigned* v1 = reinterpret_cast<const unsigned*>(&kv.v[vb][1]);
        const unsigned* v2 = reinterpret_cast<const unsigned*>(&kv.v[vb][2]);
        const unsigned* v3 = reinterpret_cast<const unsigned*>(&kv.v[vb][3]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned sel = (j & 1) ? 0x7632u : 0x5410u;       // high or low bf16 of both words
            const unsigned b0 = __byte_perm(v0[j >> 1], v1[j >> 1], sel);
            const unsigned b1 = __byte_perm(v2[j >> 1], v3[j >> 1], sel);
            mma_bf16(st.o[vb * 8 + j], pa0, pa1, pa2, pa3, b0, b1);
        }
    }
}

// Keys [tile_begin, tile_end) in units of 16, visiting every `stride`-th starting at
// tile_begin + first.  `a` and `b` are the register homes of the first and second tile; the caller
// has already issued the loads of the first `in_flight` of them (b only where PREFETCH).  q_s: this tile's queries, [16][Q_STRIDE] bf16 in shared memory.  With
// PREFETCH the loads of the next key tile are in flight while the current one is consumed.
template <bool PREFETCH>
__device__ __forceinline__ void attend(const FaParams& p, const TileGeometry& geo, const PageTable& pt,
                                       const __nv_bfloat16* q_s, int tile_begin, int tile_end, int first, int stride,
                                       int hi_tile, RowState& st, KeyTile& a, KeyTile& b, int in_flight) {
    const int lane = threadIdx.x & 31, g = lane >> 2;
    int pos_row[2], lo_row[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int tok = geo.token_of(g + 8 * i, p.group);
        if (tok < geo.n_new) {
            pos_row[i] = geo.pos0 + tok;
            lo_row[i] = (p.window > 0 && pos_row[i] - p.window + 1 > 0) ? pos_row[i] - p.window + 1 : 0;
        } else {
            pos_row[i] = -1;            // padding row: sees nothing
            lo_row[i] = 0;
        }
    }
    int first_pos = 0x7fffffff, last_lo = 0;
#pragma unroll
    for (int i = 0; i < 2; ++i)
        if (pos_row[i] >= 0) { first_pos = min(first_pos, pos_row[i]); last_lo = max(last_lo, lo_row[i]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        first_pos = min(first_pos, __shfl_xor_sync(0xffffffffu, first_pos, o));
        last_lo = max(last_lo, __shfl_xor_sync(0xffffffffu, last_lo, o));
    }
    int kt = tile_begin + first;
    if (kt >= tile_end) return;
    if (PREFETCH) {
        if (in_flight < 1) load_keys(p, geo, pt, kt, hi_tile, a);
        while (true) {
            const bool more_b = kt + stride < tile_end;
            if (more_b && in_flight < 2) load_keys(p, geo, pt, kt + stride, hi_tile, b);
            in_flight = 0;
            consume_keys(p, q_s, a, pos_row, lo_row, first_pos, last_lo, st);
            if (!more_b) break;
            kt += stride;
            const bool more_a = kt + stride < tile_end;
            if (more_a) load_keys(p, geo, pt, kt + stride, hi_tile, a);
            consume_keys(p, q_s, b, pos_row, lo_row, first_pos, last_lo, st);
            if (!more_a) break;
            kt += stride;
        }
    } else {
        for (; kt < tile_end; kt += stride) {
            if (in_flight < 1) load_keys(p, geo, pt, kt, hi_tile, a);
            in_flight = 0;
            consume_keys(p, q_s, a, pos_row, lo_row, first_pos, last_lo, st);
        }
    }
}

constexpr bool USE_PREFETCH = D <= 128;      // two key tiles in registers do not fit beyond that

__device__ __forceinline__ void init_state(RowState& st) {
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.0f;
#pragma unroll
    for (int nbo = 0; nbo < NB_O; ++nbo)
#pragma unroll
        for (int e = 0; e < 4; ++e) st.o[nbo][e] = 0.0f;
}

// Accumulator o[vb*8 + j][e] of thread (g, t) is output row g (e < 2) or g+8, element
// vb*64 + (2t + (e & 1)) * 8 + j: the thread that fed column n of B read elements n*8 + j.
__device__ __forceinline__ int out_dim(int nbo, int e, int t) {
    return (nbo >> 3) * 64 + (2 * t + (e & 1)) * 8 + (nbo & 7);
}

// ---------------------------------------------------------------------------------- prefill
// One CTA = 4 warps = 4 consecutive row tiles (64 rows) of one (sequence, kv head).  The keys
// are walked 64 at a time; each K/V tile is copied ONCE per CTA from the pages into shared
// memory with cp.async (two stages, the next tile lands while this one is used) and every
// warp takes its tensor-core fragments from there with ldmatrix (transposed for V).  16-byte
// chunks are XOR-swizzled by the key's low bits so that ldmatrix reads are conflict free.
constexpr int KEY_TILE = 64;
constexpr int CHUNKS = D / 8;                       // 16-byte chunks per key row
constexpr int KV_STAGE_ELEMS = 2 * KEY_TILE * D;    // K then V
constexpr int QO_STRIDE = D + 8;                    // bf16; rows shift by one chunk: ldmatrix conflict free
constexpr size_t PREFILL_SMEM = (size_t)(2 * KV_STAGE_ELEMS + WARPS * 16 * QO_STRIDE) * sizeof(__nv_bfloat16) +
                                TABLE_SPAN * sizeof(int);

__device__ __forceinline__ void cp_async16(__nv_bfloat16* dst, const __nv_bfloat16* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;               // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const __nv_bfloat16* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const __nv_bfloat16* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// element offset of 16-byte chunk `chunk` of key row `key` inside a swizzled [KEY_TILE][D] tile
constexpr int SWZ_MASK = CHUNKS >= 8 ? 7 : CHUNKS - 1;
__device__ __forceinline__ int swz(int key, int chunk) { return key * D + ((chunk ^ (key & SWZ_MASK)) << 3); }

// Copy keys [base, base + 64) of (sequence, kv head) into one stage.  Keys outside [lo, hi] --
// behind every row's window (their pages may have been given back) or never written by this
// sequence -- become zeros; a key inside the range without a page raises the error flag.
// Thread `tid` always moves chunk tid % CHUNKS of keys tid / CHUNKS + j * KEYS_PER_PASS.
constexpr int KEYS_PER_PASS = WARPS * 32 / CHUNKS;
constexpr int PASSES = KEY_TILE / KEYS_PER_PASS;
static_assert((WARPS * 32) % CHUNKS == 0 && KEY_TILE % KEYS_PER_PASS == 0, "head size does not tile the copy");

__device__ __forceinline__ void load_kv_stage(const FaParams& p, const PageTable& pt, int kvh, int base, int lo, int hi,
                                              __nv_bfloat16* stage) {
    const size_t page_stride = (size_t)2 * p.num_kv_heads * p.page_size * D;
    const size_t v_off = (size_t)p.num_kv_heads * p.page_size * D;
    const int chunk = threadIdx.x % CHUNKS, key0 = threadIdx.x / CHUNKS;
    const size_t head_off = (size_t)kvh * p.page_size * D + chunk * 8;
#pragma unroll
    for (int j = 0; j < PASSES; ++j) {
        const int key = key0 + j * KEYS_PER_PASS;
        const int pos = base + key;
        const bool wanted = pos >= lo && pos <= hi;
        const int page = wanted ? pt.page_of(pos / p.page_size) : -1;
        const bool ok = page >= 0 && page < p.num_pages;
        if (!ok && wanted && p.error_flag) atomicExch(p.error_flag, 3);
        const __nv_bfloat16* src = p.pages;
        if (ok) src += (size_t)page * page_stride + head_off + (size_t)(pos % p.page_size) * D;
        __nv_bfloat16* dst = stage + swz(key, chunk);
        cp_async16(dst, src, ok);
        cp_async16(dst + KEY_TILE * D, ok ? src + v_off : src, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

__global__ void __launch_bounds__(WARPS * 32, 2) fa_prefill_kernel(FaParams p) {
    pdl_prologue();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* kv_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);                  // [2][K | V][64][D]
    __nv_bfloat16* qo_s = kv_s + 2 * KV_STAGE_ELEMS;                                   // [WARPS][16][QO_STRIDE]
    int* table_s = reinterpret_cast<int*>(qo_s + WARPS * 16 * QO_STRIDE);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    // the CTA's rows: 4 tiles of 16 starting at work item's first tile; warps past the end idle along
    TileGeometry geo;
    geo.seq = p.work[2 * blockIdx.x];
    geo.kvh = blockIdx.y;
    geo.token0 = p.seq_starts[geo.seq];
    geo.n_new = p.seq_starts[geo.seq + 1] - geo.token0;
    geo.pos0 = p.seq_pos0[geo.seq];
    const int first_tile = p.work[2 * blockIdx.x + 1];
    const int total_rows = geo.n_new * p.group;
    geo.row0 = (first_tile + warp) * 16;
    const bool active = geo.row0 < total_rows;
    // key range of the whole CTA (first row's window start .. last row's position)
    const int cta_row_first = first_tile * 16, cta_row_last = min(total_rows, cta_row_first + WARPS * 16) - 1;
    const int cta_first_pos = geo.pos0 + cta_row_first / p.group, cta_last_pos = geo.pos0 + cta_row_last / p.group;
    const int cta_lo = (p.window > 0 && cta_first_pos - p.window + 1 > 0) ? cta_first_pos - p.window + 1 : 0;
    const int tile_first = cta_lo / KEY_TILE, tile_last = cta_last_pos / KEY_TILE;

    PageTable pt;
    {
        const int last_block = cta_last_pos / p.page_size;
        const int first_block = max(cta_lo / p.page_size, last_block - TABLE_SPAN + 1);
        fill_page_table(pt, table_s, p.block_table + (size_t)geo.seq * p.max_blocks, p.max_blocks, first_block, last_block,
                        threadIdx.x, WARPS * 32);
    }
    // queries of this warp's tile -> shared memory (zeros for rows that do not exist)
    __nv_bfloat16* my_q = qo_s + warp * 16 * QO_STRIDE;
    for (int i = lane; i < 16 * CHUNKS; i += 32) {
        const int r = i / CHUNKS, c = (i % CHUNKS) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (active) {
            const int tok = geo.token_of(r, p.group);
            if (tok < geo.n_new) {
                const int head = geo.kvh * p.group + (geo.row0 + r) % p.group;
                v = load16(p.q + ((size_t)(geo.token0 + tok) * p.num_heads + head) * D + c);
            }
        }
        *reinterpret_cast<uint4*>(my_q + r * QO_STRIDE + c) = v;
    }
    __syncthreads();                                   // table and queries are in place
    load_kv_stage(p, pt, geo.kvh, tile_first * KEY_TILE, cta_lo, cta_last_pos, kv_s);

    // this thread's two rows
    int pos_row[2], lo_row[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int tok = geo.token_of(g + 8 * i, p.group);
        if (active && tok < geo.n_new) {
            pos_row[i] = geo.pos0 + tok;
            lo_row[i] = (p.window > 0 && pos_row[i] - p.window + 1 > 0) ? pos_row[i] - p.window + 1 : 0;
        } else {
            pos_row[i] = -1;
            lo_row[i] = 0;
        }
    }
    // the warp's own key range: tiles outside it are skipped (it still keeps step with the CTA)
    const int warp_first_pos = geo.pos0 + geo.token_of(0, p.group);
    const int warp_last_pos = geo.pos0 + min(geo.token_of(15, p.group), geo.n_new - 1);
    const int warp_lo = (p.window > 0 && warp_first_pos - p.window + 1 > 0) ? warp_first_pos - p.window + 1 : 0;
    const int warp_lo_last = (p.window > 0 && warp_last_pos - p.window + 1 > 0) ? warp_last_pos - p.window + 1 : 0;
    const bool warp_rows_full = geo.row0 + 16 <= total_rows;

    // lane-constant parts of the swizzled ldmatrix addresses (row & 7 is the lane's low bits)
    const int lane7 = lane & 7;
    const int k_lane = lane7 * D;                                  // K: key nb*8 + lane7, chunk 2ks + (lane >> 3)
    const int v_lane = (lane7 + ((lane >> 3) & 1) * 8) * D;        // V: key 16kk + lane7 + 8*bit3, chunk nb + (lane >> 4)
    // query fragments stay in registers
    unsigned qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        ldmatrix_x4(qf[ks], my_q + (lane & 15) * QO_STRIDE + ks * 16 + (lane >> 4) * 8);

    float o[D / 8][4];
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nb][e] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    for (int kt = tile_first; kt <= tile_last; ++kt) {
        const int stage = (kt - tile_first) & 1;
        if (kt < tile_last) {
            load_kv_stage(p, pt, geo.kvh, (kt + 1) * KEY_TILE, cta_lo, cta_last_pos, kv_s + (stage ^ 1) * KV_STAGE_ELEMS);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int base = kt * KEY_TILE;
        if (active && base <= warp_last_pos && base + KEY_TILE - 1 >= warp_lo) {
            const __nv_bfloat16* k_s = kv_s + stage * KV_STAGE_ELEMS;
            const __nv_bfloat16* v_s = k_s + KEY_TILE * D;
            // ---- S = Q K^T : 8 key blocks of 8 --------------------------------------------------
            float s[8][4];
#pragma unroll
            for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nb][e] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ks += 2) {
#pragma unroll
                for (int nb = 0; nb < 8; ++nb) {
                    // four 8x8 matrices: this key block at head chunks 2ks, 2ks+1, 2ks+2, 2ks+3
                    unsigned kf[4];
                    ldmatrix_x4(kf, k_s + nb * 8 * D + k_lane + ((((ks * 2) + (lane >> 3)) ^ (lane7 & SWZ_MASK)) << 3));
                    mma_bf16(s[nb], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], kf[0], kf[1]);
                    mma_bf16(s[nb], qf[ks + 1][0], qf[ks + 1][1], qf[ks + 1][2], qf[ks + 1][3], kf[2], kf[3]);
                }
            }
            // ---- masks and the running softmax ----------------------------------------------------
            float mx[2] = {-INFINITY, -INFINITY};
            // a tile that lies inside every row's range (all 16 rows exist) needs no mask
            const bool interior = base + KEY_TILE - 1 <= warp_first_pos && base >= warp_lo_last && warp_rows_full;
            if (interior) {
#pragma unroll
                for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        s[nb][e] *= p.scale_log2;
                        mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
                    }
            } else {
#pragma unroll
                for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = e >> 1;
                        const int key = base + nb * 8 + 2 * t + (e & 1);
                        const bool ok = key >= lo_row[i] && key <= pos_row[i];
                        s[nb][e] = ok ? s[nb][e] * p.scale_log2 : -INFINITY;
                        mx[i] = fmaxf(mx[i], s[nb][e]);
                    }
            }
            float corr[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m_run[i], mx[i]);
                corr[i] = (m_new == -INFINITY) ? 1.0f : exp2f(m_run[i] - m_new);
                m_run[i] = m_new;
            }
            float rowsum[2] = {0.0f, 0.0f};
#pragma unroll
            for (int nb = 0; nb < 8; ++nb)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const float pv = (s[nb][e] == -INFINITY) ? 0.0f : exp2f(s[nb][e] - m_run[i]);
                    s[nb][e] = pv;
                    rowsum[i] += pv;
                }
#pragma unroll
            for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + rowsum[i];
#pragma unroll
            for (int nb = 0; nb < D / 8; ++nb) {
                o[nb][0] *= corr[0]; o[nb][1] *= corr[0];
                o[nb][2] *= corr[1]; o[nb][3] *= corr[1];
            }
            // ---- O += P V : 4 key steps of 16, D/8 output blocks --------------------------------
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const unsigned pa0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                const unsigned pa1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                const unsigned pa2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                const unsigned pa3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int nb = 0; nb < D / 8; nb += 2) {
                    // four 8x8 matrices, transposed on the way: keys 16kk..+7 / +8..15 at output chunks nb, nb+1
                    unsigned vf[4];
                    ldmatrix_x4_trans(vf, v_s + kk * 16 * D + v_lane + (((nb + (lane >> 4)) ^ (lane7 & SWZ_MASK)) << 3));
                    mma_bf16(o[nb], pa0, pa1, pa2, pa3, vf[0], vf[1]);
                    mma_bf16(o[nb + 1], pa0, pa1, pa2, pa3, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();                               // the stage may be overwritten next round
    }
    if (!active) return;
    // normalise and write through shared memory so that rows leave as whole 16-byte pieces
    float inv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float l = l_run[i];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        inv[i] = l > 0.0f ? 1.0f / l : 0.0f;
    }
    __syncwarp();
#pragma unroll
    for (int nb = 0; nb < D / 8; ++nb) {
        *reinterpret_cast<__nv_bfloat162*>(my_q + g * QO_STRIDE + nb * 8 + 2 * t) =
            __floats2bfloat162_rn(o[nb][0] * inv[0], o[nb][1] * inv[0]);
        *reinterpret_cast<__nv_bfloat162*>(my_q + (g + 8) * QO_STRIDE + nb * 8 + 2 * t) =
            __floats2bfloat162_rn(o[nb][2] * inv[1], o[nb][3] * inv[1]);
    }
    __syncwarp();
    for (int i = lane; i < 16 * CHUNKS; i += 32) {
        const int r = i / CHUNKS, c = (i % CHUNKS) * 8;
        const int tok = geo.token_of(r, p.group);
        if (tok >= geo.n_new) continue;
        const int head = geo.kvh * p.group + (geo.row0 + r) % p.group;
        *reinterpret_cast<uint4*>(p.out + ((size_t)(geo.token0 + tok) * p.num_heads + head) * D + c) =
            *reinterpret_cast<const uint4*>(my_q + r * QO_STRIDE + c);
    }
}

// ---------------------------------------------------------------------------------- decode
// Every sequence brings ONE token.  A thread-block CLUSTER of `splits` CTAs (1, 2, 4 or 8)
// shares the keys of one (sequence, kv head, row tile): each CTA walks an even share of the
// key tiles, its four warps are merged in its own shared memory, and after one cluster barrier
// every CTA combines a slice of the head dimension by reading the other CTAs' results through
// distributed shared memory.  Nothing is staged in global memory and no second launch or
// atomic is needed; the sum over CTAs always runs in rank order.
constexpr int FRAGS = NB_O * 4;
constexpr int MAX_SPLITS = 16;            // clusters beyond 8 CTAs are the non-portable size, allowed on this GPU
// shared memory (dynamic): queries | per-warp fragments [DW][FRAGS][32] | warp max/sum |
// this CTA's merged rows [16][D] with their max and sum | block table
constexpr size_t decode_smem(int dw) {
    return 16 * Q_STRIDE * sizeof(__nv_bfloat16) + (size_t)dw * FRAGS * 32 * sizeof(float) + 2 * dw * 16 * sizeof(float) +
           (size_t)16 * D * sizeof(float) + 32 * sizeof(float) + TABLE_SPAN * sizeof(int);
}

// DW warps per CTA: 4 (two CTAs per SM, large batches) or 8 (few sequences: more warps, so that each
// has at most a couple of key tiles and all their loads are in flight at once)
template <int DW>
__global__ void __launch_bounds__(DW * 32, DW == 4 ? 2 : 1) fa_decode_kernel(FaParams p) {
    pdl_launch_dependents();       // the wait comes after the sequence's length and block table are on their way
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    float* frag = reinterpret_cast<float*>(smem_raw + 16 * Q_STRIDE * sizeof(__nv_bfloat16));   // [DW][FRAGS][32]
    float* warp_m = frag + DW * FRAGS * 32;        // [DW][16]
    float* warp_l = warp_m + DW * 16;              // [DW][16]
    float* cta_o = warp_l + DW * 16;               // [16][D]  this CTA's rows, scaled to cta_m
    float* cta_m = cta_o + 16 * D;                    // [16]
    float* cta_l = cta_m + 16;                        // [16]
    int* table_s = reinterpret_cast<int*>(cta_l + 16);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    // one token per sequence: the work item is (sequence, row tile) = blockIdx.x, no lookup
    const int tiles_per_seq = (p.group + 15) / 16;
    TileGeometry geo;
    geo.seq = blockIdx.x / tiles_per_seq;
    if (p.listed) geo.seq = __ldg(p.work + geo.seq);          // (the step's own lists come from the host: no wait needed)
    geo.kvh = blockIdx.y;
    geo.token0 = p.listed ? __ldg(p.seq_starts + geo.seq) : geo.seq;
    geo.n_new = 1;
    geo.row0 = (blockIdx.x % tiles_per_seq) * 16;
    const int rows_valid = min(16, p.group - geo.row0);
    const bool upper = rows_valid > 8;
    // First trip to memory: the sequence's length and its block table.  Neither is written by the kernels
    // just before this one (they come from the host or from the end of the step before), so they are
    // fetched before the wait for the predecessor; the queries, which it wrote, after it.
    const int pos0_load = __ldg(p.seq_pos0 + geo.seq);
    PageTable pt;
    fill_page_table(pt, table_s, p.block_table + (size_t)geo.seq * p.max_blocks, p.max_blocks, 0, p.max_blocks - 1,
                    threadIdx.x, DW * 32);
    geo.pos0 = pos0_load;
    const int last_pos = geo.pos0;
    const int lo = (p.window > 0 && last_pos - p.window + 1 > 0) ? last_pos - p.window + 1 : 0;
    int tile_begin = lo / 16, tile_end = last_pos / 16 + 1;
    const int splits = (int)gridDim.z, rank = (int)blockIdx.z;
    if (splits > 1) {                        // this CTA's even share of the sequence's key tiles
        const int per_split = (tile_end - tile_begin + splits - 1) / splits;
        tile_begin += rank * per_split;
        tile_end = min(tile_end, tile_begin + per_split);
    }
    __syncthreads();                         // the block table is in shared memory
    // Second trip, still before the wait: this warp's first key tile, unless it holds the new token's
    // key, which the kernel before this one is writing.
    KeyTile tile_a, tile_b;
    const int first_kt = tile_begin + warp;
    int early = 0;
    if (first_kt < tile_end && first_kt < last_pos / 16) {
        load_keys(p, geo, pt, first_kt, last_pos, tile_a);
        early = 1;
        if (USE_PREFETCH && first_kt + DW < tile_end && first_kt + DW < last_pos / 16) {
            load_keys(p, geo, pt, first_kt + DW, last_pos, tile_b);
            early = 2;
        }
    }
    pdl_wait();
    {
        constexpr int VEC_PER_ROW = D / 8;
        for (int i = threadIdx.x; i < 16 * VEC_PER_ROW; i += DW * 32) {
            const int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < rows_valid) {
                const int head = geo.kvh * p.group + geo.row0 + r;
                v = load16(p.q + ((size_t)geo.token0 * p.num_heads + head) * D + c);
            }
            *reinterpret_cast<uint4*>(q_s + r * Q_STRIDE + c) = v;
        }
    }
    __syncthreads();
    RowState st;
    init_state(st);
    attend<USE_PREFETCH>(p, geo, pt, q_s, tile_begin, tile_end, warp, DW, last_pos, st, tile_a, tile_b, early);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 1);
        st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 2);
    }
    // every warp publishes its fragments, then each thread merges a quarter of them
#pragma unroll
    for (int nbo = 0; nbo < NB_O; ++nbo) {
        frag[(warp * FRAGS + nbo * 4 + 0) * 32 + lane] = st.o[nbo][0];
        frag[(warp * FRAGS + nbo * 4 + 1) * 32 + lane] = st.o[nbo][1];
        if (upper) {
            frag[(warp * FRAGS + nbo * 4 + 2) * 32 + lane] = st.o[nbo][2];
            frag[(warp * FRAGS + nbo * 4 + 3) * 32 + lane] = st.o[nbo][3];
        }
    }
    if (t == 0) {
        warp_m[warp * 16 + g] = st.m[0]; warp_m[warp * 16 + g + 8] = st.m[1];
        warp_l[warp * 16 + g] = st.l[0]; warp_l[warp * 16 + g + 8] = st.l[1];
    }
    __syncthreads();
    float scale_w[2][DW];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        float m_all = -INFINITY;
#pragma unroll
        for (int w = 0; w < DW; ++w) m_all = fmaxf(m_all, warp_m[w * 16 + r]);
        float l_all = 0.0f;
#pragma unroll
        for (int w = 0; w < DW; ++w) {
            const float mw = warp_m[w * 16 + r];
            scale_w[i][w] = (mw == -INFINITY) ? 0.0f : exp2f(mw - m_all);
            l_all += warp_l[w * 16 + r] * scale_w[i][w];
        }
        if (warp == 0 && t == 0) { cta_m[r] = m_all; cta_l[r] = l_all; }
    }
#pragma unroll
    for (int k = 0; k < FRAGS / DW; ++k) {
        const int idx = warp + k * DW;              // this thread merges fragment idx of all warps
        const int nbo = idx >> 2, e = idx & 3, i = e >> 1, r = g + 8 * i;
        const int dim = out_dim(nbo, e, t);
        if (dim >= D || r >= rows_valid) continue;
        float val = 0.0f;
#pragma unroll
        for (int w = 0; w < DW; ++w) val += frag[(w * FRAGS + idx) * 32 + lane] * scale_w[i][w];
        cta_o[r * D + dim] = val;
    }
    // across the cluster: CTA `rank` finishes the slice [rank, rank + 1) * D / splits of every row
    cluster.sync();
    const int slice = D / splits;
    for (int i = threadIdx.x; i < rows_valid * slice; i += DW * 32) {
        const int r = i / slice, dim = rank * slice + i % slice;
        float m_all = -INFINITY;
        float ms[MAX_SPLITS];
#pragma unroll
        for (int s2 = 0; s2 < MAX_SPLITS; ++s2) {
            ms[s2] = -INFINITY;
            if (s2 < splits) ms[s2] = *cluster.map_shared_rank(cta_m + r, s2);
            m_all = fmaxf(m_all, ms[s2]);
        }
        float acc = 0.0f, l_all = 0.0f;
#pragma unroll
        for (int s2 = 0; s2 < MAX_SPLITS; ++s2) {
            if (s2 < splits && ms[s2] != -INFINITY) {
                const float w = exp2f(ms[s2] - m_all);
                acc += w * *cluster.map_shared_rank(cta_o + r * D + dim, s2);
                l_all += w * *cluster.map_shared_rank(cta_l + r, s2);
            }
        }
        const int head = geo.kvh * p.group + geo.row0 + r;
        p.out[((size_t)geo.token0 * p.num_heads + head) * D + dim] = __float2bfloat16_rn(l_all > 0.0f ? acc / l_all : 0.0f);
    }
    cluster.sync();                          // nobody leaves while its shared memory may still be read
}


// ---------------------------------------------------------------------------------- decode, keys on the M side
// The same work as fa_decode_kernel for groups of at most 8 query heads, with the roles of the MMA
// operands swapped so that the 16-row side carries KEYS and the 8-column side the group's heads:
//     S^T[16 keys, 8 heads] = K[16 keys, D] Q^T          (K straight from the page as the A operand, as a
//                                                        weight in the streaming products; Q^T from shared memory)
//     O^T[D, 8 heads]      += V^T[D, 16 keys] P^T        (V^T fragments by byte permutes of the same 16-byte loads;
//                                                        P^T moves from accumulator to B-operand layout by 4 shuffles)
// A 16-row tile of the other kernel carries 6 real rows for this model; here nothing is padding but two of
// eight columns: half the MMAs, half the accumulator registers, half the exponentials per key.
constexpr int NPAIR = (VBLOCKS + 1) / 2;    // pairs of 64-element value blocks: one MMA covers 16 rows = 8 + 8 elements
constexpr int FRAGS_T = NPAIR * 8 * 4;

struct RowStateT {
    float m[2];               // reference maximum of heads 2t and 2t+1 (equal in all lanes of the same t)
    float l[2];               // this thread's share (its own keys) of the running sums
    float o[NPAIR * 8][4];    // [pair*8 + j]: e < 2: element vb0*64 + 8g + j, e >= 2: element vb1*64 + 8g + j; head 2t + (e & 1)
};

// INTERLEAVED: which 8 head elements of a 32-element chunk pair a thread takes.  Plain: chunk c, elements
// c*32 + t*8.  Interleaved (keys read from the swizzled ring): of every 64 elements the thread takes the 16-byte
// pieces 2t and 2t+1 in turn, so that the four threads of a quad touch every second piece and the two key rows
// of a quarter warp fall into different banks.  K and Q only have to agree.
template <bool INTERLEAVED>
__device__ __forceinline__ int k_column(int c, int t) {
    return INTERLEAVED ? (c >> 1) * 64 + ((t << 1) | (c & 1)) * 8 : c * 32 + t * 8;
}

template <bool INTERLEAVED = false>
__device__ __forceinline__ void consume_keys_t(const FaParams& p, const __nv_bfloat16* q_s, const KeyTile& kv, int last_pos,
                                               int lo, RowStateT& st) {
    if (kv.base < 0) return;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    float s0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s1[4] = {0.0f, 0.0f, 0.0f, 0.0f};     // two chains
#pragma unroll
    for (int c = 0; c < KCHUNKS; ++c) {
        const uint4 q = *reinterpret_cast<const uint4*>(q_s + g * Q_STRIDE + k_column<INTERLEAVED>(c, t));       // head g
        mma_bf16(s0, kv.k[0][c].x, kv.k[1][c].x, kv.k[0][c].y, kv.k[1][c].y, q.x, q.y);
        mma_bf16(s1, kv.k[0][c].z, kv.k[1][c].z, kv.k[0][c].w, kv.k[1][c].w, q.z, q.w);
    }
    // s[0], s[1]: key base + g, heads 2t, 2t+1;   s[2], s[3]: key base + g + 8
    float s[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] = (s0[e] + s1[e]) * p.scale_log2;
    if (kv.base + 15 > last_pos || kv.base < lo) {         // an edge tile (uniform over the warp)
        const int key0 = kv.base + g, key1 = key0 + 8;
        if (key0 < lo || key0 > last_pos) s[0] = s[1] = -INFINITY;
        if (key1 < lo || key1 > last_pos) s[2] = s[3] = -INFINITY;
    }
    float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
    float corr[2];
    bool grow = false;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 4));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 8));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 16));
        const bool g_i = mx[i] > st.m[i] + RESCALE_STEP;          // true as well for the first finite maximum
        corr[i] = g_i ? (st.m[i] == -INFINITY ? 0.0f : fast_exp2(st.m[i] - mx[i])) : 1.0f;
        st.m[i] = g_i ? mx[i] : st.m[i];
        grow |= g_i;
    }
    const float ref0 = st.m[0] == -INFINITY ? 0.0f : st.m[0], ref1 = st.m[1] == -INFINITY ? 0.0f : st.m[1];
    const float p0 = fast_exp2(s[0] - ref0), p1 = fast_exp2(s[1] - ref1), p2 = fast_exp2(s[2] - ref0), p3 = fast_exp2(s[3] - ref1);
    if (__any_sync(0xffffffffu, grow)) {
        st.l[0] *= corr[0];
        st.l[1] *= corr[1];
#pragma unroll
        for (int k = 0; k < NPAIR * 8; ++k) {
            st.o[k][0] *= corr[0]; st.o[k][1] *= corr[1];
            st.o[k][2] *= corr[0]; st.o[k][3] *= corr[1];
        }
    }
    st.l[0] += p0 + p2;
    st.l[1] += p1 + p3;
    // P^T from accumulator layout (keys on g, heads on t) to B-operand layout (keys on t, head g): lane (g, t)
    // takes head g's probabilities of keys 2t, 2t+8 from lane (2t, g/2) and of keys 2t+1, 2t+9 from lane (2t+1, g/2)
    const unsigned u_even = pack_bf16(p0, p2), u_odd = pack_bf16(p1, p3);      // (key g, key g+8) of head 2t / 2t+1
    const int src1 = (2 * t) * 4 + (g >> 1), src2 = src1 + 4;
    const unsigned e1 = __shfl_sync(0xffffffffu, u_even, src1), o1 = __shfl_sync(0xffffffffu, u_odd, src1);
    const unsigned e2 = __shfl_sync(0xffffffffu, u_even, src2), o2 = __shfl_sync(0xffffffffu, u_odd, src2);
    const unsigned w1 = (g & 1) ? o1 : e1, w2 = (g & 1) ? o2 : e2;
    const unsigned b0 = __byte_perm(w1, w2, 0x5410u);       // keys 2t, 2t+1
    const unsigned b1 = __byte_perm(w1, w2, 0x7632u);       // keys 2t+8, 2t+9
#pragma unroll
    for (int pp = 0; pp < NPAIR; ++pp) {
        const int vb0 = 2 * pp, vb1 = 2 * pp + 1;
        const unsigned* x0 = reinterpret_cast<const unsigned*>(&kv.v[vb0][0]);
        const unsigned* x1 = reinterpret_cast<const unsigned*>(&kv.v[vb0][1]);
        const unsigned* x2 = reinterpret_cast<const unsigned*>(&kv.v[vb0][2]);
        const unsigned* x3 = reinterpret_cast<const unsigned*>(&kv.v[vb0][3]);
        const unsigned* y0 = reinterpret_cast<const unsigned*>(&kv.v[vb1 < VBLOCKS ? vb1 : vb0][0]);
        const unsigned* y1 = reinterpret_cast<const unsigned*>(&kv.v[vb1 < VBLOCKS ? vb1 : vb0][1]);
        const unsigned* y2 = reinterpret_cast<const unsigned*>(&kv.v[vb1 < VBLOCKS ? vb1 : vb0][2]);
        const unsigned* y3 = reinterpret_cast<const unsigned*>(&kv.v[vb1 < VBLOCKS ? vb1 : vb0][3]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned sel = (j & 1) ? 0x7632u : 0x5410u;       // high or low bf16 of both words
            const unsigned a0 = __byte_perm(x0[j >> 1], x1[j >> 1], sel);     // element vb0*64 + 8g + j of keys 2t, 2t+1
            const unsigned a2 = __byte_perm(x2[j >> 1], x3[j >> 1], sel);     // ... of keys 2t+8, 2t+9
            const unsigned a1 = vb1 < VBLOCKS ? __byte_perm(y0[j >> 1], y1[j >> 1], sel) : 0u;
            const unsigned a3 = vb1 < VBLOCKS ? __byte_perm(y2[j >> 1], y3[j >> 1], sel) : 0u;
            mma_bf16(st.o[pp * 8 + j], a0, a1, a2, a3, b0, b1);
        }
    }
}

// What follows the key loop of the keys-on-M decode kernels: the warps of a CTA merge their shares in shared
// memory, then the CTAs of the cluster merge theirs through distributed shared memory, CTA `rank` finishing the
// slice [rank, rank + 1) * D / splits of every head.  Every thread of the CTA calls it (it holds CTA- and
// cluster-wide barriers); `active` is false for threads of a warp that walked no keys (a copy-issuing warp).
template <int DW>
__device__ __forceinline__ void merge_and_store_t(const FaParams& p, const TileGeometry& geo, RowStateT& st, float* frag,
                                                  float* warp_m, float* warp_l, float* cta_o, float* cta_m, float* cta_l,
                                                  int heads, int splits, int rank, bool active) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (active) {
        // a head's sum over this warp's keys: the lanes of equal t hold its shares
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 4);
            st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 8);
            st.l[i] += __shfl_xor_sync(0xffffffffu, st.l[i], 16);
        }
        // every warp publishes its fragments, then each thread merges a share of them
#pragma unroll
        for (int k = 0; k < NPAIR * 8; ++k)
#pragma unroll
            for (int e = 0; e < 4; ++e) frag[(warp * FRAGS_T + k * 4 + e) * 32 + lane] = st.o[k][e];
        if (g == 0) {
            warp_m[warp * 8 + 2 * t] = st.m[0]; warp_m[warp * 8 + 2 * t + 1] = st.m[1];
            warp_l[warp * 8 + 2 * t] = st.l[0]; warp_l[warp * 8 + 2 * t + 1] = st.l[1];
        }
    }
    __syncthreads();
    if (active) {
        float scale_w[2][DW];                    // of heads 2t and 2t+1
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int h = 2 * t + i;
            float m_all = -INFINITY;
#pragma unroll
            for (int w = 0; w < DW; ++w) m_all = fmaxf(m_all, warp_m[w * 8 + h]);
            float l_all = 0.0f;
#pragma unroll
            for (int w = 0; w < DW; ++w) {
                const float mw = warp_m[w * 8 + h];
                scale_w[i][w] = (mw == -INFINITY) ? 0.0f : exp2f(mw - m_all);
                l_all += warp_l[w * 8 + h] * scale_w[i][w];
            }
            if (warp == 0 && g == 0) { cta_m[h] = m_all; cta_l[h] = l_all; }
        }
#pragma unroll
        for (int k = 0; k < FRAGS_T / DW; ++k) {
            const int idx = warp + k * DW;              // this thread merges fragment idx of all warps
            const int kk = idx >> 2, e = idx & 3, i = e & 1, h = 2 * t + i;
            const int dim = (2 * (kk >> 3) + (e >> 1)) * 64 + 8 * g + (kk & 7);
            if (dim >= D || h >= heads) continue;
            float val = 0.0f;
#pragma unroll
            for (int w = 0; w < DW; ++w) val += frag[(w * FRAGS_T + idx) * 32 + lane] * scale_w[i][w];
            cta_o[h * D + dim] = val;
        }
    }
    // across the cluster: CTA `rank` finishes the slice [rank, rank + 1) * D / splits of every head
    cluster.sync();
    const int slice = D / splits;
    for (int i = active ? (int)threadIdx.x : heads * slice; i < heads * slice; i += DW * 32) {
        const int r = i / slice, dim = rank * slice + i % slice;
        float m_all = -INFINITY;
        float ms[MAX_SPLITS];
#pragma unroll
        for (int s2 = 0; s2 < MAX_SPLITS; ++s2) {
            ms[s2] = -INFINITY;
            if (s2 < splits) ms[s2] = *cluster.map_shared_rank(cta_m + r, s2);
            m_all = fmaxf(m_all, ms[s2]);
        }
        float acc = 0.0f, l_all = 0.0f;
#pragma unroll
        for (int s2 = 0; s2 < MAX_SPLITS; ++s2) {
            if (s2 < splits && ms[s2] != -INFINITY) {
                const float w = exp2f(ms[s2] - m_all);
                acc += w * *cluster.map_shared_rank(cta_o + r * D + dim, s2);
                l_all += w * *cluster.map_shared_rank(cta_l + r, s2);
            }
        }
        const int head = geo.kvh * p.group + r;
        p.out[((size_t)geo.token0 * p.num_heads + head) * D + dim] = __float2bfloat16_rn(l_all > 0.0f ? acc / l_all : 0.0f);
    }
    cluster.sync();                          // nobody leaves while its shared memory may still be read
}

// shared memory (dynamic): queries | per-warp fragments [DW][FRAGS_T][32] | warp max/sum per head |
// this CTA's merged heads [8][D] with their max and sum | block table
constexpr size_t decode_t_smem(int dw) {
    return 16 * Q_STRIDE * sizeof(__nv_bfloat16) + (size_t)dw * FRAGS_T * 32 * sizeof(float) + 2 * dw * 8 * sizeof(float) +
           (size_t)8 * D * sizeof(float) + 16 * sizeof(float) + TABLE_SPAN * sizeof(int);
}

template <int DW>
__global__ void __launch_bounds__(DW * 32, DW == 4 ? 2 : 1) fa_decode_t_kernel(FaParams p) {
    pdl_launch_dependents();       // the wait comes after the sequence's length, block table and first keys are on their way
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);                             // [8 heads used of 16][Q_STRIDE]
    float* frag = reinterpret_cast<float*>(smem_raw + 16 * Q_STRIDE * sizeof(__nv_bfloat16));   // [DW][FRAGS_T][32]
    float* warp_m = frag + DW * FRAGS_T * 32;      // [DW][8]
    float* warp_l = warp_m + DW * 8;               // [DW][8]
    float* cta_o = warp_l + DW * 8;                // [8][D]  this CTA's heads, scaled to cta_m
    float* cta_m = cta_o + 8 * D;                  // [8]
    float* cta_l = cta_m + 8;                      // [8]
    int* table_s = reinterpret_cast<int*>(cta_l + 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

    // one token per sequence and at most 8 heads per group: the work item is the sequence = blockIdx.x
    TileGeometry geo;
    geo.seq = p.listed ? __ldg(p.work + blockIdx.x) : (int)blockIdx.x;   // (the step's own lists come from the host: no wait needed)
    geo.kvh = blockIdx.y;
    geo.token0 = p.listed ? __ldg(p.seq_starts + geo.seq) : geo.seq;
    geo.n_new = 1;
    geo.row0 = 0;
    const int heads = p.group;                     // <= 8
    const int pos0_load = __ldg(p.seq_pos0 + geo.seq);
    PageTable pt;
    fill_page_table(pt, table_s, p.block_table + (size_t)geo.seq * p.max_blocks, p.max_blocks, 0, p.max_blocks - 1,
                    threadIdx.x, DW * 32);
    geo.pos0 = pos0_load;
    const int last_pos = geo.pos0;
    const int lo = (p.window > 0 && last_pos - p.window + 1 > 0) ? last_pos - p.window + 1 : 0;
    int tile_begin = lo / 16, tile_end = last_pos / 16 + 1;
    const int splits = (int)gridDim.z, rank = (int)blockIdx.z;
    if (splits > 1) {                        // this CTA's even share of the sequence's key tiles
        const int per_split = (tile_end - tile_begin + splits - 1) / splits;
        tile_begin += rank * per_split;
        tile_end = min(tile_end, tile_begin + per_split);
    }
    __syncthreads();                         // the block table is in shared memory
    // still before the wait: this warp's first key tiles, unless they hold the new token's key
    KeyTile tile_a, tile_b;
    int kt = tile_begin + warp;
    int in_flight = 0;
    if (kt < tile_end && kt < last_pos / 16) {
        load_keys(p, geo, pt, kt, last_pos, tile_a);
        in_flight = 1;
        if (USE_PREFETCH && kt + DW < tile_end && kt + DW < last_pos / 16) {
            load_keys(p, geo, pt, kt + DW, last_pos, tile_b);
            in_flight = 2;
        }
    }
    pdl_wait();
    {
        constexpr int VEC_PER_ROW = D / 8;
        for (int i = threadIdx.x; i < 8 * VEC_PER_ROW; i += DW * 32) {
            const int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < heads) v = load16(p.q + ((size_t)geo.token0 * p.num_heads + geo.kvh * p.group + r) * D + c);
            *reinterpret_cast<uint4*>(q_s + r * Q_STRIDE + c) = v;
        }
    }
    __syncthreads();
    RowStateT st;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.0f;
#pragma unroll
    for (int k = 0; k < NPAIR * 8; ++k)
#pragma unroll
        for (int e = 0; e < 4; ++e) st.o[k][e] = 0.0f;
    if (kt < tile_end) {
        if (USE_PREFETCH) {
            if (in_flight < 1) load_keys(p, geo, pt, kt, last_pos, tile_a);
            while (true) {
                const bool more_b = kt + DW < tile_end;
                if (more_b && in_flight < 2) load_keys(p, geo, pt, kt + DW, last_pos, tile_b);
                in_flight = 0;
                consume_keys_t(p, q_s, tile_a, last_pos, lo, st);
                if (!more_b) break;
                kt += DW;
                const bool more_a = kt + DW < tile_end;
                if (more_a) load_keys(p, geo, pt, kt + DW, last_pos, tile_a);
                consume_keys_t(p, q_s, tile_b, last_pos, lo, st);
                if (!more_a) break;
                kt += DW;
            }
        } else {
            for (; kt < tile_end; kt += DW) {
                if (in_flight < 1) load_keys(p, geo, pt, kt, last_pos, tile_a);
                in_flight = 0;
                consume_keys_t(p, q_s, tile_a, last_pos, lo, st);
            }
        }
    }
    merge_and_store_t<DW>(p, geo, st, frag, warp_m, warp_l, cta_o, cta_m, cta_l, heads, splits, rank, true);
}


// ---------------------------------------------------------------------------------- decode, keys through a ring
// The keys-on-M decode kernel again, for steps that read much more than a few megabytes of keys (many
// sequences, long contexts).  There the kernel above is bound by what its warps can keep in flight: two key
// tiles of registers per warp, the second one's loads only issued while the first is being used.  Here a fifth
// warp issues the copies: TMA (cp.async.bulk.tensor, 128-byte swizzle) brings the K and V of 64 keys per stage
// into a ring of RING_STAGES stages of shared memory, as far ahead of the four working warps as the ring is
// deep and without a register of theirs.  A working warp takes its 16 keys of a stage out of the ring with
// 16-byte loads in exactly the fragment layout the kernel above loads from global memory (the swizzle makes
// them conflict-free), hands the stage back at once, and runs the same consume_keys_t.  The merge over warps and
// over the cluster is the same function.  Heads of 128 elements.
constexpr int RING_STAGES = 3;
constexpr int RING_TILE_BYTES = 16 * D * 2;                 // the K (or V) of one 16-key tile
constexpr int RING_STAGE_BYTES = 4 * 2 * RING_TILE_BYTES;   // four tiles, K and V: 32 KB at D = 128
constexpr int RING_SPIN_LIMIT = 1 << 22;

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
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
    return ok != 0;
}
// false when the bound was hit: the caller stops waiting, the flag tells the host
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* error_flag, int code) {
    for (int i = 0; i < RING_SPIN_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (error_flag) atomicExch(error_flag, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// 16 bytes of a [16 rows x 64 elements] box as TMA's 128-byte swizzle laid it out: 16-byte chunk `chunk` of row
// `row` sits at chunk ^ (row % 8)
__device__ __forceinline__ uint4 ring_load16(const unsigned char* box, int row, int chunk) {
    return *reinterpret_cast<const uint4*>(box + row * 128 + ((chunk ^ (row & 7)) << 4));
}

// this warp's 16 keys of a stage, from the ring into the registers consume_keys_t wants (see load_keys)
__device__ __forceinline__ void ring_take_keys(const unsigned char* tile, int base, int last_pos, KeyTile& kv) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    kv.base = base;
    const unsigned char* kbox = tile;                             // [span (D / 64)][16 rows][128 bytes]
    const unsigned char* vbox = tile + RING_TILE_BYTES;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int c = 0; c < KCHUNKS; ++c) kv.k[nb][c] = ring_load16(kbox + (c >> 1) * (16 * 128), nb * 8 + g, (t << 1) | (c & 1));     // k_column<true>
#pragma unroll
    for (int vb = 0; vb < VBLOCKS; ++vb)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int key = 2 * t + (r & 1) + 8 * (r >> 1);       // this thread's keys: 2t, 2t+1, 2t+8, 2t+9
            // slots behind the sequence's last key were never written: zero, so that zero probability times them stays zero
            kv.v[vb][r] = base + key <= last_pos ? ring_load16(vbox + vb * (16 * 128), key, g) : make_uint4(0, 0, 0, 0);
        }
}

constexpr size_t decode_ring_smem() {
    // ring (1024-byte aligned; the per-warp fragments of the merge reuse it) | queries | warp max/sum | merged heads | table
    return 1024 + (size_t)RING_STAGES * RING_STAGE_BYTES + 16 * Q_STRIDE * sizeof(__nv_bfloat16) + 2 * 4 * 8 * sizeof(float) +
           (size_t)8 * D * sizeof(float) + 16 * sizeof(float) + TABLE_SPAN * sizeof(int);
}

__global__ void __launch_bounds__(160, 2) fa_decode_ring_kernel(const __grid_constant__ CUtensorMap map_kv, FaParams p) {
    pdl_launch_dependents();
    constexpr int DW = 4;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long full_bar[RING_STAGES], empty_bar[RING_STAGES];
    unsigned char* ring = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    float* frag = reinterpret_cast<float*>(ring);                  // [DW][FRAGS_T][32], once the ring is drained
    static_assert((size_t)DW * FRAGS_T * 32 * sizeof(float) <= (size_t)RING_STAGES * RING_STAGE_BYTES, "the merge's fragments must fit the ring");
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(ring + RING_STAGES * RING_STAGE_BYTES);
    float* warp_m = reinterpret_cast<float*>(q_s + 16 * Q_STRIDE);     // [DW][8]
    float* warp_l = warp_m + DW * 8;
    float* cta_o = warp_l + DW * 8;                // [8][D]
    float* cta_m = cta_o + 8 * D;
    float* cta_l = cta_m + 8;
    int* table_s = reinterpret_cast<int*>(cta_l + 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    TileGeometry geo;
    geo.seq = p.listed ? __ldg(p.work + blockIdx.x) : (int)blockIdx.x;
    geo.kvh = blockIdx.y;
    geo.token0 = p.listed ? __ldg(p.seq_starts + geo.seq) : geo.seq;
    geo.n_new = 1;
    geo.row0 = 0;
    const int heads = p.group;                     // <= 8
    const int pos0_load = __ldg(p.seq_pos0 + geo.seq);
    PageTable pt;
    fill_page_table(pt, table_s, p.block_table + (size_t)geo.seq * p.max_blocks, p.max_blocks, 0, p.max_blocks - 1,
                    threadIdx.x, 160);
    if (threadIdx.x == 0) {
        for (int s = 0; s < RING_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), DW);           // one arrival per working warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    geo.pos0 = pos0_load;
    const int last_pos = geo.pos0;
    const int lo = (p.window > 0 && last_pos - p.window + 1 > 0) ? last_pos - p.window + 1 : 0;
    int tile_begin = lo / 16, tile_end = last_pos / 16 + 1;
    const int splits = (int)gridDim.z, rank = (int)blockIdx.z;
    if (splits > 1) {                        // this CTA's even share of the sequence's key tiles
        const int per_split = (tile_end - tile_begin + splits - 1) / splits;
        tile_begin += rank * per_split;
        tile_end = min(tile_end, tile_begin + per_split);
    }
    const int num_stages = tile_end > tile_begin ? (tile_end - tile_begin + 3) / 4 : 0;      // 64 keys each
    __syncthreads();                         // the block table and the barriers are in shared memory

    RowStateT st;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.0f;
#pragma unroll
    for (int k = 0; k < NPAIR * 8; ++k)
#pragma unroll
        for (int e = 0; e < 4; ++e) st.o[k][e] = 0.0f;

    if (warp == DW) {
        // ---------------------------------------------------------------- the copying warp
        if (lane == 0) {
            bool waited = false, ok = true;
            int issued = 0;
            for (int i = 0; i < num_stages && ok; ++i) {
                lag_point();
                const int s = i % RING_STAGES;
                if (i >= RING_STAGES && !mbar_wait(smem_u32(&empty_bar[s]), ((i / RING_STAGES) - 1) & 1, p.error_flag, 61)) { ok = false; break; }
                const int kt0 = tile_begin + 4 * i, n_tiles = min(4, tile_end - kt0);
                // the tile that holds the new token's key was written by the kernel in front: everything before it
                // travels while that kernel still runs
                if (!waited && kt0 + n_tiles > last_pos / 16) { pdl_wait(); waited = true; }
                uint32_t bytes = 0;
                int page_of_tile[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    page_of_tile[j] = -1;
                    if (j < n_tiles) {
                        const int base = (kt0 + j) * 16;
                        const int page = pt.page_of(p.page_shift >= 0 ? base >> p.page_shift : base / p.page_size);
                        if (page >= 0 && page < p.num_pages) { page_of_tile[j] = page; bytes += 2 * RING_TILE_BYTES; }
                    }
                }
                const uint32_t bar = smem_u32(&full_bar[s]);
                if (bytes == 0) { mbar_arrive(bar); issued = i + 1; continue; }        // nothing to copy: the stage is "full" at once
                mbar_expect_tx(bar, bytes);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (page_of_tile[j] < 0) continue;
                    const int base = (kt0 + j) * 16;
                    const int slot = p.page_shift >= 0 ? base & (p.page_size - 1) : base % p.page_size;
                    const int row_k = ((page_of_tile[j] * 2) * p.num_kv_heads + geo.kvh) * p.page_size + slot;
                    const int row_v = row_k + p.num_kv_heads * p.page_size;
                    const uint32_t dst = smem_u32(ring) + s * RING_STAGE_BYTES + j * 2 * RING_TILE_BYTES;
#pragma unroll
                    for (int span = 0; span < D / 64; ++span) {
                        tma_load_2d(dst + span * (16 * 128), &map_kv, span * 64, row_k, bar);
                        tma_load_2d(dst + RING_TILE_BYTES + span * (16 * 128), &map_kv, span * 64, row_v, bar);
                    }
                }
                issued = i + 1;
            }
            if (!ok) {
                // given up: let the copies already issued land before the shared memory is handed back
                for (int i = max(0, issued - RING_STAGES); i < issued; ++i)
                    mbar_wait(smem_u32(&full_bar[i % RING_STAGES]), (i / RING_STAGES) & 1, nullptr, 0);
            }
        }
    } else {
        // ---------------------------------------------------------------- the working warps
        pdl_wait();
        {
            constexpr int VEC_PER_ROW = D / 8;
            for (int i = threadIdx.x; i < 8 * VEC_PER_ROW; i += DW * 32) {
                const int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (r < heads) v = load16(p.q + ((size_t)geo.token0 * p.num_heads + geo.kvh * p.group + r) * D + c);
                *reinterpret_cast<uint4*>(q_s + r * Q_STRIDE + c) = v;
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");          // the queries are in shared memory (the four working warps only)
        bool ok = true;
        for (int i = 0; i < num_stages && ok; ++i) {
            lag_point();
            const int s = i % RING_STAGES;
            const int kt = tile_begin + 4 * i + warp;
            ok = mbar_wait(smem_u32(&full_bar[s]), (i / RING_STAGES) & 1, p.error_flag, 62);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            KeyTile tile;
            tile.base = -1;
            if (kt < tile_end) {
                const int base = kt * 16;
                const int page = pt.page_of(p.page_shift >= 0 ? base >> p.page_shift : base / p.page_size);
                if (page >= 0 && page < p.num_pages) ring_take_keys(ring + s * RING_STAGE_BYTES + warp * 2 * RING_TILE_BYTES, base, last_pos, tile);
                else if (lane == 0 && p.error_flag) atomicExch(p.error_flag, 3);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));      // the stage may be refilled while this tile is used
            consume_keys_t<true>(p, q_s, tile, last_pos, lo, st);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");          // every warp has taken its last tile: the ring may become the merge's scratch
    }
    merge_and_store_t<DW>(p, geo, st, frag, warp_m, warp_l, cta_o, cta_m, cta_l, heads, splits, rank, warp < DW);
}

}  // namespace


// ---- the tensor map of the paged cache for the ring kernel: rows = (page, K|V, kv head, slot), D columns; a box is
// one 16-key tile by 64 elements, 128-byte swizzled.  Encoded once per cache (its address and size) and kept.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int cache_tensor_map(CUtensorMap* map, const void* pages, long long rows) {
    static std::mutex mutex;
    static std::unordered_map<unsigned long long, CUtensorMap> known;
    const unsigned long long key = (unsigned long long)(uintptr_t)pages * 1000003ull ^ (unsigned long long)rows;
    {
        std::lock_guard<std::mutex> lock(mutex);
        auto found = known.find(key);
        if (found != known.end()) { *map = found->second; return MLB_OK; }
    }
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)sym;
    }
    if (!fn) return fail(MLB_CUDA_ERROR, "paged_attention_mma: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64u, 16u};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(MLB_CUDA_ERROR, "paged_attention_mma: cuTensorMapEncodeTiled failed with %d", (int)r);
    std::lock_guard<std::mutex> lock(mutex);
    if (known.size() > 4096) known.clear();
    known.emplace(key, *map);
    return MLB_OK;
}

// up to this many CTAs the decode shape runs eight warps per CTA (measured: one sequence of two kv heads gains,
// eight sequences lose)
constexpr int WIDE_LIMIT_CTAS = 48;

MLB_EXPORT int mlb_fa_head_dim() { return D; }
MLB_EXPORT int mlb_fa_max_splits() { return MAX_SPLITS; }

// mode 0: prefill shape (work items name the first of 4 row tiles of a sequence).
// mode 1: decode shape: every sequence brings one token (num_work = sequences * ceil(group / 16));
// the keys are cut `splits` ways (1, 2, 4, 8 or 16; D / splits must be whole) over a thread-block cluster.
// mode 2: the decode shape for SOME sequences of a step that also holds prompt portions: `work` lists the
// sequences that bring exactly one token (num_work = listed sequences * ceil(group / 16)).
// Heads of 128 with groups of at most 8 heads and clusters of at most 8: adding 4 to the mode asks for the kernel that
// brings the keys through a shared-memory ring (the caller knows the context lengths and decides when it pays),
// adding 8 forbids it; with neither, a grid of at least one CTA per multiprocessor takes it.
MLB_EXPORT int mlb_paged_attention_mma(const void* q, const void* pages, void* out, const int* seq_starts,
                                       const int* seq_pos0, const int* block_table, const int* work, int num_work,
                                       int max_blocks, int num_pages, int page_size, int num_heads, int num_kv_heads,
                                       int window, float scale, int mode, int splits, int* error_flag,
                                       cudaStream_t stream) {
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_mma: bad head counts %d/%d", num_heads, num_kv_heads);
    if (page_size <= 0 || page_size % 16 != 0)
        return fail(MLB_UNSUPPORTED_SIZE, "paged_attention_mma: page_size %d must be a multiple of 16", page_size);
    if (num_pages <= 0 || max_blocks <= 0 || window < 0 || num_work < 0)
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_mma: bad cache geometry");
    const bool force_ring = (mode & 4) != 0, forbid_ring = (mode & 8) != 0;
    mode &= 3;
    if (mode < 0 || mode > 2) return fail(MLB_INVALID_ARGUMENT, "paged_attention_mma: unknown mode %d", mode);
    if (mode == 2 && !work) return fail(MLB_INVALID_ARGUMENT, "paged_attention_mma: mode 2 needs the list of sequences");
    if (mode >= 1 && !(splits == 1 || splits == 2 || splits == 4 || splits == 8 || splits == 16))
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_mma: %d splits, expected 1, 2, 4, 8 or 16", splits);
    if (mode >= 1 && D % splits != 0)
        return fail(MLB_UNSUPPORTED_SIZE, "paged_attention_mma: %d splits do not divide the head size %d", splits, D);
    if (num_work == 0) return MLB_OK;
    FaParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, (__nv_bfloat16*)out, seq_starts, seq_pos0,
               block_table, work, max_blocks, num_pages, page_size, num_heads, num_kv_heads,
               num_heads / num_kv_heads, window, scale * LOG2E, (page_size & (page_size - 1)) == 0 ? __builtin_ctz((unsigned)page_size) : -1, error_flag,
               mode == 2 ? 1 : 0};
    if (mode == 0) {
        static bool prefill_configured_on[MAX_DEVICES] = {false};
        bool& prefill_configured = prefill_configured_on[device_index()];
        if (!prefill_configured) {
            cudaError_t e = cudaFuncSetAttribute(fa_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREFILL_SMEM);
            if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "fa_prefill: cannot reserve %d bytes of shared memory: %s",
                                              (int)PREFILL_SMEM, cudaGetErrorString(e));
            prefill_configured = true;
        }
        launch_kernel(fa_prefill_kernel, dim3(num_work, num_kv_heads, 1), WARPS * 32, PREFILL_SMEM, stream, p);
        return check_launch("fa_prefill");
    }
    // a handful of CTAs (one or two sequences): eight warps each; otherwise four warps, two CTAs per SM
    const bool wide = (long long)num_work * num_kv_heads * splits <= WIDE_LIMIT_CTAS;
    // groups of at most 8 heads: the kernel with keys on the 16-row side of the MMA (half the work per key)
    const bool keys_on_m = p.group <= 8 && D % 64 == 0 && USE_PREFETCH;   // two key tiles in registers
    static bool configured_on[MAX_DEVICES] = {false};
    bool& configured = configured_on[device_index()];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(fa_decode_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(4));
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(fa_decode_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem(8));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_decode_kernel<4>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_decode_kernel<8>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_decode_t_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_t_smem(4));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_decode_t_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_t_smem(8));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_decode_t_kernel<4>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(fa_decode_t_kernel<8>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "fa_decode: cannot reserve %d bytes of shared memory: %s",
                                          (int)decode_smem(8), cudaGetErrorString(e));
        configured = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(num_work, num_kv_heads, splits);
    config.blockDim = dim3((wide ? 8 : 4) * 32);
    config.dynamicSmemBytes = keys_on_m ? (wide ? decode_t_smem(8) : decode_t_smem(4)) : (wide ? decode_smem(8) : decode_smem(4));
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 1;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = splits;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    if (splits > 8) {
        // the non-portable cluster size: ask once whether such a cluster can be resident at all
        static int clusters16_on[MAX_DEVICES];
        static bool clusters16_asked[MAX_DEVICES] = {false};
        const int dev = device_index();
        if (!clusters16_asked[dev]) { clusters16_on[dev] = -1; clusters16_asked[dev] = true; }
        int& clusters16 = clusters16_on[dev];
        if (clusters16 < 0) {
            cudaLaunchConfig_t probe = config;
            probe.numAttrs = 1;
            int n = 0;
            cudaError_t e = wide ? cudaOccupancyMaxActiveClusters(&n, fa_decode_kernel<8>, &probe)
                                 : cudaOccupancyMaxActiveClusters(&n, fa_decode_kernel<4>, &probe);      // the larger of the two kernels
            clusters16 = (e == cudaSuccess) ? n : 0;
            cudaGetLastError();
        }
        if (clusters16 < 1) return fail(MLB_UNSUPPORTED_SIZE, "fa_decode: clusters of %d CTAs cannot be resident on this device", splits);
    }
    const long long grid_ctas = (long long)num_work * num_kv_heads * splits;
    if (keys_on_m && D == 128 && !forbid_ring && splits <= 8 && (force_ring || (!wide && grid_ctas >= sm_count()))) {
        const long long rows = (long long)num_pages * 2 * num_kv_heads * page_size;
        if (rows >= (1ll << 31)) return fail(MLB_UNSUPPORTED_SIZE, "paged_attention_mma: the cache has too many rows (%lld)", rows);
        if (((uintptr_t)pages & 15) != 0) return fail(MLB_UNSUPPORTED_SIZE, "paged_attention_mma: the cache must be 16-byte aligned");
        CUtensorMap map_kv;
        int status = cache_tensor_map(&map_kv, pages, rows);
        if (status != MLB_OK) return status;
        static bool ring_configured_on[MAX_DEVICES] = {false};
        bool& ring_configured = ring_configured_on[device_index()];
        if (!ring_configured) {
            cudaError_t e = cudaFuncSetAttribute(fa_decode_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_ring_smem());
            if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "fa_decode_ring: cannot reserve %d bytes of shared memory: %s",
                                              (int)decode_ring_smem(), cudaGetErrorString(e));
            ring_configured = true;
        }
        config.blockDim = dim3(160);
        config.dynamicSmemBytes = decode_ring_smem();
        cudaLaunchKernelEx(&config, fa_decode_ring_kernel, map_kv, p);
        return check_launch("fa_decode_ring");
    }
    if (keys_on_m) {
        if (wide) cudaLaunchKernelEx(&config, fa_decode_t_kernel<8>, p);
        else cudaLaunchKernelEx(&config, fa_decode_t_kernel<4>, p);
        return check_launch("fa_decode_t");
    }
    if (wide) cudaLaunchKernelEx(&config, fa_decode_kernel<8>, p);
    else cudaLaunchKernelEx(&config, fa_decode_kernel<4>, p);
    return check_launch("fa_decode");
}
