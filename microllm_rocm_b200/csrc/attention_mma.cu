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
// Two launch shapes of the same warp routine:
//   prefill  one CTA = 4 warps = 4 consecutive row tiles; no key split
//   decode   one CTA = one row tile, its 4 warps take every 4th key tile and are merged in
//            shared memory; the keys are further split over gridDim.z CTAs that leave partial
//            results (normalised output + log-sum-exp) in scratch memory, and the CTA that
//            finishes last merges them, always in split order.
//
// Operand layout trick: mma.sync only needs A and B to agree on which contraction index a
// register holds.  Thread t of a quad therefore loads 8 CONSECUTIVE head elements of a key
// (one 16-byte load) and uses them as the fragments of two k-steps; Q is read from shared
// memory with the same permutation.  For V the output columns are permuted instead.
#include "common.cuh"

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
    float* part_o;                  // [T*NH, splits, D]   scratch, decode with splits > 1
    float* part_lse;                // [T*NH, splits]
    int* tickets;                   // [num_work * NKV] zero between launches: which split finished last
    const int* seq_starts;          // [A+1] first flat token of each sequence
    const int* seq_pos0;            // [A]   tokens cached before this step
    const int* block_table;         // [A, max_blocks]
    const int* work;                // [num_work, 2] (sequence, first row tile)
    int max_blocks, num_pages, page_size;
    int num_heads, num_kv_heads, group;
    int window;
    float scale_log2;               // softmax scale * log2(e)
    int splits;
    int* error_flag;
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

__device__ __forceinline__ uint4 load16(const __nv_bfloat16* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
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
    const int page = pt.page_of(base / p.page_size);
    if (page < 0 || page >= p.num_pages) {
        if (lane == 0 && p.error_flag) atomicExch(p.error_flag, 3);
        kv.base = -1;
        return;
    }
    kv.base = base;
    const size_t page_stride = (size_t)2 * p.num_kv_heads * p.page_size * D;
    const __nv_bfloat16* kbase = p.pages + (size_t)page * page_stride +
                                 ((size_t)geo.kvh * p.page_size + (base % p.page_size)) * D;
    const __nv_bfloat16* vbase = kbase + (size_t)p.num_kv_heads * p.page_size * D;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int c = 0; c < KCHUNKS; ++c) kv.k[nb][c] = load16(kbase + (size_t)(nb * 8 + g) * D + c * 32 + t * 8);
#pragma unroll
    for (int vb = 0; vb < VBLOCKS; ++vb) {
        const int col = vb * 64 + g * 8;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int key = 2 * t + (r & 1) + 8 * (r >> 1);       // this thread's keys: 2t, 2t+1, 2t+8, 2t+9
            kv.v[vb][r] = (col < D && base + key <= hi_tile) ? load16(vbase + (size_t)key * D + col) : make_uint4(0, 0, 0, 0);
        }
    }
}

// One 16-key tile through scores, running softmax and the value product.
__device__ __forceinline__ void consume_keys(const FaParams& p, const __nv_bfloat16* q_s, const KeyTile& kv,
                                             const int (&pos_row)[2], const int (&lo_row)[2], RowState& st) {
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
    float mx[2] = {-INFINITY, -INFINITY};
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
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float m_new = fmaxf(st.m[i], mx[i]);
        corr[i] = (m_new == -INFINITY) ? 1.0f : exp2f(st.m[i] - m_new);
        st.m[i] = m_new;
    }
    float rowsum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = e >> 1;
            const float pv = (s[nb][e] == -INFINITY) ? 0.0f : exp2f(s[nb][e] - st.m[i]);
            s[nb][e] = pv;
            rowsum[i] += pv;
        }
#pragma unroll
    for (int i = 0; i < 2; ++i) st.l[i] = st.l[i] * corr[i] + rowsum[i];
#pragma unroll
    for (int nbo = 0; nbo < NB_O; ++nbo) {
        st.o[nbo][0] *= corr[0]; st.o[nbo][1] *= corr[0];
        st.o[nbo][2] *= corr[1]; st.o[nbo][3] *= corr[1];
    }
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
// tile_begin + first.  q_s: this tile's queries, [16][Q_STRIDE] bf16 in shared memory.  With
// PREFETCH the loads of the next key tile are in flight while the current one is consumed.
template <bool PREFETCH>
__device__ __forceinline__ void attend(const FaParams& p, const TileGeometry& geo, const PageTable& pt,
                                       const __nv_bfloat16* q_s, int tile_begin, int tile_end, int first, int stride,
                                       int hi_tile, RowState& st) {
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
    int kt = tile_begin + first;
    if (kt >= tile_end) return;
    if (PREFETCH) {
        KeyTile a, b;
        load_keys(p, geo, pt, kt, hi_tile, a);
        while (true) {
            const bool more_b = kt + stride < tile_end;
            if (more_b) load_keys(p, geo, pt, kt + stride, hi_tile, b);
            consume_keys(p, q_s, a, pos_row, lo_row, st);
            if (!more_b) break;
            kt += stride;
            const bool more_a = kt + stride < tile_end;
            if (more_a) load_keys(p, geo, pt, kt + stride, hi_tile, a);
            consume_keys(p, q_s, b, pos_row, lo_row, st);
            if (!more_a) break;
            kt += stride;
        }
    } else {
        KeyTile a;
        for (; kt < tile_end; kt += stride) {
            load_keys(p, geo, pt, kt, hi_tile, a);
            consume_keys(p, q_s, a, pos_row, lo_row, st);
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

__device__ __forceinline__ void load_q_tile(const FaParams& p, const TileGeometry& geo, __nv_bfloat16* q_s, int lane,
                                            int lanes) {
    constexpr int VEC_PER_ROW = D / 8;        // 16 rows x D elements, 16 bytes per load
    for (int i = lane; i < 16 * VEC_PER_ROW; i += lanes) {
        const int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
        const int tok = geo.token_of(r, p.group);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < geo.n_new) {
            const int head = geo.kvh * p.group + (geo.row0 + r) % p.group;
            v = load16(p.q + ((size_t)(geo.token0 + tok) * p.num_heads + head) * D + c);
        }
        *reinterpret_cast<uint4*>(q_s + r * Q_STRIDE + c) = v;
    }
}

__device__ __forceinline__ bool geometry(const FaParams& p, int work_index, int tile_offset, int kvh, TileGeometry& geo) {
    geo.seq = p.work[2 * work_index];
    const int tile = p.work[2 * work_index + 1] + tile_offset;
    geo.kvh = kvh;
    geo.token0 = p.seq_starts[geo.seq];
    geo.n_new = p.seq_starts[geo.seq + 1] - geo.token0;
    geo.pos0 = p.seq_pos0[geo.seq];
    geo.row0 = tile * 16;
    return geo.row0 < geo.n_new * p.group;
}

// ---------------------------------------------------------------------------------- prefill
__global__ void __launch_bounds__(WARPS * 32) fa_prefill_kernel(FaParams p) {
    pdl_prologue();
    __shared__ __align__(16) __nv_bfloat16 q_s[WARPS][16 * Q_STRIDE];
    __shared__ int table_s[WARPS][TABLE_SPAN / WARPS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    TileGeometry geo;
    if (!geometry(p, blockIdx.x, warp, blockIdx.y, geo)) return;
    const int first_tok = geo.token_of(0, p.group);
    const int last_tok = min(geo.token_of(15, p.group), geo.n_new - 1);
    const int first_pos = geo.pos0 + first_tok, last_pos = geo.pos0 + last_tok;
    const int lo = (p.window > 0 && first_pos - p.window + 1 > 0) ? first_pos - p.window + 1 : 0;
    // each warp keeps the LAST blocks of its key range at hand (it reaches them however long
    // the range is); earlier blocks of a very long range are looked up in global memory
    PageTable pt;
    {
        const int last_block = last_pos / p.page_size;
        const int first_block = max(lo / p.page_size, last_block - TABLE_SPAN / WARPS + 1);
        fill_page_table(pt, table_s[warp], p.block_table + (size_t)geo.seq * p.max_blocks, p.max_blocks, first_block,
                        last_block, lane, 32);
        pt.count = min(pt.count, TABLE_SPAN / WARPS);
    }
    load_q_tile(p, geo, q_s[warp], lane, 32);
    __syncwarp();
    RowState st;
    init_state(st);
    attend<USE_PREFETCH>(p, geo, pt, q_s[warp], lo / 16, last_pos / 16 + 1, 0, 1, last_pos, st);
    // normalise and write through shared memory so that rows leave as whole 16-byte pieces
    float inv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float l = st.l[i];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        inv[i] = l > 0.0f ? 1.0f / l : 0.0f;
    }
    __syncwarp();
    __nv_bfloat16* o_s = q_s[warp];
#pragma unroll
    for (int nbo = 0; nbo < NB_O; ++nbo)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int dim = out_dim(nbo, e, t);
            if (dim < D) o_s[(g + 8 * (e >> 1)) * Q_STRIDE + dim] = __float2bfloat16_rn(st.o[nbo][e] * inv[e >> 1]);
        }
    __syncwarp();
    constexpr int VEC_PER_ROW = D / 8;
    for (int i = lane; i < 16 * VEC_PER_ROW; i += 32) {
        const int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
        const int tok = geo.token_of(r, p.group);
        if (tok >= geo.n_new) continue;
        const int head = geo.kvh * p.group + (geo.row0 + r) % p.group;
        *reinterpret_cast<uint4*>(p.out + ((size_t)(geo.token0 + tok) * p.num_heads + head) * D + c) =
            *reinterpret_cast<const uint4*>(o_s + r * Q_STRIDE + c);
    }
}

// ---------------------------------------------------------------------------------- decode
// Shared memory of the decode kernel (dynamic): the query tile, then per warp its output
// fragments in thread order (conflict free), its row maxima and sums, and the weights of the
// final merge.
constexpr int FRAGS = NB_O * 4;
constexpr int MAX_SPLITS = 64;
constexpr size_t DECODE_SMEM = 16 * Q_STRIDE * sizeof(__nv_bfloat16) + (size_t)WARPS * FRAGS * 32 * sizeof(float) +
                               2 * WARPS * 16 * sizeof(float) + 16 * MAX_SPLITS * sizeof(float) + 16 +
                               TABLE_SPAN * sizeof(int);

template <bool PREFETCH>
__global__ void __launch_bounds__(WARPS * 32, PREFETCH ? 2 : 3) fa_decode_kernel(FaParams p) {
    pdl_prologue();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    float* frag = reinterpret_cast<float*>(smem_raw + 16 * Q_STRIDE * sizeof(__nv_bfloat16));   // [WARPS][FRAGS][32]
    float* warp_m = frag + WARPS * FRAGS * 32;        // [WARPS][16]
    float* warp_l = warp_m + WARPS * 16;              // [WARPS][16]
    float* split_w = warp_l + WARPS * 16;             // [16][MAX_SPLITS] normalised weights of the final merge
    int* ticket_s = reinterpret_cast<int*>(split_w + 16 * MAX_SPLITS);
    int* table_s = ticket_s + 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    TileGeometry geo;
    if (!geometry(p, blockIdx.x, 0, blockIdx.y, geo)) return;          // uniform over the CTA
    const int rows_valid = min(16, geo.n_new * p.group - geo.row0);
    const bool upper = rows_valid > 8;                                // rows 8..15 hold anything at all
    // queries: only rows that exist are read, the rest of the tile is zero
    {
        constexpr int VEC_PER_ROW = D / 8;
        for (int i = threadIdx.x; i < 16 * VEC_PER_ROW; i += WARPS * 32) {
            const int r = i / VEC_PER_ROW, c = (i % VEC_PER_ROW) * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < rows_valid) {
                const int tok = geo.token_of(r, p.group);
                const int head = geo.kvh * p.group + (geo.row0 + r) % p.group;
                v = load16(p.q + ((size_t)(geo.token0 + tok) * p.num_heads + head) * D + c);
            }
            *reinterpret_cast<uint4*>(q_s + r * Q_STRIDE + c) = v;
        }
    }
    const int first_tok = geo.token_of(0, p.group);
    const int last_tok = min(geo.token_of(15, p.group), geo.n_new - 1);
    const int first_pos = geo.pos0 + first_tok, last_pos = geo.pos0 + last_tok;
    const int lo = (p.window > 0 && first_pos - p.window + 1 > 0) ? first_pos - p.window + 1 : 0;
    int tile_begin = lo / 16, tile_end = last_pos / 16 + 1;
    if (p.splits > 1) {                       // this CTA's even share of the sequence's key tiles
        const int per_split = (tile_end - tile_begin + p.splits - 1) / p.splits;
        tile_begin += (int)blockIdx.z * per_split;
        tile_end = min(tile_end, tile_begin + per_split);
    }
    PageTable pt;
    fill_page_table(pt, table_s, p.block_table + (size_t)geo.seq * p.max_blocks, p.max_blocks,
                    tile_begin * 16 / p.page_size, max(tile_begin, tile_end - 1) * 16 / p.page_size, threadIdx.x, WARPS * 32);
    // where this thread's two rows (g and g+8) go
    size_t out_row[2];
    bool row_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        row_ok[i] = r < rows_valid;
        const int tok = row_ok[i] ? geo.token_of(r, p.group) : 0;
        const int head = geo.kvh * p.group + (geo.row0 + r) % p.group;
        out_row[i] = (size_t)(geo.token0 + tok) * p.num_heads + head;
    }
    __syncthreads();
    RowState st;
    init_state(st);
    attend<PREFETCH>(p, geo, pt, q_s, tile_begin, tile_end, warp, WARPS, last_pos, st);
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
    float m_all[2], inv_l[2], scale_w[2][WARPS];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        m_all[i] = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) m_all[i] = fmaxf(m_all[i], warp_m[w * 16 + r]);
        float l_all = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = warp_m[w * 16 + r];
            scale_w[i][w] = (mw == -INFINITY) ? 0.0f : exp2f(mw - m_all[i]);
            l_all += warp_l[w * 16 + r] * scale_w[i][w];
        }
        inv_l[i] = l_all > 0.0f ? 1.0f / l_all : 0.0f;
        if (p.splits > 1 && warp == 0 && t == 0 && row_ok[i])
            p.part_lse[out_row[i] * p.splits + blockIdx.z] = l_all > 0.0f ? m_all[i] + log2f(l_all) : -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) scale_w[i][w] *= inv_l[i];
    }
#pragma unroll
    for (int k = 0; k < FRAGS / WARPS; ++k) {
        const int idx = warp + k * WARPS;              // this thread merges fragment idx of all warps
        const int nbo = idx >> 2, e = idx & 3, i = e >> 1;
        const int dim = out_dim(nbo, e, t);
        if (dim >= D || !row_ok[i]) continue;
        float val = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) val += frag[(w * FRAGS + idx) * 32 + lane] * scale_w[i][w];
        if (p.splits > 1) p.part_o[(out_row[i] * p.splits + blockIdx.z) * D + dim] = val;
        else p.out[out_row[i] * D + dim] = __float2bfloat16_rn(val);
    }
    if (p.splits == 1) return;
    // the CTA that finishes last for this (row tile, kv head) merges the splits: no second launch
    const int work_slot = blockIdx.x * p.num_kv_heads + blockIdx.y;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *ticket_s = atomicAdd(p.tickets + work_slot, 1);
    __syncthreads();
    if (*ticket_s != p.splits - 1) return;
    __threadfence();
    if (threadIdx.x == 0) p.tickets[work_slot] = 0;        // ready for the next launch
    // weights 2^(lse_s - max) / sum of every row at once: one warp per row, one lane per split
    for (int r = warp; r < rows_valid; r += WARPS) {
        const int tok = geo.token_of(r, p.group);
        const int head = geo.kvh * p.group + (geo.row0 + r) % p.group;
        const size_t row = (size_t)(geo.token0 + tok) * p.num_heads + head;
        float lse[MAX_SPLITS / 32];
        float mx = -INFINITY;
#pragma unroll
        for (int k = 0; k < MAX_SPLITS / 32; ++k) {
            const int s = lane + 32 * k;
            lse[k] = s < p.splits ? __ldcg(p.part_lse + row * p.splits + s) : -INFINITY;
            mx = fmaxf(mx, lse[k]);
        }
        mx = warp_max(mx);
        float w[MAX_SPLITS / 32], sum = 0.0f;
#pragma unroll
        for (int k = 0; k < MAX_SPLITS / 32; ++k) {
            w[k] = (lse[k] == -INFINITY) ? 0.0f : exp2f(lse[k] - mx);
            sum += w[k];
        }
        sum = warp_sum(sum);
        const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
#pragma unroll
        for (int k = 0; k < MAX_SPLITS / 32; ++k)
            if (lane + 32 * k < p.splits) split_w[r * MAX_SPLITS + lane + 32 * k] = w[k] * inv;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows_valid * D; i += WARPS * 32) {
        const int r = i / D, dim = i % D;
        const int tok = geo.token_of(r, p.group);
        const int head = geo.kvh * p.group + (geo.row0 + r) % p.group;
        const size_t row = (size_t)(geo.token0 + tok) * p.num_heads + head;
        const float* src = p.part_o + row * p.splits * D + dim;
        float acc = 0.0f;
        for (int s0 = 0; s0 < p.splits; s0 += 16) {    // sixteen loads in flight; the sum keeps split order
            float part[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) part[k] = s0 + k < p.splits ? __ldcg(src + (size_t)(s0 + k) * D) : 0.0f;
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (s0 + k < p.splits) acc += split_w[r * MAX_SPLITS + s0 + k] * part[k];
        }
        p.out[row * D + dim] = __float2bfloat16_rn(acc);
    }
}

}  // namespace

MLB_EXPORT int mlb_fa_head_dim() { return D; }
MLB_EXPORT int mlb_fa_max_splits() { return MAX_SPLITS; }

// mode 0: prefill shape (work items name the first of 4 row tiles).
// mode 1: decode shape (one row tile per work item, keys split `splits` ways).  With
// splits > 1 it needs scratch: part_o [rows, splits, D] and part_lse [rows, splits] fp32, and
// `tickets`, one int per (work item, kv head) that is ZERO before the first launch (the
// kernel leaves it zero again).
MLB_EXPORT int mlb_paged_attention_mma(const void* q, const void* pages, void* out, float* part_o, float* part_lse,
                                       int* tickets, const int* seq_starts, const int* seq_pos0,
                                       const int* block_table, const int* work, int num_work, int max_blocks,
                                       int num_pages, int page_size, int num_heads, int num_kv_heads, int window,
                                       float scale, int mode, int splits, int long_loops, int* error_flag,
                                       cudaStream_t stream) {
    if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_mma: bad head counts %d/%d", num_heads, num_kv_heads);
    if (page_size <= 0 || page_size % 16 != 0)
        return fail(MLB_UNSUPPORTED_SIZE, "paged_attention_mma: page_size %d must be a multiple of 16", page_size);
    if (num_pages <= 0 || max_blocks <= 0 || window < 0 || num_work < 0)
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_mma: bad cache geometry");
    if (mode == 1 && (splits < 1 || splits > MAX_SPLITS || (splits > 1 && (!part_o || !part_lse || !tickets))))
        return fail(MLB_INVALID_ARGUMENT, "paged_attention_mma: bad split arguments (1..%d splits, scratch required)", MAX_SPLITS);
    if (num_work == 0) return MLB_OK;
    FaParams p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)pages, (__nv_bfloat16*)out, part_o, part_lse, tickets,
               seq_starts, seq_pos0, block_table, work, max_blocks, num_pages, page_size, num_heads, num_kv_heads,
               num_heads / num_kv_heads, window, scale * LOG2E, mode == 1 ? splits : 1, error_flag};
    if (mode == 0) {
        launch_kernel(fa_prefill_kernel, dim3(num_work, num_kv_heads, 1), WARPS * 32, 0, stream, p);
        return check_launch("fa_prefill");
    }
    // long_loops: every warp walks several key tiles, so loads of the next tile are worth their
    // registers; otherwise the leaner instance fits more warps on an SM
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(fa_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(fa_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DECODE_SMEM);
        if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "fa_decode: cannot reserve %d bytes of shared memory: %s",
                                          (int)DECODE_SMEM, cudaGetErrorString(e));
        configured = true;
    }
    if (long_loops && USE_PREFETCH)
        launch_kernel(fa_decode_kernel<true>, dim3(num_work, num_kv_heads, splits), WARPS * 32, DECODE_SMEM, stream, p);
    else
        launch_kernel(fa_decode_kernel<false>, dim3(num_work, num_kv_heads, splits), WARPS * 32, DECODE_SMEM, stream, p);
    return check_launch("fa_decode");
}
