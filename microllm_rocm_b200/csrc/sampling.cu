// Token selection on the device: greedy argmax and seeded temperature / top-k sampling,
// one thread block per logits row, so only one int per row ever travels to the host.
//
// Greedy follows the reference exactly (src/inference/generator.cpp:46-49 and the device
// argmax, src/ops/hip/basic_kernels.hip:654-706): first maximum, i.e. smallest index on
// ties, and -1 when any logit is not finite.
//
// Sampling keeps the reference's quantities (generator.cpp:50-68): candidates are the top_k
// largest logits (all when top_k == 0), weight_i = exp(double(l_i / T - l_max / T)) with the
// division and subtraction in fp32.  The reference then draws with
// std::discrete_distribution over a std::mt19937_64, whose mapping is implementation
// defined; here the draw is spelled out so that host and device agree:
//   u      = splitmix64(seed + GOLDEN * (draw + 1)) >> 11, times 2^-53      in [0, 1)
//   choose the first candidate, in index order, whose running weight sum exceeds u * total.
// Ties at the top-k threshold go to the smaller index.
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

constexpr int THREADS = 1024;

__device__ __forceinline__ unsigned sortable_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);       // larger float <-> larger key
}

__device__ __forceinline__ double uniform_from(unsigned long long seed, unsigned long long draw) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (draw + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}

// (value, index) maximum with the smallest index on ties; all threads get the result
__device__ void block_argmax(float& value, int& index, float* s_val, int* s_idx) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, value, o);
        const int oi = __shfl_xor_sync(0xffffffffu, index, o);
        if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
    }
    __syncthreads();
    if (lane == 0) { s_val[warp] = value; s_idx[warp] = index; }
    __syncthreads();
    const int warps = blockDim.x >> 5;
    value = lane < warps ? s_val[lane] : -INFINITY;
    index = lane < warps ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, value, o);
        const int oi = __shfl_xor_sync(0xffffffffu, index, o);
        if (ov > value || (ov == value && oi < index)) { value = ov; index = oi; }
    }
}

// exclusive prefix over one value per thread (block of THREADS); returns the prefix, and the
// block total through `total`
template <typename T>
__device__ T block_exclusive_scan(T v, T* s_warp, T& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const T n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) s_warp[warp] = inc;
    __syncthreads();
    T warp_prefix = 0, all = 0;
    const int warps = blockDim.x >> 5;
    for (int w = 0; w < warps; ++w) {           // 32 values: a serial walk keeps the order fixed
        const T s = s_warp[w];
        if (w < warp) warp_prefix += s;
        all += s;
    }
    total = all;
    return warp_prefix + inc - v;
}

struct SampleParams {
    const float* logits;     // [rows, ld]
    long long ld;
    int vocab;
    const float* temperature;            // [rows]   0 -> greedy
    const int* top_k;                    // [rows]   0 -> whole vocabulary
    const unsigned long long* seed;      // [rows]
    const unsigned long long* draw;      // [rows]   how many tokens this request has drawn so far
    int* out;                            // [rows]
    int skip_greedy;                     // 1: greedy rows were already selected by argmax_split_kernel
};

__global__ void __launch_bounds__(THREADS) sample_rows_kernel(SampleParams p) {
    pdl_prologue();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ double s_dbl[32];
    __shared__ int s_int[32];
    __shared__ unsigned s_hist[256];
    __shared__ int s_flag, s_pick;
    __shared__ unsigned s_prefix;
    __shared__ int s_remaining;

    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = p.logits + (size_t)row * p.ld;
    const int V = p.vocab;
    if (p.skip_greedy && ((p.temperature ? p.temperature[row] : 0.0f) == 0.0f || (p.top_k ? p.top_k[row] : 0) == 1)) return;

    // pass 1: maximum, its first index, finiteness
    if (tid == 0) { s_flag = 0; s_pick = 0x7fffffff; }
    __syncthreads();
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    bool bad = false;
    for (int i = tid; i < V; i += THREADS) {
        const float v = x[i];
        if (!isfinite(v)) bad = true;
        if (v > best) { best = v; best_i = i; }       // strided walk visits indices in increasing order
    }
    if (bad) atomicExch(&s_flag, 1);
    block_argmax(best, best_i, s_val, s_idx);
    __syncthreads();
    if (s_flag) { if (tid == 0) p.out[row] = -1; return; }

    const float T = p.temperature ? p.temperature[row] : 0.0f;
    int k = p.top_k ? p.top_k[row] : 0;
    if (T == 0.0f || k == 1) { if (tid == 0) p.out[row] = best_i; return; }
    if (k <= 0 || k > V) k = V;

    // threshold key of the k-th largest logit and how many equal to it are kept
    unsigned thr_key = 0u;
    int keep_equal = 0x7fffffff;
    if (k < V) {
        if (tid == 0) { s_prefix = 0u; s_remaining = k; }
        __syncthreads();
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) s_hist[tid] = 0u;
            __syncthreads();
            const unsigned prefix = s_prefix;
            const unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
            for (int i = tid; i < V; i += THREADS) {
                const unsigned key = sortable_key(x[i]);
                if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                int remaining = s_remaining;
                int digit = 255;
                for (; digit > 0; --digit) {
                    const int c = (int)s_hist[digit];
                    if (c >= remaining) break;
                    remaining -= c;
                }
                s_prefix = prefix | ((unsigned)digit << shift);
                s_remaining = remaining;
            }
            __syncthreads();
        }
        thr_key = s_prefix;
        keep_equal = s_remaining;          // of the logits equal to the threshold, keep this many
    }

    // each thread owns a contiguous span of indices, so prefix sums follow index order
    const int span = (V + THREADS - 1) / THREADS;
    const int begin = min(tid * span, V), end = min(begin + span, V);
    int equal_before = 0;
    if (k < V) {
        int mine = 0;
        for (int i = begin; i < end; ++i) mine += sortable_key(x[i]) == thr_key ? 1 : 0;
        int total_equal;
        equal_before = block_exclusive_scan<int>(mine, s_int, total_equal);
    }
    const float max_scaled = best / T;
    double partial = 0.0;
    {
        int eq = equal_before;
        for (int i = begin; i < end; ++i) {
            const unsigned key = sortable_key(x[i]);
            bool cand = true;
            if (k < V) {
                if (key < thr_key) cand = false;
                else if (key == thr_key) { cand = eq < keep_equal; ++eq; }
            }
            if (cand) partial += exp((double)(x[i] / T - max_scaled));
        }
    }
    double total;
    const double before = block_exclusive_scan<double>(partial, s_dbl, total);
    const double target = uniform_from(p.seed[row], p.draw[row]) * total;
    if (partial > 0.0 && before + partial > target) atomicMin(&s_pick, tid);
    __syncthreads();
    int owner = s_pick;
    if (owner == 0x7fffffff) {                     // rounding left the target at the very end
        if (partial > 0.0) atomicMax(&s_flag, tid + 1);
        __syncthreads();
        owner = s_flag - 1;
    }
    if (tid == owner) {
        double running = before;
        int chosen = -1, last = -1;
        int eq = equal_before;
        for (int i = begin; i < end; ++i) {
            const unsigned key = sortable_key(x[i]);
            bool cand = true;
            if (k < V) {
                if (key < thr_key) cand = false;
                else if (key == thr_key) { cand = eq < keep_equal; ++eq; }
            }
            if (!cand) continue;
            last = i;
            running += exp((double)(x[i] / T - max_scaled));
            if (running > target) { chosen = i; break; }
        }
        p.out[row] = chosen >= 0 ? chosen : last;
    }
}

__global__ void __launch_bounds__(THREADS) argmax_rows_kernel(const float* __restrict__ logits, long long ld,
                                                              int vocab, int* __restrict__ out) {
    pdl_prologue();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ int s_flag;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * ld;
    if (tid == 0) s_flag = 0;
    __syncthreads();
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    bool bad = false;
    for (int i = tid; i < vocab; i += THREADS) {
        const float v = x[i];
        if (!isfinite(v)) bad = true;
        if (v > best) { best = v; best_i = i; }
    }
    if (bad) atomicExch(&s_flag, 1);
    block_argmax(best, best_i, s_val, s_idx);
    __syncthreads();
    if (tid == 0) out[row] = s_flag ? -1 : best_i;
}

// ------------------------------------------------------------------------------ greedy selection over a large vocabulary
// One block per row reads 600 KB of logits alone; here a row is cut into `parts` slices, one block each.  Every
// block leaves (maximum, first index, finiteness) of its slice; the block that arrives last at the row's ticket
// merges them (largest value, smallest index on ties: the result does not depend on which block is last) and
// resets the ticket.  The scratch is a file-scope device array: launches on different streams would share it.
constexpr int SPLIT_THREADS = 256;
constexpr int SPLIT_MAX_ROWS = 4096;
constexpr int SPLIT_MAX_PARTS = 32;
constexpr int SPLIT_MIN_VOCAB = 16384;
constexpr int SPLIT_SLICE = 8192;

__device__ float g_part_val[SPLIT_MAX_ROWS * SPLIT_MAX_PARTS];
__device__ int g_part_idx[SPLIT_MAX_ROWS * SPLIT_MAX_PARTS];
__device__ int g_part_bad[SPLIT_MAX_ROWS * SPLIT_MAX_PARTS];
__device__ int g_tickets[SPLIT_MAX_ROWS];

__global__ void __launch_bounds__(SPLIT_THREADS) argmax_split_kernel(const float* __restrict__ logits, long long ld, int vocab,
                                                                     int parts, const float* __restrict__ temperature,
                                                                     const int* __restrict__ top_k, int* __restrict__ out) {
    pdl_prologue();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ int s_flag, s_last;
    const int row = blockIdx.x, part = blockIdx.y, tid = threadIdx.x;
    // with per-row settings, only greedy rows are selected here (the sampling kernel takes the others)
    if (temperature && temperature[row] != 0.0f && !(top_k && top_k[row] == 1)) return;
    const int per = (vocab + parts - 1) / parts;
    const int begin = part * per, end = min(vocab, begin + per);
    const float* x = logits + (size_t)row * ld;
    if (tid == 0) s_flag = 0;
    __syncthreads();
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    bool bad = false;
    for (int i = begin + tid; i < end; i += SPLIT_THREADS) {
        const float v = x[i];
        if (!isfinite(v)) bad = true;
        if (v > best) { best = v; best_i = i; }        // strided walk visits indices in increasing order
    }
    if (bad) atomicExch(&s_flag, 1);
    block_argmax(best, best_i, s_val, s_idx);
    __syncthreads();
    if (tid == 0) {
        const int slot = row * SPLIT_MAX_PARTS + part;
        g_part_val[slot] = best; g_part_idx[slot] = best_i; g_part_bad[slot] = s_flag;
        __threadfence();
        s_last = atomicAdd(&g_tickets[row], 1) == parts - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!s_last || tid >= 32) return;
    __threadfence();
    float v = -INFINITY;
    int idx = 0x7fffffff, any_bad = 0;
    if (tid < parts) {
        const int slot = row * SPLIT_MAX_PARTS + tid;
        v = __ldcg(&g_part_val[slot]); idx = __ldcg(&g_part_idx[slot]); any_bad = __ldcg(&g_part_bad[slot]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        any_bad |= __shfl_xor_sync(0xffffffffu, any_bad, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (tid == 0) {
        out[row] = any_bad ? -1 : idx;
        g_tickets[row] = 0;
    }
}

int split_parts(int rows, int vocab) {
    if (vocab < SPLIT_MIN_VOCAB || rows > SPLIT_MAX_ROWS) return 0;
    int parts = vocab / SPLIT_SLICE;
    if (parts > SPLIT_MAX_PARTS) parts = SPLIT_MAX_PARTS;
    return parts < 2 ? 0 : parts;
}

}  // namespace

MLB_EXPORT int mlb_argmax_rows(const float* logits, long long ld, int rows, int vocab, int* out,
                               cudaStream_t stream) {
    if (rows < 0 || vocab <= 0 || ld < vocab) return fail(MLB_INVALID_ARGUMENT, "argmax_rows: bad sizes");
    if (rows == 0) return MLB_OK;
    const int parts = split_parts(rows, vocab);
    if (parts) {
        launch_kernel(argmax_split_kernel, dim3(rows, parts), SPLIT_THREADS, 0, stream, logits, ld, vocab, parts,
                      (const float*)nullptr, (const int*)nullptr, out);
        return check_launch("argmax_split");
    }
    launch_kernel(argmax_rows_kernel, rows, THREADS, 0, stream, logits, ld, vocab, out);
    return check_launch("argmax_rows");
}

MLB_EXPORT int mlb_sample_rows(const float* logits, long long ld, int rows, int vocab, const float* temperature,
                               const int* top_k, const unsigned long long* seed, const unsigned long long* draw,
                               int* out, cudaStream_t stream) {
    if (rows < 0 || vocab <= 0 || ld < vocab) return fail(MLB_INVALID_ARGUMENT, "sample_rows: bad sizes");
    if (!seed || !draw) return fail(MLB_INVALID_ARGUMENT, "sample_rows: seed and draw arrays are required");
    if (rows == 0) return MLB_OK;
    SampleParams p{logits, ld, vocab, temperature, top_k, seed, draw, out, 0};
    const int parts = split_parts(rows, vocab);
    if (parts && temperature) {
        // greedy rows by many blocks per row; the rows that sample by the one-block-per-row kernel, which then skips the others
        launch_kernel(argmax_split_kernel, dim3(rows, parts), SPLIT_THREADS, 0, stream, logits, ld, vocab, parts, temperature, top_k, out);
        int status = check_launch("argmax_split");
        if (status != MLB_OK) return status;
        p.skip_greedy = 1;
    }
    launch_kernel(sample_rows_kernel, rows, THREADS, 0, stream, p);
    return check_launch("sample_rows");
}
