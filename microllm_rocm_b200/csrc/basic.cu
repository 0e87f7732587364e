// Row-wise and element-wise kernels of the decoder: token embedding gather, RMSNorm
// (alone, with the residual add fused in front, and on selected rows), SiLU(gate)*up.
// All arithmetic in fp32; storage types are template parameters.
//
// Formulas follow the reference's CPU loops:
//   embedding        src/ops/ops.cpp:581-618      out[t,:] = table[id[t],:], bad id -> NaN
//                    (src/ops/hip/basic_kernels.hip:339-352)
//   rms_norm         src/ops/ops.cpp:684-699      y = x * (1/sqrt(sum(x^2)/W + eps)) * w
//   add_rms_norm     src/ops/ops.cpp:702-740      s = l + r (stored), then rms_norm(s)
//   swiglu           src/ops/ops.cpp:72-76,760-785  g*sigmoid(g)*u, two-branch sigmoid
#include "common.cuh"

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

// ------------------------------------------------------------------ embedding gather
template <typename TableT>
__global__ void embed_gather_kernel(const TableT* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int tokens, int width, int vocab) {
    pdl_prologue();
    const int t = blockIdx.x;
    if (t >= tokens) return;
    const int id = ids[t];
    float* dst = out + (size_t)t * width;
    if (id < 0 || id >= vocab) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = nanf("");
        return;
    }
    const TableT* src = table + (size_t)id * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = to_f32(src[c]);
}

MLB_EXPORT int mlb_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                                int tokens, int width, int vocab, cudaStream_t stream) {
    if (tokens < 0 || width <= 0 || vocab <= 0) return fail(MLB_INVALID_ARGUMENT, "embed_gather: bad sizes");
    if (tokens == 0) return MLB_OK;
    const int threads = width >= 1024 ? 256 : 128;
    if (table_dtype == MLB_F32)
        launch_kernel(embed_gather_kernel<float>, tokens, threads, 0, stream, (const float*)table, ids, out, tokens, width, vocab);
    else if (table_dtype == MLB_BF16)
        launch_kernel(embed_gather_kernel<__nv_bfloat16>, tokens, threads, 0, stream, (const __nv_bfloat16*)table, ids, out, tokens, width, vocab);
    else
        return fail(MLB_INVALID_ARGUMENT, "embed_gather: unknown table dtype %d", table_dtype);
    return check_launch("embed_gather");
}

// ------------------------------------------------------------------ RMSNorm family
// One block per output row.  `rows` (may be null) selects input rows: out[r] = norm(x[rows[r]]).
// With ADD, `delta` is first added into `x` in place (x is the fp32 residual stream) and the
// sum is what gets normalised.  `delta` may be `n_delta` partial results laid `delta_stride`
// elements apart (a product whose K range was split over CTAs): they are added in order,
// which is the split's reduction.  The reduction order depends only on `width` and the block
// size, never on the number of rows.
constexpr int NORM_THREADS = 512;
constexpr int NORM_VECS = 4;            // float4 per thread kept in registers: widths up to 8192

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// sum of the partial deltas at one float4, eight loads in flight, added in split order
__device__ __forceinline__ float4 delta_sum4(const float* delta, int n_delta, long long stride) {
    float4 d = ld4(delta);
    for (int k0 = 1; k0 < n_delta; k0 += 8) {
        float4 part[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            part[k] = k0 + k < n_delta ? ld4(delta + (size_t)(k0 + k) * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 8; ++k) { d.x += part[k].x; d.y += part[k].y; d.z += part[k].z; d.w += part[k].w; }
    }
    return d;
}

template <typename OutT, bool ADD>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta, long long delta_stride,
               const float* __restrict__ weight, OutT* __restrict__ out, const int* __restrict__ rows, int width,
               float eps, int vectorised) {
    pdl_launch_dependents();
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    if (vectorised) {                       // width % 4 == 0, 16-byte aligned rows, width <= NORM_VECS * 4 * threads
        // the norm's weight is never written by a kernel: it is fetched before the wait for the predecessor
        float4 w[NORM_VECS];
#pragma unroll
        for (int i = 0; i < NORM_VECS; ++i) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c < width) w[i] = ld4(weight + c);
        }
        pdl_wait();
        const size_t src_row = rows ? (size_t)rows[r] : (size_t)r;
        float* xr = x + src_row * width;
        OutT* yr = out + (size_t)r * width;
        float ss = 0.0f;
        const int nvec = width / 4;
        float4 v[NORM_VECS];
#pragma unroll
        for (int i = 0; i < NORM_VECS; ++i) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c >= width) break;
            v[i] = ld4(xr + c);
            if (ADD) {
                const float4 d = delta_sum4(delta + src_row * width + c, n_delta, delta_stride);
                v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
                *reinterpret_cast<float4*>(xr + c) = v[i];
            }
            ss += v[i].x * v[i].x; ss += v[i].y * v[i].y; ss += v[i].z * v[i].z; ss += v[i].w * v[i].w;
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
        for (int i = 0; i < NORM_VECS; ++i) {
            const int c = (threadIdx.x + i * blockDim.x) * 4;
            if (c >= width) break;
            yr[c + 0] = from_f32<OutT>(v[i].x * inv * w[i].x);
            yr[c + 1] = from_f32<OutT>(v[i].y * inv * w[i].y);
            yr[c + 2] = from_f32<OutT>(v[i].z * inv * w[i].z);
            yr[c + 3] = from_f32<OutT>(v[i].w * inv * w[i].w);
        }
        (void)nvec;
        return;
    }
    pdl_wait();
    const size_t src_row = rows ? (size_t)rows[r] : (size_t)r;
    float* xr = x + src_row * width;
    OutT* yr = out + (size_t)r * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = xr[c];
        if (ADD) {
            float d = delta[src_row * width + c];
            for (int k = 1; k < n_delta; ++k) d += delta[(size_t)k * delta_stride + src_row * width + c];
            v += d;
            xr[c] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        yr[c] = from_f32<OutT>(xr[c] * inv * weight[c]);
    }
}

template <bool ADD>
static int launch_rmsnorm(float* x, const float* delta, int n_delta, long long delta_stride, const float* w, void* out,
                          int out_dtype, const int* rows, int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows < 0 || width <= 0 || !(eps > 0.0f)) return fail(MLB_INVALID_ARGUMENT, "rmsnorm: bad sizes or eps");
    if (n_rows == 0) return MLB_OK;
    const bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) && (!delta || (uintptr_t)delta % 16 == 0) &&
                         (delta_stride % 4 == 0);
    const int vectorised = (width % 4 == 0 && aligned && width <= NORM_VECS * 4 * NORM_THREADS) ? 1 : 0;   // NORM_THREADS is the widest block
    int threads = NORM_THREADS;
    if (!vectorised) threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    else if (n_rows >= 256 && out_dtype == MLB_BF16) {
        // many rows (a prompt portion): the smallest block that still covers the row with NORM_VECS float4 per
        // thread, so that several rows share an SM and every thread has several loads in flight; a few rows
        // (decoding) keep the widest block, which is the shortest path through one row.  Only on the bf16
        // path: the fp32 path keeps ONE block size, so that a row's sum never depends on the batch.
        threads = 128;
        while (threads * 4 * NORM_VECS < width) threads *= 2;
    }
    if (out_dtype == MLB_F32)
        launch_kernel(rmsnorm_kernel<float, ADD>, n_rows, threads, 0, stream, x, delta, n_delta, delta_stride, w, (float*)out, rows, width, eps, vectorised);
    else if (out_dtype == MLB_BF16)
        launch_kernel(rmsnorm_kernel<__nv_bfloat16, ADD>, n_rows, threads, 0, stream, x, delta, n_delta, delta_stride, w, (__nv_bfloat16*)out, rows, width, eps, vectorised);
    else
        return fail(MLB_INVALID_ARGUMENT, "rmsnorm: unknown output dtype %d", out_dtype);
    return check_launch("rmsnorm");
}

MLB_EXPORT int mlb_rmsnorm(const float* x, const float* weight, void* out, int out_dtype, const int* rows,
                           int n_rows, int width, float eps, cudaStream_t stream) {
    return launch_rmsnorm<false>(const_cast<float*>(x), nullptr, 0, 0, weight, out, out_dtype, rows, n_rows, width, eps, stream);
}

MLB_EXPORT int mlb_add_rmsnorm(float* residual, const float* delta, int n_delta, long long delta_stride,
                               const float* weight, void* out, int out_dtype, int n_rows, int width, float eps,
                               cudaStream_t stream) {
    if (!delta || n_delta < 1) return fail(MLB_INVALID_ARGUMENT, "add_rmsnorm: delta is missing");
    return launch_rmsnorm<true>(residual, delta, n_delta, delta_stride, weight, out, out_dtype, nullptr, n_rows, width, eps, stream);
}

// ------------------------------------------------------------------ residual add
__global__ void add_inplace_kernel(float* __restrict__ x, const float* __restrict__ delta, int n_delta,
                                   long long delta_stride, size_t n) {
    pdl_prologue();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float d = delta[i];
    for (int k = 1; k < n_delta; ++k) d += delta[(size_t)k * delta_stride + i];
    x[i] += d;
}

MLB_EXPORT int mlb_add_inplace(float* x, const float* delta, int n_delta, long long delta_stride, long long n,
                               cudaStream_t stream) {
    if (n < 0 || n_delta < 1) return fail(MLB_INVALID_ARGUMENT, "add_inplace: bad sizes");
    if (n == 0) return MLB_OK;
    launch_kernel(add_inplace_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, x, delta, n_delta, delta_stride, (size_t)n);
    return check_launch("add_inplace");
}

// ------------------------------------------------------------------ SiLU(gate) * up
__device__ __forceinline__ float stable_sigmoid(float v) {
    // the reference's overflow-safe two-branch form (ops.cpp:72-76)
    if (v >= 0.0f) return 1.0f / (1.0f + expf(-v));
    const float e = expf(v);
    return e / (1.0f + e);
}

template <typename InT, typename OutT>
__global__ void silu_mul_kernel(const InT* __restrict__ gate, const InT* __restrict__ up, long long in_stride,
                                int n_partials, long long partial_stride, OutT* __restrict__ out, int rows, int width) {
    pdl_prologue();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * width) return;
    const int r = (int)(i / width), c = (int)(i % width);
    float g = to_f32(gate[r * in_stride + c]);
    float u = to_f32(up[r * in_stride + c]);
    for (int k = 1; k < n_partials; ++k) {           // partial results of a split product, added in order
        g += to_f32(gate[(size_t)k * partial_stride + r * in_stride + c]);
        u += to_f32(up[(size_t)k * partial_stride + r * in_stride + c]);
    }
    out[i] = from_f32<OutT>(g * stable_sigmoid(g) * u);
}

// bf16 in, bf16 out, eight elements per thread (16-byte loads and stores)
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                       long long in_stride, __nv_bfloat16* __restrict__ out, int rows, int width) {
    pdl_prologue();
    const int vec_per_row = width / 8;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * vec_per_row) return;
    const int r = (int)(i / vec_per_row), c = (int)(i % vec_per_row) * 8;
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + (size_t)r * in_stride + c);
    const uint4 uv = *reinterpret_cast<const uint4*>(up + (size_t)r * in_stride + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
        o2[k] = __floats2bfloat162_rn(g.x * stable_sigmoid(g.x) * u.x, g.y * stable_sigmoid(g.y) * u.y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * width + c) = ov;
}

// gate and up are two column blocks of one [rows, in_stride] matrix (the fused gate/up
// projection) or two separate matrices; `in_stride` is their row pitch in elements.  The input
// may be `n_partials` partial results `partial_stride` elements apart.
MLB_EXPORT int mlb_silu_mul(const void* gate, const void* up, long long in_stride, int in_dtype, int n_partials,
                            long long partial_stride, void* out, int out_dtype, int rows, int width,
                            cudaStream_t stream) {
    if (rows < 0 || width <= 0 || in_stride < width || n_partials < 1) return fail(MLB_INVALID_ARGUMENT, "silu_mul: bad sizes");
    if (rows == 0) return MLB_OK;
    const long long n = (long long)rows * width;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (in_dtype == MLB_F32 && out_dtype == MLB_F32)
        launch_kernel(silu_mul_kernel<float, float>, blocks, 256, 0, stream, (const float*)gate, (const float*)up, in_stride, n_partials, partial_stride, (float*)out, rows, width);
    else if (in_dtype == MLB_BF16 && out_dtype == MLB_BF16 && n_partials == 1 && width % 8 == 0 && in_stride % 8 == 0 &&
             (uintptr_t)gate % 16 == 0 && (uintptr_t)up % 16 == 0 && (uintptr_t)out % 16 == 0)
        launch_kernel(silu_mul_bf16x8_kernel, (unsigned)((n / 8 + 255) / 256), 256, 0, stream, (const __nv_bfloat16*)gate,
                      (const __nv_bfloat16*)up, in_stride, (__nv_bfloat16*)out, rows, width);
    else if (in_dtype == MLB_BF16 && out_dtype == MLB_BF16)
        launch_kernel(silu_mul_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, in_stride, n_partials, partial_stride, (__nv_bfloat16*)out, rows, width);
    else if (in_dtype == MLB_F32 && out_dtype == MLB_BF16)
        launch_kernel(silu_mul_kernel<float, __nv_bfloat16>, blocks, 256, 0, stream, (const float*)gate, (const float*)up, in_stride, n_partials, partial_stride, (__nv_bfloat16*)out, rows, width);
    else
        return fail(MLB_INVALID_ARGUMENT, "silu_mul: unsupported dtype pair %d -> %d", in_dtype, out_dtype);
    return check_launch("silu_mul");
}

// ------------------------------------------------------------------ fp32 -> bf16 cast
__global__ void cast_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
    pdl_prologue();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}

MLB_EXPORT int mlb_cast_f32_bf16(const float* in, void* out, long long n, cudaStream_t stream) {
    if (n < 0) return fail(MLB_INVALID_ARGUMENT, "cast: negative size");
    if (n == 0) return MLB_OK;
    launch_kernel(cast_bf16_kernel, (unsigned)((n + 255) / 256), 256, 0, stream, in, (__nv_bfloat16*)out, (size_t)n);
    return check_launch("cast_f32_bf16");
}

// ------------------------------------------------------------------ decode bookkeeping
// After a captured decode step: every sequence holds one token more.  The selected tokens
// already sit in the token buffer (the sampler wrote them there); this advances the
// positions, the per-sequence extents and the per-request draw counters on the device, so
// that the same captured step can run again without the host touching its inputs.
__global__ void decode_advance_kernel(int* __restrict__ positions, int* __restrict__ seq_pos0,
                                      int* __restrict__ seq_lens, long long* __restrict__ draw, int n,
                                      const int* __restrict__ tokens, const int* __restrict__ error_flag,
                                      int* __restrict__ result, const int* __restrict__ grows) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0 && result) result[n] = error_flag ? *error_flag : 0;
    if (i >= n) return;
    const int by = grows ? grows[i] : 1;      // 0 for a row that only fills the batch up: it stays at its first position
    positions[i] += by;
    seq_pos0[i] += by;
    seq_lens[i] += by;
    draw[i] += by;
    if (result) result[i] = tokens[i];
}

// `result` (may be null): n + 1 ints that receive the step's selected tokens and then the error flag, so
// that one device -> host copy brings everything the host wants to see of a step.  `grows` (may be null: every
// row grows): 1 or 0 per row.
MLB_EXPORT int mlb_decode_advance(int* positions, int* seq_pos0, int* seq_lens, long long* draw, int n,
                                  const int* tokens, const int* error_flag, int* result, const int* grows,
                                  cudaStream_t stream) {
    if (n < 0) return fail(MLB_INVALID_ARGUMENT, "decode_advance: negative size");
    if (result && !tokens) return fail(MLB_INVALID_ARGUMENT, "decode_advance: a result buffer needs the tokens");
    if (n == 0) return MLB_OK;
    launch_kernel(decode_advance_kernel, (n + 127) / 128, 128, 0, stream, positions, seq_pos0, seq_lens, draw, n, tokens,
                  error_flag, result, grows);
    return check_launch("decode_advance");
}

// ------------------------------------------------------------------ small copies without a framework in between
// A decode step moves a few dozen bytes each way; the launch path of a tensor library costs more
// than the copy.  Host memory must be pinned for the copy to be asynchronous.
MLB_EXPORT int mlb_copy_async(void* dst, const void* src, long long bytes, int to_device, cudaStream_t stream) {
    if (bytes < 0 || (bytes > 0 && (!dst || !src))) return fail(MLB_INVALID_ARGUMENT, "copy_async: bad arguments");
    if (bytes == 0) return MLB_OK;
    cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "copy_async: %s", cudaGetErrorString(e));
    return MLB_OK;
}

// ------------------------------------------------------------------ tokens from one step's selection into the next step's input
// dst[dst_index[i]] = src[src_index[i]]: the tokens a step selected go where the next step, whose metadata the
// host packed before it knew them, reads its input tokens.  Indices outside either array are skipped.
__global__ void scatter_int_kernel(int* __restrict__ dst, int dst_len, const int* __restrict__ dst_index,
                                   const int* __restrict__ src, int src_len, const int* __restrict__ src_index, int n) {
    pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int to = dst_index[i], from = src_index[i];
    if (to < 0 || to >= dst_len || from < 0 || from >= src_len) return;
    dst[to] = src[from];
}

MLB_EXPORT int mlb_scatter_int(int* dst, int dst_len, const int* dst_index, const int* src, int src_len,
                               const int* src_index, int n, cudaStream_t stream) {
    if (n < 0 || dst_len < 0 || src_len < 0) return fail(MLB_INVALID_ARGUMENT, "scatter_int: negative size");
    if (n == 0) return MLB_OK;
    if (!dst || !dst_index || !src || !src_index) return fail(MLB_INVALID_ARGUMENT, "scatter_int: an array is missing");
    launch_kernel(scatter_int_kernel, (n + 127) / 128, 128, 0, stream, dst, dst_len, dst_index, src, src_len, src_index, n);
    return check_launch("scatter_int");
}

// ------------------------------------------------------------------ a second stream for independent work of a step
// Two kernels of a step that do not depend on each other (the attention of the prompt portions and the attention
// of the decoded tokens beside them) may run side by side: the first goes to a second stream that starts where
// the main stream stands (fork) and the main stream waits for it before it goes on (join).  One stream and one
// event of each kind per device, made at first use.
namespace {
struct SideStream { cudaStream_t stream; cudaEvent_t forked, joined; bool made; };
SideStream side_streams[MAX_DEVICES] = {};

SideStream* side_stream_of_device() {
    SideStream& s = side_streams[device_index()];
    if (!s.made) {
        if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
        if (cudaEventCreateWithFlags(&s.forked, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        if (cudaEventCreateWithFlags(&s.joined, cudaEventDisableTiming) != cudaSuccess) return nullptr;
        s.made = true;
    }
    return &s;
}
}  // namespace

MLB_EXPORT void* mlb_side_stream() {
    SideStream* s = side_stream_of_device();
    return s ? (void*)s->stream : nullptr;
}

// the side stream continues from where `stream` stands now
MLB_EXPORT int mlb_stream_fork(cudaStream_t side, cudaStream_t stream) {
    SideStream* s = side_stream_of_device();
    if (!s || side != s->stream) return fail(MLB_INVALID_ARGUMENT, "stream_fork: not this device's side stream");
    cudaError_t e = cudaEventRecord(s->forked, stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(side, s->forked, 0);
    if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "stream_fork: %s", cudaGetErrorString(e));
    return MLB_OK;
}

// `stream` goes on only when everything queued on the side stream so far has run
MLB_EXPORT int mlb_stream_join(cudaStream_t side, cudaStream_t stream) {
    SideStream* s = side_stream_of_device();
    if (!s || side != s->stream) return fail(MLB_INVALID_ARGUMENT, "stream_join: not this device's side stream");
    cudaError_t e = cudaEventRecord(s->joined, side);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(stream, s->joined, 0);
    if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "stream_join: %s", cudaGetErrorString(e));
    return MLB_OK;
}

MLB_EXPORT int mlb_stream_synchronize(cudaStream_t stream) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail(MLB_CUDA_ERROR, "stream_synchronize: %s", cudaGetErrorString(e));
    return MLB_OK;
}
