// The library matrix product of the bf16 path, called without a tensor framework in between:
//     y[M, N] = x[M, K] * W[N, K]^T  (+ y),   bf16 operands, fp32 accumulation, y in bf16 or fp32.
// The reference calls hipBLASLt for the same projections (src/ops/optimized.cpp:349-403: bf16 x bf16 with
// 32-bit compute); this is the cuBLASLt call of the same shape, as one C call with cached plans and no tensor
// framework on the way (the host cost of a product, ~12 us, is the library's own either way).
//
// cuBLASLt is taken from the process (dlopen by soname: the copy that is already loaded is returned), so the
// library needs no link-time dependency.  Plans (operation and layout descriptors plus the heuristic's first
// algorithm) are cached per shape; the workspace belongs to the caller.
#include "common.cuh"

#include <cublasLt.h>
#include <dlfcn.h>

#include <map>
#include <mutex>
#include <tuple>

using namespace mlb;

MLB_DEFINE_LAST_ERROR()

namespace {

struct Api {
    cublasStatus_t (*create)(cublasLtHandle_t*);
    cublasStatus_t (*desc_create)(cublasLtMatmulDesc_t*, cublasComputeType_t, cudaDataType_t);
    cublasStatus_t (*desc_set)(cublasLtMatmulDesc_t, cublasLtMatmulDescAttributes_t, const void*, size_t);
    cublasStatus_t (*layout_create)(cublasLtMatrixLayout_t*, cudaDataType, uint64_t, uint64_t, int64_t);
    cublasStatus_t (*pref_create)(cublasLtMatmulPreference_t*);
    cublasStatus_t (*pref_set)(cublasLtMatmulPreference_t, cublasLtMatmulPreferenceAttributes_t, const void*, size_t);
    cublasStatus_t (*pref_destroy)(cublasLtMatmulPreference_t);
    cublasStatus_t (*heuristic)(cublasLtHandle_t, cublasLtMatmulDesc_t, cublasLtMatrixLayout_t, cublasLtMatrixLayout_t,
                                cublasLtMatrixLayout_t, cublasLtMatrixLayout_t, cublasLtMatmulPreference_t, int,
                                cublasLtMatmulHeuristicResult_t*, int*);
    cublasStatus_t (*matmul)(cublasLtHandle_t, cublasLtMatmulDesc_t, const void*, const void*, cublasLtMatrixLayout_t,
                             const void*, cublasLtMatrixLayout_t, const void*, const void*, cublasLtMatrixLayout_t, void*,
                             cublasLtMatrixLayout_t, const cublasLtMatmulAlgo_t*, void*, size_t, cudaStream_t);
    cublasLtHandle_t handle;
    bool ready;
};

Api& api() {
    static Api a = {};
    static std::once_flag once;
    std::call_once(once, [] {
        void* so = dlopen("libcublasLt.so.12", RTLD_NOW | RTLD_GLOBAL);
        if (!so) so = dlopen("libcublasLt.so", RTLD_NOW | RTLD_GLOBAL);
        if (!so) return;
#define MLB_SYM(field, name) a.field = reinterpret_cast<decltype(a.field)>(dlsym(so, name)); if (!a.field) return
        MLB_SYM(create, "cublasLtCreate");
        MLB_SYM(desc_create, "cublasLtMatmulDescCreate");
        MLB_SYM(desc_set, "cublasLtMatmulDescSetAttribute");
        MLB_SYM(layout_create, "cublasLtMatrixLayoutCreate");
        MLB_SYM(pref_create, "cublasLtMatmulPreferenceCreate");
        MLB_SYM(pref_set, "cublasLtMatmulPreferenceSetAttribute");
        MLB_SYM(pref_destroy, "cublasLtMatmulPreferenceDestroy");
        MLB_SYM(heuristic, "cublasLtMatmulAlgoGetHeuristic");
        MLB_SYM(matmul, "cublasLtMatmul");
#undef MLB_SYM
        a.ready = a.create(&a.handle) == CUBLAS_STATUS_SUCCESS;
    });
    return a;
}

struct Plan {
    cublasLtMatmulDesc_t op;
    cublasLtMatrixLayout_t w, x, y;
    cublasLtMatmulAlgo_t algo;
};

using Key = std::tuple<int, int, int, long long, long long, long long, int, size_t>;
std::map<Key, Plan> plans;          // lives as long as the process: a model has a handful of shapes
std::mutex plans_lock;

// Row-major y[M, N] = x[M, K] W[N, K]^T is, in the library's column-major terms, y^T[N, M] = op_T(Wc) * xc with
// Wc the K x N view of W (leading dimension ldw) and xc the K x M view of x.
int make_plan(Api& a, const Key& key, Plan& plan) {
    const int M = std::get<0>(key), N = std::get<1>(key), K = std::get<2>(key);
    const long long ldx = std::get<3>(key), ldw = std::get<4>(key), ldo = std::get<5>(key);
    const int out_bf16 = std::get<6>(key);
    const size_t workspace = std::get<7>(key);
    if (a.desc_create(&plan.op, CUBLAS_COMPUTE_32F, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS)
        return fail(MLB_CUDA_ERROR, "gemm_lib: cannot create the operation descriptor");
    const cublasOperation_t transposed = CUBLAS_OP_T, plain = CUBLAS_OP_N;
    a.desc_set(plan.op, CUBLASLT_MATMUL_DESC_TRANSA, &transposed, sizeof(transposed));
    a.desc_set(plan.op, CUBLASLT_MATMUL_DESC_TRANSB, &plain, sizeof(plain));
    const cudaDataType out_type = out_bf16 ? CUDA_R_16BF : CUDA_R_32F;
    if (a.layout_create(&plan.w, CUDA_R_16BF, (uint64_t)K, (uint64_t)N, ldw) != CUBLAS_STATUS_SUCCESS ||
        a.layout_create(&plan.x, CUDA_R_16BF, (uint64_t)K, (uint64_t)M, ldx) != CUBLAS_STATUS_SUCCESS ||
        a.layout_create(&plan.y, out_type, (uint64_t)N, (uint64_t)M, ldo) != CUBLAS_STATUS_SUCCESS)
        return fail(MLB_CUDA_ERROR, "gemm_lib: cannot create the matrix layouts");
    cublasLtMatmulPreference_t pref;
    if (a.pref_create(&pref) != CUBLAS_STATUS_SUCCESS) return fail(MLB_CUDA_ERROR, "gemm_lib: cannot create the preference");
    a.pref_set(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &workspace, sizeof(workspace));
    cublasLtMatmulHeuristicResult_t found = {};
    int count = 0;
    const cublasStatus_t st = a.heuristic(a.handle, plan.op, plan.w, plan.x, plan.y, plan.y, pref, 1, &found, &count);
    a.pref_destroy(pref);
    if (st != CUBLAS_STATUS_SUCCESS || count < 1)
        return fail(MLB_UNSUPPORTED_SIZE, "gemm_lib: the library has no algorithm for M=%d N=%d K=%d (status %d)", M, N, K, (int)st);
    plan.algo = found.algo;
    return MLB_OK;
}

}  // namespace

// 1 when cuBLASLt could be taken from the process
MLB_EXPORT int mlb_lt_available() { return api().ready ? 1 : 0; }

// out[M, N] (bf16 or fp32, row pitch ldo) = x[M, K] * w[N, K]^T (+ out, fp32 only, when accumulate).
// `workspace`: scratch of workspace_bytes on the device, owned by the caller and used by one stream at a time.
MLB_EXPORT int mlb_lt_matmul(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo,
                             int out_bf16, int accumulate, int M, int N, int K, void* workspace, long long workspace_bytes,
                             cudaStream_t stream) {
    Api& a = api();
    if (!a.ready) return fail(MLB_CUDA_ERROR, "gemm_lib: cuBLASLt is not available in this process");
    if (M <= 0 || N <= 0 || K <= 0 || ldx < K || ldw < K || ldo < N) return fail(MLB_INVALID_ARGUMENT, "gemm_lib: bad sizes M=%d N=%d K=%d", M, N, K);
    if (accumulate && out_bf16) return fail(MLB_INVALID_ARGUMENT, "gemm_lib: accumulation needs an fp32 output");
    if (!x || !w || !out || workspace_bytes < 0 || (workspace_bytes > 0 && !workspace)) return fail(MLB_INVALID_ARGUMENT, "gemm_lib: missing operand");
    const Key key(M, N, K, ldx, ldw, ldo, out_bf16, (size_t)workspace_bytes);
    Plan plan;
    {
        std::lock_guard<std::mutex> guard(plans_lock);
        auto it = plans.find(key);
        if (it == plans.end()) {
            Plan fresh = {};
            const int status = make_plan(a, key, fresh);
            if (status != MLB_OK) return status;
            it = plans.emplace(key, fresh).first;
        }
        plan = it->second;
    }
    const float one = 1.0f, zero = 0.0f;
    const cublasStatus_t st = a.matmul(a.handle, plan.op, &one, w, plan.w, x, plan.x, accumulate ? &one : &zero, out, plan.y, out,
                                       plan.y, &plan.algo, workspace, (size_t)workspace_bytes, stream);
    if (st != CUBLAS_STATUS_SUCCESS) return fail(MLB_CUDA_ERROR, "gemm_lib: cublasLtMatmul failed with status %d (M=%d N=%d K=%d)", (int)st, M, N, K);
    return MLB_OK;
}
