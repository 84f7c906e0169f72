// TEST / BASELINE INFRASTRUCTURE, NOT PRODUCT.
//
// llmt's matmul refuses bf16 (src/kernels/matmul.cpp:72-77,185-188), so "what llmt's own
// path would do in bf16" has to be a harness: this file repeats llmt's cuBLASLt call
// pattern — the row-major -> column-major operand swap of src/kernels/matmul.cpp:7-21 and
// :119-138 (B goes into Lt's A slot, A into the B slot, each keeps its transpose flag, the
// problem is (N, M, K), every leading dimension is the row-major column count), a 32 MiB
// workspace (include/llmt/core/device.h:39), top-1 heuristic cached per problem — with
// CUDA_R_16BF operands, CUBLAS_COMPUTE_32F accumulation and fp32 scale type.  Optional Lt
// epilogues (BIAS, GELU_BIAS) for the fused cases.  Used as a second checker for accuracy
// ("no worse than 2x cuBLASLt's error") and as a speed comparator.  Nothing in llmt_b200
// links it.
#include <cublasLt.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <map>
#include <tuple>

#define CMP_API extern "C" __attribute__((visibility("default")))

namespace {
struct Ctx {
    cublasLtHandle_t lt = nullptr;
    void* ws = nullptr;
    size_t ws_bytes = 32ull << 20;
    std::map<std::tuple<int64_t, int64_t, int64_t, int64_t, int, int, int, int>, cublasLtMatmulAlgo_t> cache;
};
}  // namespace

CMP_API void* cmp_create() {
    Ctx* c = new Ctx;
    if (cublasLtCreate(&c->lt) != CUBLAS_STATUS_SUCCESS) { delete c; return nullptr; }
    if (cudaMalloc(&c->ws, c->ws_bytes) != cudaSuccess) { cublasLtDestroy(c->lt); delete c; return nullptr; }
    return c;
}

CMP_API void cmp_destroy(void* h) {
    Ctx* c = static_cast<Ctx*>(h);
    if (!c) return;
    cudaFree(c->ws);
    cublasLtDestroy(c->lt);
    delete c;
}

// C[M,N] = alpha*op(A)*op(B) + beta*C (row-major, contiguous), bf16 A/B, C bf16 (c_fp32 = 0)
// or fp32.  epilogue: 0 none, 1 bias (fp32 or bf16 per Lt's rule = C's type), 3 bias + tanh-GELU,
// 4 bias gradient: `bias` receives sum_p op(A)[i, p] for i < M (after the operand swap our A
// sits in Lt's B slot, so this is Lt's BGRADB; Lt overwrites, it does not accumulate).
// Returns 0 on success, otherwise the failing cublasStatus_t (or -1 when no algorithm exists).
CMP_API int cmp_matmul_bf16(void* h, void* c, const void* a, const void* b, int64_t m, int64_t n, int64_t k,
                            int64_t batch, int trans_a, int trans_b, float alpha, float beta, int c_fp32,
                            int epilogue, const void* bias, void* stream) {
    Ctx* ctx = static_cast<Ctx*>(h);
    const int64_t a_rows = trans_a ? k : m, a_cols = trans_a ? m : k;
    const int64_t b_rows = trans_b ? n : k, b_cols = trans_b ? k : n;
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t la = nullptr, lb = nullptr, lc = nullptr;
    cublasStatus_t st = cublasLtMatmulDescCreate(&op, CUBLAS_COMPUTE_32F, CUDA_R_32F);
    if (st != CUBLAS_STATUS_SUCCESS) return st;
    const cublasOperation_t slot_a = trans_b ? CUBLAS_OP_T : CUBLAS_OP_N;  // B sits in Lt's A slot
    const cublasOperation_t slot_b = trans_a ? CUBLAS_OP_T : CUBLAS_OP_N;
    cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSA, &slot_a, sizeof slot_a);
    cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_TRANSB, &slot_b, sizeof slot_b);
    if (epilogue != 0) {
        const cublasLtEpilogue_t epi = epilogue == 3 ? CUBLASLT_EPILOGUE_GELU_BIAS
                                     : epilogue == 4 ? CUBLASLT_EPILOGUE_BGRADB : CUBLASLT_EPILOGUE_BIAS;
        cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_EPILOGUE, &epi, sizeof epi);
        cublasLtMatmulDescSetAttribute(op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof bias);
    }
    auto layout = [&](cublasLtMatrixLayout_t* l, cudaDataType_t t, int64_t rows, int64_t cols) {
        // a row-major [rows, cols] buffer read column-major is [cols, rows] with ld = cols
        cublasLtMatrixLayoutCreate(l, t, static_cast<uint64_t>(cols), static_cast<uint64_t>(rows), cols);
        if (batch > 1) {
            const int32_t bc = static_cast<int32_t>(batch);
            const int64_t stride = rows * cols;
            cublasLtMatrixLayoutSetAttribute(*l, CUBLASLT_MATRIX_LAYOUT_BATCH_COUNT, &bc, sizeof bc);
            cublasLtMatrixLayoutSetAttribute(*l, CUBLASLT_MATRIX_LAYOUT_STRIDED_BATCH_OFFSET, &stride, sizeof stride);
        }
    };
    layout(&la, CUDA_R_16BF, b_rows, b_cols);
    layout(&lb, CUDA_R_16BF, a_rows, a_cols);
    layout(&lc, c_fp32 ? CUDA_R_32F : CUDA_R_16BF, m, n);

    const auto key = std::make_tuple(m, n, k, batch, trans_a, trans_b, c_fp32, epilogue);
    auto it = ctx->cache.find(key);
    int rc = 0;
    if (it == ctx->cache.end()) {
        cublasLtMatmulPreference_t pref = nullptr;
        cublasLtMatmulPreferenceCreate(&pref);
        cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ctx->ws_bytes,
                                             sizeof ctx->ws_bytes);
        cublasLtMatmulHeuristicResult_t res{};
        int found = 0;
        st = cublasLtMatmulAlgoGetHeuristic(ctx->lt, op, la, lb, lc, lc, pref, 1, &res, &found);
        cublasLtMatmulPreferenceDestroy(pref);
        if (st != CUBLAS_STATUS_SUCCESS || found == 0) rc = st != CUBLAS_STATUS_SUCCESS ? st : -1;
        else it = ctx->cache.emplace(key, res.algo).first;
    }
    if (rc == 0) {
        st = cublasLtMatmul(ctx->lt, op, &alpha, b, la, a, lb, &beta, c, lc, c, lc, &it->second, ctx->ws,
                            ctx->ws_bytes, static_cast<cudaStream_t>(stream));
        rc = st;
    }
    cublasLtMatrixLayoutDestroy(la);
    cublasLtMatrixLayoutDestroy(lb);
    cublasLtMatrixLayoutDestroy(lc);
    cublasLtMatmulDescDestroy(op);
    return rc;
}
