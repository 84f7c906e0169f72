// kernels::matmul over the llmt_b200 C ABI.  The validation order and the abort
// messages follow llmt's check() (src/kernels/matmul.cpp:175-214) so a caller
// sees the same behaviour; the product itself is llmt_b200_gemm.
#include <string>

#include "llmt/core/error.h"
#include "llmt/kernels/algo_cache.h"
#include "llmt/kernels/matmul.h"
#include "llmt_b200.h"

namespace llmt::kernels {

namespace {

// The last two dimensions of a rank-2/3 tensor as a matrix, plus how many of them there are.
struct MatrixView {
    int64_t rows, cols, items, item_stride;
    static MatrixView of(const Tensor& t) noexcept {
        const int last = t.shape.rank - 1;
        MatrixView v{t.shape[last - 1], t.shape[last], 1, 0};
        if (t.shape.rank == 3) {
            v.items = t.shape[0];
            v.item_stride = v.rows * v.cols;
        }
        return v;
    }
    // op(X): the same storage read as its transpose
    MatrixView op(bool transposed) const noexcept {
        return transposed ? MatrixView{cols, rows, items, item_stride} : *this;
    }
};

struct Problem {
    int64_t m, n, k, batch, stride_a, stride_b, stride_c;
};

bool supported(DType t) noexcept { return t == DType::FP32 || t == DType::BF16; }

// The checks llmt makes, in llmt's order and with llmt's messages, so that a caller that trips
// one sees the same abort.
Problem check(const Tensor& c, const Tensor& a, const Tensor& b, bool trans_a, bool trans_b) noexcept {
    const int rank = c.shape.rank;
    if (rank != 2 && rank != 3) detail::fatal("matmul", "expected rank-2 or rank-3 tensors (got %d)", rank);
    if (a.shape.rank != rank || b.shape.rank != rank) detail::fatal("matmul", "mixed ranks in one matmul");
    if (a.dtype != b.dtype) detail::fatal("matmul", "mixed dtypes in one matmul");
    if (!c.valid() || !a.valid() || !b.valid()) detail::fatal("matmul", "invalid tensor (null data)");
    if (!supported(a.dtype)) detail::fatal("matmul", "dtype %s not yet supported", dtype_name(a.dtype));
    if (a.dtype == DType::FP32 && c.dtype != DType::FP32) detail::fatal("matmul", "mixed dtypes in one matmul");
    if (!supported(c.dtype)) detail::fatal("matmul", "dtype %s not yet supported", dtype_name(c.dtype));
    const MatrixView va = MatrixView::of(a), vb = MatrixView::of(b), vc = MatrixView::of(c);
    const MatrixView oa = va.op(trans_a), ob = vb.op(trans_b);  // [m, k] and [k, n]
    if (oa.cols != ob.rows)
        detail::fatal("matmul", "inner dims disagree: %lld vs %lld", static_cast<long long>(oa.cols),
                      static_cast<long long>(ob.rows));
    if (vc.rows != oa.rows || vc.cols != ob.cols) detail::fatal("matmul", "C shape mismatch");
    if (vb.items != va.items || vc.items != va.items) detail::fatal("matmul", "batch sizes disagree");
    return Problem{oa.rows, ob.cols, oa.cols, va.items, va.item_stride, vb.item_stride, vc.item_stride};
}

// The precision policy must name the arithmetic the operand dtype implies
// (llmt's single capability guard, matmul.cpp:72-77, extended by the bf16 mode).
void check_policy(const RunCtx& ctx, DType ab) noexcept {
    const PrecisionPolicy& pp = ctx.precision;
    const bool ok = (ab == DType::FP32 && pp.gemm_compute == DType::FP32 && pp.reduce == DType::FP32) ||
                    (ab == DType::BF16 && pp.gemm_compute == DType::BF16 && pp.reduce == DType::FP32);
    if (!ok)
        detail::fatal("matmul", "gemm_compute/reduce precision %s/%s not yet supported for %s operands",
                      dtype_name(pp.gemm_compute), dtype_name(pp.reduce), dtype_name(ab));
}

// Validates one call the way llmt does and fills the C-ABI descriptor for it.
llmt_b200_gemm_desc make_desc(const RunCtx& ctx, const Tensor& c, const Tensor& a, const Tensor& b,
                              bool trans_a, bool trans_b, float alpha, float beta,
                              const Epilogue& epi) noexcept {
    const Problem p = check(c, a, b, trans_a, trans_b);
    check_policy(ctx, a.dtype);
    const int r = c.shape.rank - 2;
    llmt_b200_gemm_desc d{};
    d.m = p.m; d.n = p.n; d.k = p.k; d.batch = p.batch;
    d.lda = a.shape[r + 1]; d.ldb = b.shape[r + 1]; d.ldc = c.shape[r + 1];  // contiguous views
    d.stride_a = p.stride_a; d.stride_b = p.stride_b; d.stride_c = p.stride_c;
    d.trans_a = trans_a; d.trans_b = trans_b;
    d.dtype_ab = static_cast<int32_t>(a.dtype);
    d.dtype_c = static_cast<int32_t>(c.dtype);
    d.alpha = alpha; d.beta = beta;
    if (epi.bias != nullptr) {
        if (!epi.bias->valid() || epi.bias->numel() != p.n) detail::fatal("matmul", "bias must be [N]");
        d.epilogue |= LLMT_B200_EPI_BIAS;
        d.bias = epi.bias->data;
        d.bias_dtype = static_cast<int32_t>(epi.bias->dtype);
    }
    if (epi.gelu) d.epilogue |= LLMT_B200_EPI_GELU;
    if (epi.save_pre != nullptr || epi.gelu_bwd_of != nullptr) {
        const Tensor* aux = epi.save_pre != nullptr ? epi.save_pre : epi.gelu_bwd_of;
        if (epi.save_pre != nullptr && epi.gelu_bwd_of != nullptr) detail::fatal("matmul", "save_pre and gelu_bwd_of exclude each other");
        if (!aux->valid() || aux->shape != c.shape || aux->dtype != c.dtype)
            detail::fatal("matmul", "the pre-activation must have C's shape and dtype");
        d.epilogue |= epi.save_pre != nullptr ? LLMT_B200_EPI_SAVE_PRE : LLMT_B200_EPI_GELU_BWD;
        d.aux = aux->data;
    }
    if (epi.dbias != nullptr) {
        if (!epi.dbias->valid() || epi.dbias->numel() != p.m || epi.dbias->dtype != DType::FP32)
            detail::fatal("matmul", "dbias must be fp32 [M]");
        d.dbias = static_cast<float*>(epi.dbias->data);
        d.dbias_beta = epi.dbias_beta;
    }
    if (ctx.algo_cache != nullptr) {
        const AlgoKey key{p.m, p.n, p.k, p.batch, (trans_a ? 1LL : 0LL) | (trans_b ? 2LL : 0LL),
                          static_cast<int64_t>(a.dtype), static_cast<int64_t>(c.dtype),
                          static_cast<int64_t>(d.epilogue) | (d.dbias != nullptr ? 256LL : 0LL)};
        auto& map = ctx.algo_cache->map;
        if (map.find(key) == map.end()) {
            char buf[256];
            llmt_b200_gemm_plan(&d, buf, sizeof buf);
            map.emplace(key, std::string(buf));
        }
    }
    return d;
}

}  // namespace

void matmul_ex(const RunCtx& ctx, Tensor& c, const Tensor& a, const Tensor& b, bool trans_a,
               bool trans_b, float alpha, float beta, const Epilogue& epi) noexcept {
    llmt_b200_gemm_desc d = make_desc(ctx, c, a, b, trans_a, trans_b, alpha, beta, epi);
    d.workspace = ctx.blas_workspace;
    d.workspace_bytes = ctx.blas_workspace_bytes;
    const int st = llmt_b200_gemm(&d, c.data, a.data, b.data, ctx.stream);
    if (st != LLMT_B200_OK) detail::fatal("matmul", "%s", llmt_b200_last_error());
}

void matmul_grouped(const RunCtx& ctx, const MatmulCall* calls, int count) noexcept {
    constexpr int kMax = 8;
    if (count < 1 || count > kMax) detail::fatal("matmul_grouped", "count must be 1..%d", kMax);
    bool all_bf16 = true;
    for (int i = 0; i < count; ++i) {
        if (calls[i].c == nullptr || calls[i].a == nullptr || calls[i].b == nullptr)
            detail::fatal("matmul_grouped", "invalid tensor (null data)");
        all_bf16 = all_bf16 && calls[i].a->dtype == DType::BF16;
    }
    if (!all_bf16) {  // the strict fp32 path has no grouped kernel
        for (int i = 0; i < count; ++i)
            matmul_ex(ctx, *calls[i].c, *calls[i].a, *calls[i].b, calls[i].trans_a, calls[i].trans_b,
                      calls[i].alpha, calls[i].beta, calls[i].epi);
        return;
    }
    llmt_b200_gemm_desc d[kMax];
    void* c[kMax];
    const void* a[kMax];
    const void* b[kMax];
    for (int i = 0; i < count; ++i) {
        d[i] = make_desc(ctx, *calls[i].c, *calls[i].a, *calls[i].b, calls[i].trans_a, calls[i].trans_b,
                         calls[i].alpha, calls[i].beta, calls[i].epi);
        c[i] = calls[i].c->data; a[i] = calls[i].a->data; b[i] = calls[i].b->data;
    }
    // Carve the Device-owned scratch into one 256-byte aligned piece per problem.
    uint64_t need[kMax];
    if (llmt_b200_gemm_grouped_workspace_bytes(d, count, need) != LLMT_B200_OK)
        detail::fatal("matmul_grouped", "%s", llmt_b200_last_error());
    size_t off = 0;
    for (int i = 0; i < count; ++i) {
        if (need[i] == 0) continue;
        if (off + need[i] > ctx.blas_workspace_bytes)
            detail::fatal("matmul_grouped", "workspace too small: need %zu B, have %zu B",
                          off + static_cast<size_t>(need[i]), ctx.blas_workspace_bytes);
        d[i].workspace = static_cast<char*>(ctx.blas_workspace) + off;
        d[i].workspace_bytes = need[i];
        off += (static_cast<size_t>(need[i]) + 255) / 256 * 256;
    }
    if (llmt_b200_gemm_grouped(d, c, a, b, count, ctx.stream) != LLMT_B200_OK)
        detail::fatal("matmul_grouped", "%s", llmt_b200_last_error());
}

void matmul(const RunCtx& ctx, Tensor& c, const Tensor& a, const Tensor& b, bool trans_a,
            bool trans_b, float alpha, float beta) noexcept {
    matmul_ex(ctx, c, a, b, trans_a, trans_b, alpha, beta, Epilogue{});
}

}  // namespace llmt::kernels
