// kernels::cross_entropy_fwd over the llmt_b200 C ABI, with llmt's checks and messages
// (src/kernels/cross_entropy.cu:81-106), and the fused LM-head form.
#include <initializer_list>

#include "llmt/core/error.h"
#include "llmt/kernels/cross_entropy.h"
#include "llmt_b200.h"

namespace llmt::kernels {

namespace {
// The checks both forms share: what the rows are, and the four per-row tensors.
void check_rows(const char* who, const Shape& rows, const Tensor& loss, const Tensor& row_nll, const Tensor& targets,
                const Tensor& mask) noexcept {
    if (targets.shape != rows) detail::fatal(who, "targets must be [B, T]");
    if (mask.shape != rows) detail::fatal(who, "mask must be [B, T]");
    if (row_nll.shape != rows) detail::fatal(who, "row_nll must be [B, T]");
    if (loss.numel() != 1) detail::fatal(who, "loss must be a [1] scalar");
    if (targets.dtype != DType::I32) detail::fatal(who, "targets must be I32");
    if (loss.dtype != DType::FP32 || row_nll.dtype != DType::FP32)
        detail::fatal(who, "loss/row_nll must be %s (host_result_t)", dtype_name(DType::FP32));
}
}  // namespace

void cross_entropy_fwd(const RunCtx& ctx, Tensor& loss, Tensor& row_nll, const Tensor& logits,
                       const Tensor& targets, const Tensor& mask) noexcept {
    if (logits.shape.rank != 3) detail::fatal("cross_entropy_fwd", "logits must be [B, T, V]");
    const int64_t rows = logits.shape[0] * logits.shape[1], v = logits.shape[2];
    check_rows("cross_entropy_fwd", Shape{logits.shape[0], logits.shape[1]}, loss, row_nll, targets, mask);
    if (mask.dtype != logits.dtype) detail::fatal("cross_entropy_fwd", "mask/logits dtype mismatch");
    for (const Tensor* t : std::initializer_list<const Tensor*>{&loss, &row_nll, &logits, &targets, &mask})
        if (!t->valid()) detail::fatal("cross_entropy_fwd", "invalid tensor (null data)");
    if (ctx.precision.reduce != DType::FP32)
        detail::fatal("cross_entropy_fwd", "no kernel instantiated for reduce precision %s", dtype_name(ctx.precision.reduce));
    if (logits.dtype != DType::FP32)
        detail::fatal("cross_entropy_fwd", "no kernel instantiated for dtype %s", dtype_name(logits.dtype));
    const int st = llmt_b200_cross_entropy_fwd(static_cast<float*>(loss.data), static_cast<float*>(row_nll.data),
                                               static_cast<const float*>(logits.data), static_cast<const int32_t*>(targets.data),
                                               static_cast<const float*>(mask.data), rows, v, v, ctx.stream);
    if (st != LLMT_B200_OK) detail::fatal("cross_entropy_fwd", "%s", llmt_b200_last_error());
}

namespace {
llmt_b200_gemm_desc lm_head_desc(const Tensor& x, const Tensor& w) noexcept {
    llmt_b200_gemm_desc d{};
    d.m = x.shape[0] * x.shape[1];
    d.k = x.shape[2];
    d.n = w.shape[0];
    d.batch = 1;
    d.lda = d.k; d.ldb = d.k; d.ldc = d.n;
    d.trans_a = 0; d.trans_b = 1;            // logits = x * w^T, w stored [V, C]
    d.dtype_ab = LLMT_B200_BF16;
    d.dtype_c = LLMT_B200_FP32;
    d.alpha = 1.0f;
    return d;
}
}  // namespace

size_t lm_head_cross_entropy_workspace_bytes(const Tensor& x, const Tensor& w) noexcept {
    if (x.shape.rank != 3 || w.shape.rank != 2) return 0;
    const llmt_b200_gemm_desc d = lm_head_desc(x, w);
    return static_cast<size_t>(llmt_b200_lm_head_ce_workspace_bytes(&d, x.data, w.data));
}

void lm_head_cross_entropy_fwd(const RunCtx& ctx, Tensor& loss, Tensor& row_nll, Tensor* logits, const Tensor& x,
                               const Tensor& w, const Tensor* bias, const Tensor& targets,
                               const Tensor& mask) noexcept {
    const char* who = "lm_head_cross_entropy_fwd";
    if (x.shape.rank != 3) detail::fatal(who, "x must be [B, T, C]");
    if (w.shape.rank != 2 || w.shape[1] != x.shape[2]) detail::fatal(who, "w must be [V, C]");
    if (x.dtype != DType::BF16 || w.dtype != DType::BF16) detail::fatal(who, "x and w must be bf16");
    check_rows(who, Shape{x.shape[0], x.shape[1]}, loss, row_nll, targets, mask);
    if (mask.dtype != DType::FP32) detail::fatal(who, "mask must be fp32");
    for (const Tensor* t : std::initializer_list<const Tensor*>{&loss, &row_nll, &x, &w, &targets, &mask})
        if (!t->valid()) detail::fatal(who, "invalid tensor (null data)");
    llmt_b200_gemm_desc d = lm_head_desc(x, w);
    if (logits != nullptr) {
        if (!logits->valid() || logits->dtype != DType::FP32 || logits->shape != Shape{x.shape[0], x.shape[1], w.shape[0]})
            detail::fatal(who, "logits must be fp32 [B, T, V]");
    }
    if (bias != nullptr) {
        if (!bias->valid() || bias->numel() != w.shape[0]) detail::fatal(who, "bias must be [V]");
        d.epilogue = LLMT_B200_EPI_BIAS;
        d.bias = bias->data;
        d.bias_dtype = static_cast<int32_t>(bias->dtype);
    }
    d.workspace = ctx.blas_workspace;
    d.workspace_bytes = ctx.blas_workspace_bytes;
    const int st = llmt_b200_lm_head_ce_fwd(&d, logits != nullptr ? logits->data : nullptr, x.data, w.data,
                                            static_cast<const int32_t*>(targets.data), static_cast<const float*>(mask.data),
                                            static_cast<float*>(row_nll.data), static_cast<float*>(loss.data), ctx.stream);
    if (st != LLMT_B200_OK) detail::fatal(who, "%s", llmt_b200_last_error());
}

void cross_entropy_bwd(const RunCtx& ctx, Tensor& dlogits, const Tensor& logits, const Tensor& targets,
                       const Tensor& mask, float dloss) noexcept {
    const char* who = "cross_entropy_bwd";
    if (logits.shape.rank != 3) detail::fatal(who, "logits must be [B, T, V]");
    if (dlogits.shape != logits.shape) detail::fatal(who, "dlogits/logits shape mismatch");
    if (logits.dtype != DType::FP32 || dlogits.dtype != DType::FP32) detail::fatal(who, "logits and dlogits must be fp32");
    const Shape bt{logits.shape[0], logits.shape[1]};
    if (targets.shape != bt || targets.dtype != DType::I32) detail::fatal(who, "targets must be [B, T] I32");
    if (mask.shape != bt || mask.dtype != DType::FP32) detail::fatal(who, "mask must be [B, T] fp32");
    for (const Tensor* t : std::initializer_list<const Tensor*>{&dlogits, &logits, &targets, &mask})
        if (!t->valid()) detail::fatal(who, "invalid tensor (null data)");
    const int64_t v = logits.shape[2];
    const int st = llmt_b200_cross_entropy_bwd(static_cast<float*>(dlogits.data), static_cast<const float*>(logits.data),
                                               static_cast<const int32_t*>(targets.data), static_cast<const float*>(mask.data),
                                               dloss, bt[0] * bt[1], v, v, v, ctx.stream);
    if (st != LLMT_B200_OK) detail::fatal(who, "%s", llmt_b200_last_error());
}

void lm_head_cross_entropy_bwd(const RunCtx& ctx, Tensor& dlogits, const Tensor& x, const Tensor& w, const Tensor* bias,
                               const Tensor& targets, const Tensor& mask, float dloss, bool stats_valid) noexcept {
    const char* who = "lm_head_cross_entropy_bwd";
    if (x.shape.rank != 3) detail::fatal(who, "x must be [B, T, C]");
    if (w.shape.rank != 2 || w.shape[1] != x.shape[2]) detail::fatal(who, "w must be [V, C]");
    if (x.dtype != DType::BF16 || w.dtype != DType::BF16) detail::fatal(who, "x and w must be bf16");
    const Shape bt{x.shape[0], x.shape[1]};
    if (dlogits.shape != Shape{bt[0], bt[1], w.shape[0]}) detail::fatal(who, "dlogits must be [B, T, V]");
    if (dlogits.dtype != DType::BF16 && dlogits.dtype != DType::FP32) detail::fatal(who, "dlogits must be bf16 or fp32");
    if (targets.shape != bt || targets.dtype != DType::I32) detail::fatal(who, "targets must be [B, T] I32");
    if (mask.shape != bt || mask.dtype != DType::FP32) detail::fatal(who, "mask must be [B, T] fp32");
    for (const Tensor* t : std::initializer_list<const Tensor*>{&dlogits, &x, &w, &targets, &mask})
        if (!t->valid()) detail::fatal(who, "invalid tensor (null data)");
    llmt_b200_gemm_desc d = lm_head_desc(x, w);
    d.dtype_c = static_cast<int32_t>(dlogits.dtype);
    if (bias != nullptr) {
        if (!bias->valid() || bias->numel() != w.shape[0]) detail::fatal(who, "bias must be [V]");
        d.epilogue = LLMT_B200_EPI_BIAS;
        d.bias = bias->data;
        d.bias_dtype = static_cast<int32_t>(bias->dtype);
    }
    d.workspace = ctx.blas_workspace;
    d.workspace_bytes = ctx.blas_workspace_bytes;
    const int st = llmt_b200_lm_head_ce_bwd(&d, dlogits.data, x.data, w.data, static_cast<const int32_t*>(targets.data),
                                            static_cast<const float*>(mask.data), dloss, stats_valid ? 1 : 0, ctx.stream);
    if (st != LLMT_B200_OK) detail::fatal(who, "%s", llmt_b200_last_error());
}

}  // namespace llmt::kernels
