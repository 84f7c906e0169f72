// Attention forward/backward as compositions of the strided-batched GEMMs and
// the masked softmax helpers (llmt src/kernels/attention.cpp:34-64; backward
// products from llmt docs/TODO.md:226-228).
#include <cmath>
#include <initializer_list>

#include "llmt/core/error.h"
#include "llmt/kernels/attention.h"
#include "llmt/kernels/matmul.h"
#include "llmt/kernels/permute.h"
#include "llmt_b200.h"

namespace llmt::kernels {

namespace {
// [B,H,T,x] -> [B*H,T,x]: same bytes (llmt attention.cpp:28-30).
Tensor fold(const Tensor& t) noexcept {
    Tensor r = t;
    r.shape = Shape{t.shape[0] * t.shape[1], t.shape[2], t.shape[3]};
    return r;
}
}  // namespace

namespace {
// probs = softmax(alpha * A B^T) through the fused launch pair, if the tensors are bf16 and the
// context's workspace holds the statistics; false = the caller composes GEMM and softmax itself.
bool fused_scores_softmax(const RunCtx& ctx, llmt_b200_gemm_desc d, void* probs, const void* a, const void* b,
                          MaskSpec mask, const char* who) noexcept {
    if (d.dtype_ab != LLMT_B200_BF16) return false;
    const uint64_t need = llmt_b200_gemm_softmax_workspace_bytes(&d, a, b);
    if (need == 0 || ctx.blas_workspace == nullptr || need > ctx.blas_workspace_bytes) return false;
    d.workspace = ctx.blas_workspace;
    d.workspace_bytes = ctx.blas_workspace_bytes;
    if (llmt_b200_gemm_softmax_fwd(&d, probs, a, b, mask.kind == MaskKind::Causal, nullptr, ctx.stream) != LLMT_B200_OK)
        detail::fatal(who, "%s", llmt_b200_last_error());
    return true;
}
}  // namespace

void softmax_fwd(const RunCtx& ctx, Tensor& y, const Tensor& x, MaskSpec mask) noexcept {
    if (x.shape.rank != 3) detail::fatal("softmax_fwd", "x must be [batch, Tq, Tk]");
    if (y.shape != x.shape) detail::fatal("softmax_fwd", "y/x shape mismatch");
    if (y.dtype != x.dtype) detail::fatal("softmax_fwd", "y/x dtype mismatch");
    if (!y.valid() || !x.valid()) detail::fatal("softmax_fwd", "invalid tensor (null data)");
    const int st = llmt_b200_softmax_fwd(y.data, x.data, x.shape[0] * x.shape[1], x.shape[1], x.shape[2],
                                         static_cast<int32_t>(x.dtype), mask.kind == MaskKind::Causal,
                                         ctx.stream);
    if (st != LLMT_B200_OK) detail::fatal("softmax_fwd", "%s", llmt_b200_last_error());
}

void attention_fwd(const RunCtx& ctx, Tensor& y, Tensor& scores, Tensor& y_heads, const Tensor& q,
                   const Tensor& k, const Tensor& v, MaskSpec mask) noexcept {
    if (ctx.backend != KernelBackend::Naive) detail::fatal("attention_fwd", "no fused variant implemented yet");
    for (const Tensor* t : std::initializer_list<const Tensor*>{&scores, &y_heads, &q, &k, &v}) {
        if (!t->valid()) detail::fatal("attention_fwd", "invalid tensor (null data)");
        if (t->shape.rank != 4) detail::fatal("attention_fwd", "expected rank-4 head tensors");
    }
    if (k.shape != q.shape || v.shape != q.shape || y_heads.shape != q.shape)
        detail::fatal("attention_fwd", "q/k/v/y_heads must share one [B, H, T, hd] shape");
    const int64_t b = q.shape[0], h = q.shape[1], t = q.shape[2], hd = q.shape[3];
    if (scores.shape != Shape{b, h, t, t}) detail::fatal("attention_fwd", "scores must be [B, H, T, T]");
    Tensor s3 = fold(scores), o3 = fold(y_heads);
    const Tensor q3 = fold(q), k3 = fold(k), v3 = fold(v);
    const float scale = 1.0f / std::sqrt(static_cast<float>(hd));
    llmt_b200_gemm_desc sd{};
    sd.m = t; sd.n = t; sd.k = hd; sd.batch = b * h;
    sd.lda = hd; sd.ldb = hd; sd.ldc = t;
    sd.stride_a = t * hd; sd.stride_b = t * hd; sd.stride_c = t * t;
    sd.trans_a = 0; sd.trans_b = 1;
    sd.dtype_ab = static_cast<int32_t>(q.dtype); sd.dtype_c = static_cast<int32_t>(scores.dtype);
    sd.alpha = scale; sd.beta = 0.0f;
    if (k.dtype != q.dtype || !fused_scores_softmax(ctx, sd, s3.data, q3.data, k3.data, mask, "attention_fwd")) {
        matmul(ctx, s3, q3, k3, false, true, scale, 0.0f);
        softmax_fwd(ctx, s3, s3, mask);
    }
    matmul(ctx, o3, s3, v3, false, false, 1.0f, 0.0f);
    if (y.data != nullptr) {
        if (y.shape != Shape{b, t, h * hd}) detail::fatal("attention_fwd", "y must be [B, T, H·hd]");
        permute_merge(ctx.stream, y, y_heads);  // [B,H,T,hd] -> [B,T,H*hd], one launch
    }
}

void attention_fwd_packed(const RunCtx& ctx, Tensor& y, Tensor& scores, const Tensor& qkv, int64_t n_head,
                          MaskSpec mask) noexcept {
    if (ctx.backend != KernelBackend::Naive) detail::fatal("attention_fwd", "no fused variant implemented yet");
    for (const Tensor* t : std::initializer_list<const Tensor*>{&y, &scores, &qkv})
        if (!t->valid()) detail::fatal("attention_fwd_packed", "invalid tensor (null data)");
    if (qkv.shape.rank != 3 || y.shape.rank != 3 || scores.shape.rank != 4)
        detail::fatal("attention_fwd_packed", "expected qkv [B,T,3A], y [B,T,A], scores [B,H,T,T]");
    const int64_t b = qkv.shape[0], t = qkv.shape[1], a3 = qkv.shape[2], h = n_head;
    if (h <= 0 || a3 % (3 * h) != 0) detail::fatal("attention_fwd_packed", "qkv must be [B, T, 3·H·hd]");
    const int64_t a = a3 / 3, hd = a / h;
    if (y.shape != Shape{b, t, a}) detail::fatal("attention_fwd_packed", "y must be [B, T, H·hd]");
    if (scores.shape != Shape{b, h, t, t}) detail::fatal("attention_fwd_packed", "scores must be [B, H, T, T]");
    if (y.dtype != qkv.dtype || scores.dtype != qkv.dtype) detail::fatal("attention_fwd_packed", "dtype mismatch");
    const size_t es = dtype_size(qkv.dtype);
    const char* base = static_cast<const char*>(qkv.data);
    // S[b,h] = alpha Q[b,h] K[b,h]^T: operands are [T, hd] views with row pitch 3A inside qkv
    llmt_b200_gemm_desc d{};
    d.m = t; d.n = t; d.k = hd; d.batch = b * h; d.batch_inner = h;
    d.lda = a3; d.ldb = a3; d.ldc = t;
    d.stride_a = hd; d.stride_b = hd; d.stride_c = t * t;
    d.stride_a_outer = t * a3; d.stride_b_outer = t * a3; d.stride_c_outer = h * t * t;
    d.trans_a = 0; d.trans_b = 1;
    d.dtype_ab = d.dtype_c = static_cast<int32_t>(qkv.dtype);
    d.alpha = 1.0f / std::sqrt(static_cast<float>(hd)); d.beta = 0.0f;
    d.workspace = ctx.blas_workspace; d.workspace_bytes = ctx.blas_workspace_bytes;
    if (!fused_scores_softmax(ctx, d, scores.data, base, base + a * es, mask, "attention_fwd_packed")) {
        if (llmt_b200_gemm(&d, scores.data, base, base + a * es, ctx.stream) != LLMT_B200_OK)
            detail::fatal("attention_fwd_packed", "%s", llmt_b200_last_error());
        Tensor s3 = scores;
        s3.shape = Shape{b * h, t, t};
        softmax_fwd(ctx, s3, s3, mask);
    }
    // O[b,h] = P[b,h] V[b,h], written into columns h*hd .. of y's token rows
    llmt_b200_gemm_desc o{};
    o.m = t; o.n = hd; o.k = t; o.batch = b * h; o.batch_inner = h;
    o.lda = t; o.ldb = a3; o.ldc = a;
    o.stride_a = t * t; o.stride_b = hd; o.stride_c = hd;
    o.stride_a_outer = h * t * t; o.stride_b_outer = t * a3; o.stride_c_outer = t * a;
    o.trans_a = 0; o.trans_b = 0;
    o.dtype_ab = o.dtype_c = static_cast<int32_t>(qkv.dtype);
    o.alpha = 1.0f; o.beta = 0.0f;
    o.workspace = ctx.blas_workspace; o.workspace_bytes = ctx.blas_workspace_bytes;
    if (llmt_b200_gemm(&o, y.data, scores.data, base + 2 * a * es, ctx.stream) != LLMT_B200_OK)
        detail::fatal("attention_fwd_packed", "%s", llmt_b200_last_error());
}

void permute_split(cudaStream_t s, Tensor& q, Tensor& k, Tensor& v, const Tensor& qkv, int64_t n_head) noexcept {
    for (const Tensor* t : std::initializer_list<const Tensor*>{&q, &k, &v, &qkv})
        if (!t->valid()) detail::fatal("permute_split", "invalid tensor (null data)");
    if (qkv.shape.rank != 3 || q.shape.rank != 4) detail::fatal("permute_split", "expected qkv [B,T,3A] and q/k/v [B,H,T,hd]");
    if (k.shape != q.shape || v.shape != q.shape) detail::fatal("permute_split", "q/k/v must share one [B,H,T,hd] shape");
    if (q.dtype != qkv.dtype || k.dtype != qkv.dtype || v.dtype != qkv.dtype) detail::fatal("permute_split", "dtype mismatch");
    const int64_t b = q.shape[0], h = q.shape[1], t = q.shape[2], hd = q.shape[3];
    if (h != n_head || qkv.shape != Shape{b, t, 3 * h * hd}) detail::fatal("permute_split", "qkv must be [B, T, 3·H·hd]");
    const int st = llmt_b200_head_split(q.data, k.data, v.data, qkv.data, b, h, t, hd, static_cast<int32_t>(qkv.dtype), s);
    if (st != LLMT_B200_OK) detail::fatal("permute_split", "%s", llmt_b200_last_error());
}

void permute_merge(cudaStream_t s, Tensor& y, const Tensor& x) noexcept {
    if (!y.valid() || !x.valid()) detail::fatal("permute_merge", "invalid tensor (null data)");
    if (x.shape.rank != 4 || y.shape.rank != 3) detail::fatal("permute_merge", "expected x [B,H,T,hd] and y [B,T,A]");
    const int64_t b = x.shape[0], h = x.shape[1], t = x.shape[2], hd = x.shape[3];
    if (y.shape != Shape{b, t, h * hd}) detail::fatal("permute_merge", "y must be [B, T, H·hd]");
    if (y.dtype != x.dtype) detail::fatal("permute_merge", "dtype mismatch");
    const int st = llmt_b200_head_merge(y.data, x.data, b, h, t, hd, static_cast<int32_t>(x.dtype), s);
    if (st != LLMT_B200_OK) detail::fatal("permute_merge", "%s", llmt_b200_last_error());
}

void attention_bwd(const RunCtx& ctx, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& dscores,
                   const Tensor& d_y_heads, const Tensor& probs, const Tensor& q, const Tensor& k,
                   const Tensor& v) noexcept {
    attention_bwd(ctx, dq, dk, dv, dscores, d_y_heads, probs, q, k, v, nullptr, MaskSpec{MaskKind::None});
}

void attention_bwd(const RunCtx& ctx, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& dscores,
                   const Tensor& d_y_heads, const Tensor& probs, const Tensor& q, const Tensor& k,
                   const Tensor& v, const Tensor* y_heads, MaskSpec mask) noexcept {
    for (const Tensor* t :
         std::initializer_list<const Tensor*>{&dq, &dk, &dv, &dscores, &d_y_heads, &probs, &q, &k, &v}) {
        if (!t->valid()) detail::fatal("attention_bwd", "invalid tensor (null data)");
        if (t->shape.rank != 4) detail::fatal("attention_bwd", "expected rank-4 head tensors");
    }
    if (y_heads != nullptr && (!y_heads->valid() || y_heads->shape != d_y_heads.shape || y_heads->dtype != d_y_heads.dtype))
        detail::fatal("attention_bwd", "y_heads must match d_y_heads");
    const float scale = 1.0f / std::sqrt(static_cast<float>(q.shape[3]));
    Tensor dq3 = fold(dq), dk3 = fold(dk), dv3 = fold(dv), ds3 = fold(dscores);
    const Tensor do3 = fold(d_y_heads), p3 = fold(probs), q3 = fold(q), k3 = fold(k), v3 = fold(v);
    matmul(ctx, dv3, p3, do3, true, false, 1.0f, 0.0f);   // dV = P^T dO
    // dS = P * (dP - D), D = rowsum(dP * P) = rowsum(dO * O).  With O at hand and bf16 tensors D is
    // a row-wise dot product of two [.., hd] tensors and dS leaves the dP = dO V^T launch directly;
    // D lives at the head of the context's workspace (the launch needs no workspace of its own
    // for operands TMA can address: the case below checks that).
    bool fused = false;
    if (y_heads != nullptr && do3.dtype == DType::BF16 && v3.dtype == DType::BF16 && p3.dtype == ds3.dtype &&
        ctx.blas_workspace != nullptr) {
        const int64_t bh = p3.shape[0], t = p3.shape[1], tk = p3.shape[2], hd = do3.shape[2];
        const size_t d_bytes = (static_cast<size_t>(bh * t) * sizeof(float) + 255) / 256 * 256;
        llmt_b200_gemm_desc g{};
        g.m = t; g.n = tk; g.k = hd; g.batch = bh;
        g.lda = hd; g.ldb = hd; g.ldc = tk;
        g.stride_a = t * hd; g.stride_b = tk * hd; g.stride_c = t * tk;
        g.trans_a = 0; g.trans_b = 1;
        g.dtype_ab = LLMT_B200_BF16; g.dtype_c = static_cast<int32_t>(ds3.dtype);
        g.alpha = 1.0f; g.beta = 0.0f;
        const uint64_t need = llmt_b200_gemm_workspace_bytes_for(&g, do3.data, v3.data);
        if (d_bytes + need <= ctx.blas_workspace_bytes) {
            float* dvec = static_cast<float*>(ctx.blas_workspace);
            g.workspace = static_cast<char*>(ctx.blas_workspace) + d_bytes;
            g.workspace_bytes = ctx.blas_workspace_bytes - d_bytes;
            const Tensor o3 = fold(*y_heads);
            if (llmt_b200_rowdot(dvec, do3.data, o3.data, bh * t, hd, hd, hd, LLMT_B200_BF16, ctx.stream) != LLMT_B200_OK ||
                llmt_b200_gemm_softmax_bwd(&g, ds3.data, do3.data, v3.data, p3.data, dvec,
                                           mask.kind == MaskKind::Causal, ctx.stream) != LLMT_B200_OK)
                detail::fatal("attention_bwd", "%s", llmt_b200_last_error());
            fused = true;
        }
    }
    if (!fused) {
        matmul(ctx, ds3, do3, v3, false, true, 1.0f, 0.0f);   // dP = dO V^T
        const int st = llmt_b200_softmax_bwd(ds3.data, p3.data, ds3.data, p3.shape[0] * p3.shape[1],
                                             p3.shape[2], static_cast<int32_t>(p3.dtype), ctx.stream);
        if (st != LLMT_B200_OK) detail::fatal("attention_bwd", "%s", llmt_b200_last_error());
    }
    matmul(ctx, dq3, ds3, k3, false, false, scale, 0.0f);  // dQ = a dS K
    matmul(ctx, dk3, ds3, q3, true, false, scale, 0.0f);   // dK = a dS^T Q
}

}  // namespace llmt::kernels
