// Linear and MLP over kernels::matmul (llmt src/layers/linear.cpp:12-30,
// src/layers/mlp.cpp:10-18) with the optional bias / fused-GELU extensions.
#include <utility>

#include "llmt/kernels/matmul.h"
#include "llmt/layers/linear.h"
#include "llmt/layers/mlp.h"

namespace llmt {

Linear::Linear(ParamStore& ps, std::string name, int64_t in_features, int64_t out_features, Role role,
               bool bias) noexcept
    : weight_(ps.add(name, {out_features, in_features}, role)),
      bias_(bias ? &ps.add(name + ".bias", {out_features}, Role::Bias) : nullptr) {}

void Linear::forward(const RunCtx& ctx, Tensor& y, const Tensor& x) const noexcept {
    kernels::Epilogue epi;
    if (bias_ != nullptr) epi.bias = &bias_->weight;
    kernels::matmul_ex(ctx, y, x, weight_.weight, false, true, 1.0f, 0.0f, epi);  // y = x W^T (+ b)
}

void Linear::forward_gelu(const RunCtx& ctx, Tensor& y, const Tensor& x) const noexcept {
    kernels::Epilogue epi;
    if (bias_ != nullptr) epi.bias = &bias_->weight;
    epi.gelu = true;
    kernels::matmul_ex(ctx, y, x, weight_.weight, false, true, 1.0f, 0.0f, epi);
}

void Linear::forward_gelu(const RunCtx& ctx, Tensor& y, Tensor& pre, const Tensor& x) const noexcept {
    kernels::Epilogue epi;
    if (bias_ != nullptr) epi.bias = &bias_->weight;
    epi.gelu = true;
    epi.save_pre = &pre;
    kernels::matmul_ex(ctx, y, x, weight_.weight, false, true, 1.0f, 0.0f, epi);
}

void Linear::backward_through_gelu(const RunCtx& ctx, Tensor& dx, const Tensor& dy, const Tensor& x,
                                   const Tensor& pre) const noexcept {
    kernels::MatmulCall calls[2];
    calls[0].c = &dx; calls[0].a = &dy; calls[0].b = &weight_.weight;            // dx = (dy W) * gelu'(pre)
    calls[0].epi.gelu_bwd_of = &pre;
    calls[1].c = &weight_.grad; calls[1].a = &dy; calls[1].b = &x;                // dW += dy^T x
    calls[1].trans_a = true; calls[1].beta = 1.0f;
    if (bias_ != nullptr) calls[1].epi.dbias = &bias_->grad;
    kernels::matmul_grouped(ctx, calls, 2);
}

void Linear::backward(const RunCtx& ctx, Tensor& dx, const Tensor& dy, const Tensor& x) const noexcept {
    // dx = dy W and dW += dy^T x depend on nothing but dy: one grouped launch on the bf16
    // path (two plain matmul calls, as in llmt, on the fp32 path).
    kernels::MatmulCall calls[2];
    calls[0].c = &dx; calls[0].a = &dy; calls[0].b = &weight_.weight;            // dx = dy W
    calls[1].c = &weight_.grad; calls[1].a = &dy; calls[1].b = &x;                // dW += dy^T x
    calls[1].trans_a = true; calls[1].beta = 1.0f;
    // The bias gradient accumulates like dW (beta = 1), on both paths.
    if (bias_ != nullptr) calls[1].epi.dbias = &bias_->grad;
    kernels::matmul_grouped(ctx, calls, 2);
}

MLP::MLP(ParamStore& ps, const std::string& name, int64_t d_model, int64_t d_ff, bool bias) noexcept
    : up_(ps, name + ".up", d_model, d_ff, Role::Matrix, bias),
      down_(ps, name + ".down", d_ff, d_model, Role::ResidualProj, bias) {}

void MLP::forward(const RunCtx& ctx, Tensor& y, Tensor& h, const Tensor& x) const noexcept {
    up_.forward_gelu(ctx, h, x);  // h = gelu(x Wup^T): GELU in the GEMM epilogue, h ends post-GELU
    down_.forward(ctx, y, h);     // y = h Wdown^T
}

void MLP::forward(const RunCtx& ctx, Tensor& y, Tensor& h, Tensor& pre, const Tensor& x) const noexcept {
    up_.forward_gelu(ctx, h, pre, x);  // one launch, two results: pre and h = gelu(pre)
    down_.forward(ctx, y, h);
}

void MLP::backward(const RunCtx& ctx, Tensor& dx, Tensor& d_pre, const Tensor& dy, const Tensor& x,
                   const Tensor& h, const Tensor& pre) const noexcept {
    down_.backward_through_gelu(ctx, d_pre, dy, h, pre);
    up_.backward(ctx, dx, d_pre, x);
}

}  // namespace llmt
