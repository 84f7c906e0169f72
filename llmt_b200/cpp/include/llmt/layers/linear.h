// Linear projection with weight W[out, in] (llmt include/llmt/layers/linear.h:24-36):
//   forward   y[M,out] = x[M,in] W^T (+ bias)
//   backward  dx[M,in] = dy[M,out] W ;  dW += dy^T x ;  (dbias += sum over rows of dy)
// llmt's layer is bias-free; with bias == false this class behaves exactly like it.
#pragma once

#include <cstdint>
#include <string>

#include "llmt/core/run_ctx.h"
#include "llmt/core/types.h"
#include "llmt/model/param_store.h"

namespace llmt {

class Linear {
   public:
    Linear(ParamStore& ps, std::string name, int64_t in_features, int64_t out_features, Role role,
           bool bias = false) noexcept;

    void forward(const RunCtx& ctx, Tensor& y, const Tensor& x) const noexcept;
    // Forward with tanh-GELU fused into the GEMM epilogue (after the bias).
    void forward_gelu(const RunCtx& ctx, Tensor& y, const Tensor& x) const noexcept;
    // The same, also storing the value the GELU sees in `pre` (y's shape and dtype; bf16 path).
    void forward_gelu(const RunCtx& ctx, Tensor& y, Tensor& pre, const Tensor& x) const noexcept;
    void backward(const RunCtx& ctx, Tensor& dx, const Tensor& dy, const Tensor& x) const noexcept;
    // Backward of a layer whose INPUT came out of a GELU: dx is the gradient before that GELU,
    // dx = (dy W) * gelu'(pre), in the same launch as dW += dy^T x (bf16 path).
    void backward_through_gelu(const RunCtx& ctx, Tensor& dx, const Tensor& dy, const Tensor& x,
                               const Tensor& pre) const noexcept;

    const Param& param() const noexcept { return weight_; }
    const Param* bias_param() const noexcept { return bias_; }

   private:
    Param& weight_;
    Param* bias_ = nullptr;
};

}  // namespace llmt
