// GELU MLP  y = gelu_tanh(x Wup^T) Wdown^T  (llmt include/llmt/layers/mlp.h:26-37).
// h is caller-provided [M, d_ff] scratch and holds the post-GELU activation on
// return; y may alias x; h may alias neither.  GELU runs in the up-projection's
// epilogue instead of a separate pass over h.
#pragma once

#include <string>

#include "llmt/layers/linear.h"

namespace llmt {

class MLP {
   public:
    MLP(ParamStore& ps, const std::string& name, int64_t d_model, int64_t d_ff,
        bool bias = false) noexcept;
    void forward(const RunCtx& ctx, Tensor& y, Tensor& h, const Tensor& x) const noexcept;
    // Training forward: also keeps pre = x Wup^T (+ b), the value the GELU saw (h's shape and dtype).
    void forward(const RunCtx& ctx, Tensor& y, Tensor& h, Tensor& pre, const Tensor& x) const noexcept;
    // Backward (llmt docs/TODO.md:223-224, planned): two launches.  d_pre [M, d_ff] is scratch:
    //   d_pre = (dy Wdown) * gelu'(pre),  dWdown += dy^T h (+ dbias)      one grouped launch
    //   dx = d_pre Wup,  dWup += d_pre^T x (+ dbias)                      one grouped launch
    void backward(const RunCtx& ctx, Tensor& dx, Tensor& d_pre, const Tensor& dy, const Tensor& x,
                  const Tensor& h, const Tensor& pre) const noexcept;
    const Param& up() const noexcept { return up_.param(); }
    const Param& down() const noexcept { return down_.param(); }
    const Linear& up_layer() const noexcept { return up_; }
    const Linear& down_layer() const noexcept { return down_; }

   private:
    Linear up_, down_;
};

}  // namespace llmt
