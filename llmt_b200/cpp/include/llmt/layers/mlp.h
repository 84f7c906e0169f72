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
    const Param& up() const noexcept { return up_.param(); }
    const Param& down() const noexcept { return down_.param(); }
    const Linear& up_layer() const noexcept { return up_; }
    const Linear& down_layer() const noexcept { return down_; }

   private:
    Linear up_, down_;
};

}  // namespace llmt
