// Naive attention forward as a composition of the batched GEMMs and the masked
// softmax (llmt include/llmt/kernels/attention.h, src/kernels/attention.cpp:34-64).
#pragma once

#include "llmt/core/run_ctx.h"
#include "llmt/core/types.h"
#include "llmt/kernels/mask.h"

namespace llmt::kernels {

// q,k,v,y_heads [B,H,T,hd]; scores [B,H,T,T] (holds the probabilities on
// return).  The head merge into [B,T,H*hd] token rows is a pure copy outside
// the GEMM path; pass y with data == nullptr to skip it.
void attention_fwd(const RunCtx& ctx, Tensor& y, Tensor& scores, Tensor& y_heads, const Tensor& q,
                   const Tensor& k, const Tensor& v, MaskSpec mask) noexcept;

// Backward products of the same composition (llmt docs/TODO.md:226-228):
//   dV = P^T dO,  dP = dO V^T,  dS = P*(dP - rowsum(dP*P)),  dQ = a dS K,  dK = a dS^T Q.
// probs is the P left in `scores` by attention_fwd; dscores is [B,H,T,T] scratch.
void attention_bwd(const RunCtx& ctx, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& dscores,
                   const Tensor& d_y_heads, const Tensor& probs, const Tensor& q, const Tensor& k,
                   const Tensor& v) noexcept;

void softmax_fwd(const RunCtx& ctx, Tensor& y, const Tensor& x, MaskSpec mask) noexcept;

}  // namespace llmt::kernels
