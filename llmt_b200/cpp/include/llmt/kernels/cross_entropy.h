// Cross-entropy forward from raw logits, the consumer of the LM-head GEMM (llmt
// include/llmt/kernels/cross_entropy.h:13-39: same name, arguments and abort messages):
//   row_nll[b][t] = mask[b][t] * (log sum_v exp(logits[b][t][v]) - logits[b][t][targets[b][t]])
//   loss          = sum row_nll / sum mask          (fixed-order sums: same bits on every run)
// logits [B, T, V] fp32, targets [B, T] I32, mask [B, T] fp32, row_nll [B, T] fp32, loss [1] fp32.
//
// lm_head_cross_entropy_fwd (extension, no counterpart in llmt) computes the same from the LM-head
// product itself, logits = x * w^T (+ bias) with x [B, T, C] and w [V, C] bf16: the GEMM's epilogue
// keeps the row statistics, so the [B, T, V] logits need not exist (`logits` null) or are written on
// the way (`logits` fp32 [B, T, V]).  ctx.blas_workspace must hold
// lm_head_cross_entropy_workspace_bytes(...) bytes.
#pragma once

#include "llmt/core/run_ctx.h"
#include "llmt/core/types.h"

namespace llmt::kernels {

void cross_entropy_fwd(const RunCtx& ctx, Tensor& loss, Tensor& row_nll, const Tensor& logits,
                       const Tensor& targets, const Tensor& mask) noexcept;

size_t lm_head_cross_entropy_workspace_bytes(const Tensor& x, const Tensor& w) noexcept;
void lm_head_cross_entropy_fwd(const RunCtx& ctx, Tensor& loss, Tensor& row_nll, Tensor* logits, const Tensor& x,
                               const Tensor& w, const Tensor* bias, const Tensor& targets,
                               const Tensor& mask) noexcept;

// The backward pass (llmt docs/TODO.md:216-217, planned as cross_entropy_bwd, not written there):
//   dlogits = (softmax(logits) - onehot(targets)) * dloss * mask / sum(mask)
// cross_entropy_bwd: from fp32 logits in memory; dlogits may be the logits tensor itself (in place).
// lm_head_cross_entropy_bwd: from the LM-head product made again, so that no logits need exist;
// dlogits [B, T, V] bf16 (the operand of the LM head's dX and dW products) or fp32.  stats_valid:
// ctx.blas_workspace still holds what lm_head_cross_entropy_fwd left there for the same x and w.
void cross_entropy_bwd(const RunCtx& ctx, Tensor& dlogits, const Tensor& logits, const Tensor& targets,
                       const Tensor& mask, float dloss = 1.0f) noexcept;
void lm_head_cross_entropy_bwd(const RunCtx& ctx, Tensor& dlogits, const Tensor& x, const Tensor& w, const Tensor* bias,
                               const Tensor& targets, const Tensor& mask, float dloss = 1.0f,
                               bool stats_valid = false) noexcept;

}  // namespace llmt::kernels
