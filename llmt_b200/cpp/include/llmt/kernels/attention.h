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
// bf16 tensors take the softmax inside the scores GEMM (two launches over the same tiles: row
// statistics, then exp(s - lse) stored as the probabilities; the scores themselves are never
// stored) when ctx.blas_workspace holds the statistics; otherwise, and for fp32, llmt's
// composition GEMM -> softmax_fwd in place.
void attention_fwd(const RunCtx& ctx, Tensor& y, Tensor& scores, Tensor& y_heads, const Tensor& q,
                   const Tensor& k, const Tensor& v, MaskSpec mask) noexcept;

// Backward products of the same composition (llmt docs/TODO.md:226-228):
//   dV = P^T dO,  dP = dO V^T,  dS = P*(dP - rowsum(dP*P)),  dQ = a dS K,  dK = a dS^T Q.
// probs is the P left in `scores` by attention_fwd; dscores is [B,H,T,T] scratch.
void attention_bwd(const RunCtx& ctx, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& dscores,
                   const Tensor& d_y_heads, const Tensor& probs, const Tensor& q, const Tensor& k,
                   const Tensor& v) noexcept;

// The same with the forward pass's pre-merge output y_heads [B,H,T,hd] (what attention_fwd left)
// and the mask of the forward pass: for bf16 tensors D = rowsum(dO * O) replaces rowsum(dP * P)
// and dS leaves the launch that makes dP, so dP is never stored and P is read once (for dS) instead
// of twice.  `mask` lets the launch skip the arithmetic where P is zero by construction.
void attention_bwd(const RunCtx& ctx, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& dscores,
                   const Tensor& d_y_heads, const Tensor& probs, const Tensor& q, const Tensor& k,
                   const Tensor& v, const Tensor* y_heads, MaskSpec mask) noexcept;

void softmax_fwd(const RunCtx& ctx, Tensor& y, const Tensor& x, MaskSpec mask) noexcept;

// The same forward pass with the head split and merge folded into the GEMMs' strides:
//   qkv [B, T, 3*H*hd]  the output of the fused QKV projection (per token: Q | K | V parts)
//   scores [B, H, T, T] holds the probabilities on return, as in attention_fwd
//   y [B, T, H*hd]      token rows, ready for the output projection
// S = alpha Q K^T reads Q and K straight out of qkv (row pitch 3*H*hd, one head every hd
// elements), O = P V reads V the same way and writes each head's [T, hd] block into its
// columns of y.  Replaces permute_split -> attention_fwd -> permute_merge of llmt
// (include/llmt/kernels/permute.h:13-46, src/kernels/attention.cpp:54-63): no q/k/v/y_heads
// tensors, no copy kernels.  hd * sizeof(element) must be a multiple of 16 bytes.
void attention_fwd_packed(const RunCtx& ctx, Tensor& y, Tensor& scores, const Tensor& qkv, int64_t n_head,
                          MaskSpec mask) noexcept;

}  // namespace llmt::kernels
