// kernels::matmul — the GEMM seam of llmt (include/llmt/kernels/matmul.h:12-24),
// implemented over the llmt_b200 C ABI instead of cuBLASLt.
#pragma once

#include "llmt/core/run_ctx.h"
#include "llmt/core/types.h"

namespace llmt::kernels {

// C[M,N] = alpha*op(A)*op(B) + beta*C for row-major tensors; rank 2 = one GEMM,
// rank 3 = one independent GEMM per leading index.  Same contract, same abort
// messages as llmt.  dtype rules: all fp32 (strict fp32 path, needs
// ctx.precision == fp32()), or A/B bf16 with C bf16 or fp32 (tensor-core path,
// needs gemm_compute == BF16, reduce == FP32).
void matmul(const RunCtx& ctx, Tensor& c, const Tensor& a, const Tensor& b, bool trans_a,
            bool trans_b, float alpha, float beta) noexcept;

// Fused-epilogue extension.  Applied after alpha/beta:  + bias[n]  -> tanh-GELU
// -> cast.  dbias (fp32 [M]) receives  dbias_beta*dbias + row sums of op(A).
// A default-constructed Epilogue makes matmul_ex identical to matmul.
// save_pre (with gelu): the value the GELU sees is stored there too (C's shape and dtype).
// gelu_bwd_of: C = (alpha*op(A)*op(B)) * gelu'(*gelu_bwd_of), the saved pre-activation (C's shape
// and dtype): the dX product of the layer after a GELU leaves as the gradient before it.  Both
// are bf16-path only (llmt plans gelu_bwd as a kernel of its own, docs/TODO.md:223).
struct Epilogue {
    const Tensor* bias = nullptr;
    bool gelu = false;
    Tensor* dbias = nullptr;
    float dbias_beta = 1.0f;
    Tensor* save_pre = nullptr;
    const Tensor* gelu_bwd_of = nullptr;
};
void matmul_ex(const RunCtx& ctx, Tensor& c, const Tensor& a, const Tensor& b, bool trans_a,
               bool trans_b, float alpha, float beta, const Epilogue& epi) noexcept;

// Several independent products in one launch (bf16 operands only): the tiles of all of
// them share one queue on the GPU.  Used by Linear::backward for dx = dy W and
// dW += dy^T x, which llmt issues as two matmul calls (src/layers/linear.cpp:22-30).
// Falls back to one matmul_ex per call when an operand is fp32.
struct MatmulCall {
    Tensor* c = nullptr;
    const Tensor* a = nullptr;
    const Tensor* b = nullptr;
    bool trans_a = false, trans_b = false;
    float alpha = 1.0f, beta = 0.0f;
    Epilogue epi;
};
void matmul_grouped(const RunCtx& ctx, const MatmulCall* calls, int count) noexcept;

}  // namespace llmt::kernels
