// Head split / merge (llmt include/llmt/kernels/permute.h:21-46): pure data movement between
// token rows [B, T, ...] and per-head blocks [B, H, T, hd].
//   permute_split: q|k|v[b, h, t, d] = qkv[b, t, part*A + h*hd + d],  A = H*hd
//   permute_merge: y[b, t, h*hd + d] = x[b, h, t, d]
// Outputs must not alias inputs.
#pragma once

#include <cuda_runtime.h>

#include "llmt/core/types.h"

namespace llmt::kernels {

void permute_split(cudaStream_t s, Tensor& q, Tensor& k, Tensor& v, const Tensor& qkv, int64_t n_head) noexcept;
void permute_merge(cudaStream_t s, Tensor& y, const Tensor& x) noexcept;

}  // namespace llmt::kernels
