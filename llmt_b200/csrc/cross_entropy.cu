// Cross-entropy forward, the consumer of the LM-head logits (llmt
// include/llmt/kernels/cross_entropy.h:13-39, src/kernels/cross_entropy.cu:26-77):
//   lse[r]  = log sum_v exp(logits[r, v])
//   nll[r]  = mask[r] * (lse[r] - logits[r, targets[r]])
//   loss    = sum_r nll[r] / sum_r mask[r]
// in two forms.  From logits in memory: one warp per row, ONE pass (running maximum and
// rescaled running sum per lane, combined across the warp in a fixed tree).  From the LM-head
// GEMM itself: the GEMM's epilogue leaves, per row and per half tile, the maximum and the sum of
// exponentials of the columns it produced plus the target's logit (see the LSE epilogue of the
// grouped GEMM kernel), and `ce_from_stats_kernel` combines them, so the [rows, vocab] logits
// never have to be written or read.  The mean is one block's fixed-order tree: same bits on
// every run.
#include <cuda_bf16.h>

#include "common.h"

namespace llmt_b200 {

namespace {

constexpr int kRowsPerBlock = 8;    // one warp per row
constexpr int kMeanThreads = 256;

// (m, s) := the pair for the union of two column sets: maximum, and sum of exp(x - maximum).
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
    const float mx = fmaxf(m, m2);
    // an empty set carries (-inf, 0): its term must vanish instead of producing inf - inf
    const float a = m == -INFINITY ? 0.0f : s * __expf(m - mx);
    const float b = m2 == -INFINITY ? 0.0f : s2 * __expf(m2 - mx);
    m = mx;
    s = a + b;
}

__device__ __forceinline__ void lse_warp_combine(float& m, float& s) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        lse_merge(m, s, m2, s2);
    }
}

__global__ void __launch_bounds__(kRowsPerBlock * 32)
ce_rows_kernel(float* row_nll, const float* logits, const int32_t* targets, const float* mask, int64_t rows,
               int64_t v, int64_t ld) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = logits + row * ld;
    float m = -INFINITY, s = 0.0f;
    for (int64_t i = lane; i < v; i += 32) {
        const float xi = x[i];
        if (xi > m) {
            s = s * expf(m - xi) + 1.0f;  // exp(-inf) = 0 covers the first element
            m = xi;
        } else {
            s += expf(xi - m);
        }
    }
    lse_warp_combine(m, s);
    if (lane == 0) row_nll[row] = mask[row] * (m + logf(s) - x[targets[row]]);
}

// stats: [parts][rows] pairs (maximum, sum of exponentials) of disjoint column sets of every
// row, tgt: [rows] the target's logit.  Parts are combined in ascending order.
__global__ void __launch_bounds__(kRowsPerBlock * 32)
ce_from_stats_kernel(float* row_nll, const float2* stats, const float* tgt, const float* mask, int64_t rows, int parts) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float m = -INFINITY, s = 0.0f;
    for (int p = lane; p < parts; p += 32) {
        const float2 t = stats[static_cast<int64_t>(p) * rows + row];
        lse_merge(m, s, t.x, t.y);
    }
    lse_warp_combine(m, s);
    if (lane == 0) row_nll[row] = mask[row] * (m + logf(s) - tgt[row]);
}

__global__ void __launch_bounds__(kMeanThreads)
ce_mean_kernel(float* loss, const float* row_nll, const float* mask, int64_t rows) {
    __shared__ float sh_n[kMeanThreads];
    __shared__ float sh_m[kMeanThreads];
    float n = 0.0f, w = 0.0f;
    for (int64_t i = threadIdx.x; i < rows; i += kMeanThreads) {
        n += row_nll[i];
        w += mask[i];
    }
    sh_n[threadIdx.x] = n;
    sh_m[threadIdx.x] = w;
    __syncthreads();
    for (int o = kMeanThreads / 2; o > 0; o >>= 1) {
        if (static_cast<int>(threadIdx.x) < o) {
            sh_n[threadIdx.x] += sh_n[threadIdx.x + o];
            sh_m[threadIdx.x] += sh_m[threadIdx.x + o];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) loss[0] = sh_n[0] / sh_m[0];
}

// The rows' log-sum-exp from the per-part pairs (the first pass of a softmax fused around a GEMM).
// One thread per row, parts in ascending order: neighbouring threads read neighbouring pairs.
__global__ void __launch_bounds__(256)
lse_from_stats_kernel(float* lse, const float2* stats, int64_t rows, int parts) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (row >= rows) return;
    float m = -INFINITY, s = 0.0f;
    for (int p = 0; p < parts; ++p) {
        const float2 t = stats[static_cast<int64_t>(p) * rows + row];
        lse_merge(m, s, t.x, t.y);
    }
    lse[row] = m + logf(s);
}

// sum of the mask in one block's fixed-order tree (the denominator of the mean).
__global__ void __launch_bounds__(kMeanThreads)
mask_sum_kernel(float* out, const float* mask, int64_t rows) {
    __shared__ float sh[kMeanThreads];
    float w = 0.0f;
    for (int64_t i = threadIdx.x; i < rows; i += kMeanThreads) w += mask[i];
    sh[threadIdx.x] = w;
    __syncthreads();
    for (int o = kMeanThreads / 2; o > 0; o >>= 1) {
        if (static_cast<int>(threadIdx.x) < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] = sh[0];
}

// Per row what the dLogits epilogue of the LM-head product needs: (log-sum-exp, weight), the
// weight being dloss * mask[r] / sum(mask).  The log-sum-exp comes from the per-part pairs of a
// statistics pass, or from `lse_in` where the forward pass kept it.
__global__ void __launch_bounds__(256)
ce_grad_rows_kernel(float2* out, const float2* stats, const float* lse_in, const float* mask, const float* mask_sum,
                    float dloss, int64_t rows, int parts) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (row >= rows) return;
    float lse;
    if (lse_in != nullptr) {
        lse = lse_in[row];
    } else {
        float m = -INFINITY, s = 0.0f;
        for (int p = 0; p < parts; ++p) {
            const float2 t = stats[static_cast<int64_t>(p) * rows + row];
            lse_merge(m, s, t.x, t.y);
        }
        lse = m + logf(s);
    }
    out[row] = make_float2(lse, dloss * mask[row] / mask_sum[0]);
}

// llmt's planned cross_entropy_bwd (docs/TODO.md:216-217): dlogits = (softmax - onehot) * mask / sum(mask),
// written in place of the logits if the caller passes the same tensor.  One warp per row: the
// log-sum-exp in one pass, the gradient in a second (every element is read and written by the same lane).
__global__ void __launch_bounds__(kRowsPerBlock * 32)
ce_bwd_rows_kernel(float* dlogits, const float* logits, const int32_t* targets, const float* mask,
                   float dloss, int64_t rows, int64_t v, int64_t ld_in, int64_t ld_out) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float* x = logits + row * ld_in;
    float* y = dlogits + row * ld_out;
    // 16-byte accesses where both rows allow them; the ragged end by single values
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0u;
    const int64_t v4 = vec ? v / 4 : 0;
    float m = -INFINITY, s = 0.0f;
    auto take = [&](float xi) {
        if (xi > m) {
            s = s * __expf(m - xi) + 1.0f;
            m = xi;
        } else {
            s += __expf(xi - m);
        }
    };
    for (int64_t i = lane; i < v4; i += 32) {
        const float4 q = reinterpret_cast<const float4*>(x)[i];
        const float mx = fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w));
        if (mx > m) {
            s *= __expf(m - mx);  // exp(-inf) = 0 covers the first group
            m = mx;
        }
        s += (__expf(q.x - m) + __expf(q.y - m)) + (__expf(q.z - m) + __expf(q.w - m));
    }
    for (int64_t i = 4 * v4 + lane; i < v; i += 32) take(x[i]);
    lse_warp_combine(m, s);
    const float lse = m + logf(s);
    // The mask's sum by every warp for itself, in one fixed order: no scratch, same bits everywhere.
    float w = 0.0f;
    for (int64_t i = lane; i < rows; i += 32) w += mask[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    const float g = dloss * mask[row] / w;
    const int64_t t = targets[row];
    for (int64_t i = lane; i < v4; i += 32) {
        float4 q = reinterpret_cast<const float4*>(x)[i];
        q.x = __expf(q.x - lse) * g; q.y = __expf(q.y - lse) * g; q.z = __expf(q.z - lse) * g; q.w = __expf(q.w - lse) * g;
        if ((t >> 2) == i) {
            const int e = static_cast<int>(t & 3);
            if (e == 0) q.x -= g; else if (e == 1) q.y -= g; else if (e == 2) q.z -= g; else q.w -= g;
        }
        reinterpret_cast<float4*>(y)[i] = q;
    }
    for (int64_t i = 4 * v4 + lane; i < v; i += 32) y[i] = (__expf(x[i] - lse) - (i == t ? 1.0f : 0.0f)) * g;
}

// out[r] = sum_j x[r, j] * y[r, j] in fp32, lanes striding the row, a fixed tree across the warp.
template <typename T>
__global__ void __launch_bounds__(kRowsPerBlock * 32)
rowdot_kernel(float* out, const T* x, const T* y, int64_t rows, int64_t cols, int64_t ldx, int64_t ldy) {
    const int64_t row = static_cast<int64_t>(blockIdx.x) * kRowsPerBlock + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const T* xr = x + row * ldx;
    const T* yr = y + row * ldy;
    float acc = 0.0f;
    for (int64_t j = lane; j < cols; j += 32) acc = fmaf(static_cast<float>(xr[j]), static_cast<float>(yr[j]), acc);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) out[row] = acc;
}

unsigned row_blocks(int64_t rows) { return static_cast<unsigned>((rows + kRowsPerBlock - 1) / kRowsPerBlock); }

}  // namespace

cudaError_t launch_cross_entropy_fwd(float* loss, float* row_nll, const float* logits, const int32_t* targets,
                                     const float* mask, int64_t rows, int64_t v, int64_t ld, cudaStream_t stream) {
    ce_rows_kernel<<<row_blocks(rows), kRowsPerBlock * 32, 0, stream>>>(row_nll, logits, targets, mask, rows, v, ld);
    ce_mean_kernel<<<1, kMeanThreads, 0, stream>>>(loss, row_nll, mask, rows);
    count_launch(2);
    return cudaGetLastError();
}

cudaError_t launch_cross_entropy_from_stats(float* loss, float* row_nll, const void* stats, const float* tgt,
                                            const float* mask, int64_t rows, int parts, cudaStream_t stream) {
    ce_from_stats_kernel<<<row_blocks(rows), kRowsPerBlock * 32, 0, stream>>>(
        row_nll, static_cast<const float2*>(stats), tgt, mask, rows, parts);
    ce_mean_kernel<<<1, kMeanThreads, 0, stream>>>(loss, row_nll, mask, rows);
    count_launch(2);
    return cudaGetLastError();
}

cudaError_t launch_cross_entropy_bwd(float* dlogits, const float* logits, const int32_t* targets, const float* mask,
                                     float dloss, int64_t rows, int64_t v, int64_t ld_in, int64_t ld_out,
                                     cudaStream_t stream) {
    ce_bwd_rows_kernel<<<row_blocks(rows), kRowsPerBlock * 32, 0, stream>>>(dlogits, logits, targets, mask, dloss,
                                                                            rows, v, ld_in, ld_out);
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_ce_grad_rows(void* out, const void* stats, const float* lse_in, const float* mask, float* mask_sum,
                                float dloss, int64_t rows, int parts, cudaStream_t stream) {
    mask_sum_kernel<<<1, kMeanThreads, 0, stream>>>(mask_sum, mask, rows);
    ce_grad_rows_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, stream>>>(
        static_cast<float2*>(out), static_cast<const float2*>(stats), lse_in, mask, mask_sum, dloss, rows, parts);
    count_launch(2);
    return cudaGetLastError();
}

cudaError_t launch_lse_from_stats(float* lse, const void* stats, int64_t rows, int parts, cudaStream_t stream) {
    lse_from_stats_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, stream>>>(lse, static_cast<const float2*>(stats), rows, parts);
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_rowdot(float* out, const void* x, const void* y, int64_t rows, int64_t cols, int64_t ldx,
                          int64_t ldy, int is_bf16, cudaStream_t stream) {
    if (is_bf16)
        rowdot_kernel<__nv_bfloat16><<<row_blocks(rows), kRowsPerBlock * 32, 0, stream>>>(
            out, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y), rows, cols, ldx, ldy);
    else
        rowdot_kernel<float><<<row_blocks(rows), kRowsPerBlock * 32, 0, stream>>>(
            out, static_cast<const float*>(x), static_cast<const float*>(y), rows, cols, ldx, ldy);
    count_launch(1);
    return cudaGetLastError();
}

}  // namespace llmt_b200
