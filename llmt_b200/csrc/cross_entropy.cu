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
