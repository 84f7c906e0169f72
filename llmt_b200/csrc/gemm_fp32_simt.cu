// Strict-fp32 GEMM: fp32 storage, fp32 FMA arithmetic, no tensor cores.
//
// This is the path that must agree with llmt's fp32 golden tensors at
// rtol 1e-5 (llmt runs cuBLASLt with CUBLAS_COMPUTE_32F and refuses TF32,
// src/kernels/matmul.cpp:33-36,72-77); tcgen05 has no full-precision fp32 MMA,
// so this is a CUDA-core kernel.  64x64 output tile per 256-thread CTA,
// 4x4 outputs per thread, k ascending -> the sum order is fixed, results are
// bitwise reproducible.
#include <cuda_bf16.h>

#include <initializer_list>

#include "common.h"

namespace llmt_b200 {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256)
fp32_gemm_kernel(const Fp32GemmParams p) {
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];

    const int64_t b = blockIdx.z;
    // batch item b of a plain batch, or item (b % inner) of group (b / inner) of a two-level one
    const int64_t bi = p.batch_inner > 0 ? b % p.batch_inner : b;
    const int64_t bo = p.batch_inner > 0 ? b / p.batch_inner : 0;
    const float* A = p.a + bi * p.stride_a + bo * p.stride_a_outer;
    const float* B = p.b + bi * p.stride_b + bo * p.stride_b_outer;
    float* C = p.c + bi * p.stride_c + bo * p.stride_c_outer;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * TM;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * TN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < p.k; k0 += TK) {
        // 64x16 elements of op(A) and of op(B): 4 elements per thread each.
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = threadIdx.x + e * 256;
            int mi, ki;
            if (p.trans_a) { mi = idx % TM; ki = idx / TM; }   // A stored [k, m]: m contiguous
            else           { ki = idx % TK; mi = idx / TK; }   // A stored [m, k]: k contiguous
            const int64_t gm = m0 + mi, gk = k0 + ki;
            float v = 0.0f;
            if (gm < p.m && gk < p.k) v = p.trans_a ? A[gk * p.lda + gm] : A[gm * p.lda + gk];
            As[ki][mi] = v;
            int ni, kj;
            if (p.trans_b) { kj = idx % TK; ni = idx / TK; }   // B stored [n, k]: k contiguous
            else           { ni = idx % TN; kj = idx / TN; }   // B stored [k, n]: n contiguous
            const int64_t gn = n0 + ni, gk2 = k0 + kj;
            float w = 0.0f;
            if (gn < p.n && gk2 < p.k) w = p.trans_b ? B[gn * p.ldb + gk2] : B[gk2 * p.ldb + gn];
            Bs[kj][ni] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], bb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bb[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t gm = m0 + ty * 4 + i;
        if (gm >= p.m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t gn = n0 + tx * 4 + j;
            if (gn >= p.n) continue;
            float v = p.alpha * acc[i][j];
            float* dst = C + gm * p.ldc + gn;
            if (p.beta != 0.0f) v += p.beta * *dst;
            if (p.epi_flags & kEpiBias)
                v += p.bias_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[gn])
                                    : static_cast<const float*>(p.bias)[gn];
            if (p.epi_flags & kEpiGelu) v = gelu_tanh_precise(v);
            *dst = v;
        }
    }
}

// dbias[i] = dbias_beta * dbias[i] + sum_p op(A)[i, p] on the strict-fp32 path: one thread per
// i, p ascending, so the order of the additions is fixed.  A parity path, like the GEMM above.
__global__ void fp32_rowsum_kernel(const Fp32GemmParams p, float* dbias, float dbias_beta) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= p.m) return;
    float acc = 0.0f;
    if (p.trans_a) {
        for (int64_t q = 0; q < p.k; ++q) acc += p.a[q * p.lda + i];   // A stored [k, m]
    } else {
        for (int64_t q = 0; q < p.k; ++q) acc += p.a[i * p.lda + q];   // A stored [m, k]
    }
    dbias[i] = (dbias_beta != 0.0f ? dbias_beta * dbias[i] : 0.0f) + acc;
}

// ---- masked row softmax and its backward (fp32 arithmetic; one warp per row) ------------------

// Element access that converts at the edges: arithmetic is always fp32.
template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float get(const float* p, int64_t i) { return p[i]; }
    static __device__ __forceinline__ void put(float* p, int64_t i, float v) { p[i] = v; }
};
template <> struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ float get(const __nv_bfloat16* p, int64_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ void put(__nv_bfloat16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
};

// (running maximum, sum of exp(x - maximum)) of a set of scores; two such pairs merge exactly.
struct MaxSum {
    float mx, sum;
};
__device__ __forceinline__ MaxSum merge(MaxSum a, MaxSum b) {
    const float mx = fmaxf(a.mx, b.mx);
    if (mx == -INFINITY) return MaxSum{mx, 0.0f};
    return MaxSum{mx, a.sum * expf(a.mx - mx) + b.sum * expf(b.mx - mx)};
}

// Row softmax with llmt's masking rule (src/kernels/softmax.cu:33-50: under the causal mask
// only columns <= r % tq take part; the others are written as exact zeros; y may be x).
// One warp per row, ONE pass over the scores to find (max, sum) - each lane keeps a running
// pair that is rescaled whenever its maximum grows, the 32 pairs merge in a butterfly - and
// one pass to write, instead of llmt's three passes.
template <typename T>
__global__ void softmax_rows_kernel(T* y, const T* x, int64_t rows, int64_t tq, int64_t tk, int causal) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    const int64_t live = causal ? (r % tq) + 1 : tk;  // columns that take part
    const T* in = x + r * tk;
    T* out = y + r * tk;
    MaxSum ms{-INFINITY, 0.0f};
    for (int64_t c = lane; c < live; c += 32) {
        const float v = Elem<T>::get(in, c);
        if (v > ms.mx) {
            ms.sum = ms.sum * expf(ms.mx - v) + 1.0f;  // exp(-inf) = 0 on the first element
            ms.mx = v;
        } else {
            ms.sum += expf(v - ms.mx);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        MaxSum other;
        other.mx = __shfl_xor_sync(0xffffffffu, ms.mx, o);
        other.sum = __shfl_xor_sync(0xffffffffu, ms.sum, o);
        ms = merge(ms, other);
    }
    const float scale = 1.0f / ms.sum;
    for (int64_t c = lane; c < tk; c += 32)
        Elem<T>::put(out, c, c < live ? expf(Elem<T>::get(in, c) - ms.mx) * scale : 0.0f);
}

// dS = P * (dP - sum_c dP[c] P[c]) per row (llmt docs/TODO.md:227).  ds may be dp.
template <typename T>
__global__ void softmax_rows_bwd_kernel(T* ds, const T* p, const T* dp, int64_t rows, int64_t tk) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (r >= rows) return;
    const T* pr = p + r * tk;
    const T* gr = dp + r * tk;
    T* out = ds + r * tk;
    float dot = 0.0f;
    for (int64_t c = lane; c < tk; c += 32) dot = fmaf(Elem<T>::get(pr, c), Elem<T>::get(gr, c), dot);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    for (int64_t c = lane; c < tk; c += 32)
        Elem<T>::put(out, c, Elem<T>::get(pr, c) * (Elem<T>::get(gr, c) - dot));
}

// Copies a row-major bf16 matrix (any pitch, any 2-byte alignment) into a buffer whose base is
// 16-byte aligned and whose pitch is a multiple of 8 elements, so that TMA can address it.
// One thread per 8 output elements (one 16-byte store): the source elements come from the
// five aligned 32-bit words that cover them, shifted by 16 bits when the source row starts on
// an odd element.  Columns beyond `cols` are written as zeros.
__global__ void repack_bf16_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ src, int64_t rows,
                                   int64_t cols, int64_t ld_src, int64_t ld_dst, int64_t batch,
                                   int64_t stride_src, int64_t stride_dst) {
    const int64_t groups_per_row = ld_dst / 8;
    const int64_t total = batch * rows * groups_per_row;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t g = i % groups_per_row;
        const int64_t r = (i / groups_per_row) % rows;
        const int64_t b = i / (groups_per_row * rows);
        const int64_t c0 = g * 8;
        const uint16_t* s = src + b * stride_src + r * ld_src + c0;
        uint32_t out[4];
        if (c0 + 8 <= cols) {
            const uintptr_t addr = reinterpret_cast<uintptr_t>(s);
            const uint32_t* w = reinterpret_cast<const uint32_t*>(addr & ~static_cast<uintptr_t>(3));
            if ((addr & 2u) == 0u) {
#pragma unroll
                for (int j = 0; j < 4; ++j) out[j] = w[j];
            } else {
                uint32_t v[5];
#pragma unroll
                for (int j = 0; j < 5; ++j) v[j] = w[j];   // the first and last halves belong to neighbours
#pragma unroll
                for (int j = 0; j < 4; ++j) out[j] = __funnelshift_r(v[j], v[j + 1], 16);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo = c0 + 2 * j < cols ? s[2 * j] : 0u;
                const uint32_t hi = c0 + 2 * j + 1 < cols ? s[2 * j + 1] : 0u;
                out[j] = lo | (hi << 16);
            }
        }
        *reinterpret_cast<uint4*>(dst + b * stride_dst + r * ld_dst + c0) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

// Head split / merge as copies (llmt include/llmt/kernels/permute.h:21-46).  The GEMMs can read
// and write the per-head layout through strides, so these are only needed where a caller wants
// the re-shelved tensor itself.  One thread moves `vec` consecutive elements of one head's row
// (hd is a multiple of vec): 16 bytes when the pointers and hd allow it, else one element.
//   merge: y[b, t, h*hd + d] = x[b, h, t, d]
//   split: out[part][b, h, t, d] = qkv[b, t, part*A + h*hd + d],  A = H*hd, part = 0..parts-1
template <typename V>
__global__ void head_merge_kernel(V* __restrict__ y, const V* __restrict__ x, int64_t B, int64_t H, int64_t T,
                                  int64_t hdv) {
    const int64_t total = B * H * T * hdv;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        // i runs over the OUTPUT [B, T, H, hdv]: consecutive threads write consecutive vectors
        const int64_t d = i % hdv, h = (i / hdv) % H, t = (i / (hdv * H)) % T, b = i / (hdv * H * T);
        y[i] = x[((b * H + h) * T + t) * hdv + d];
    }
}

template <typename V>
__global__ void head_split_kernel(V* __restrict__ q, V* __restrict__ k, V* __restrict__ v, const V* __restrict__ qkv,
                                  int64_t B, int64_t H, int64_t T, int64_t hdv) {
    const int64_t per_part = B * T * H * hdv;
    const int64_t total = 3 * per_part;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        // i runs over the INPUT [B, T, 3, H, hdv]: consecutive threads read consecutive vectors
        const int64_t d = i % hdv, h = (i / hdv) % H, part = (i / (hdv * H)) % 3, t = (i / (hdv * H * 3)) % T,
                      b = i / (hdv * H * 3 * T);
        V* out = part == 0 ? q : part == 1 ? k : v;
        out[((b * H + h) * T + t) * hdv + d] = qkv[i];
    }
}

// Zeroes the flat gradient span between steps (the zero_grad of llmt's ParamStore contract,
// include/llmt/model/param_store.h:142-148).  Written here rather than left to a memset so that it
// joins the stream's programmatic dependent launches: the first GEMM of the step starts its
// prologue while this still runs.
__global__ void zero_f32_kernel(float4* __restrict__ dst, int64_t n4, float* __restrict__ tail, int n_tail) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        dst[i] = z;
    if (blockIdx.x == 0 && threadIdx.x < n_tail) tail[threadIdx.x] = 0.0f;
}

}  // namespace

cudaError_t launch_zero_f32(float* dst, int64_t n, cudaStream_t stream) {
    // 16-byte aligned body, scalar head and tail
    int64_t head = 0;
    while (head < n && (reinterpret_cast<uintptr_t>(dst + head) & 15u) != 0u) ++head;
    if (head > 0) {
        cudaError_t e = cudaMemsetAsync(dst, 0, static_cast<size_t>(head) * sizeof(float), stream);
        if (e != cudaSuccess) return e;
    }
    const int64_t n4 = (n - head) / 4;
    const int n_tail = static_cast<int>((n - head) % 4);
    int64_t grid = (n4 + 255) / 256;
    if (grid > 148 * 8) grid = 148 * 8;
    if (grid < 1) grid = 1;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, zero_f32_kernel, reinterpret_cast<float4*>(dst + head), n4,
                                             dst + head + n4 * 4, n_tail);
    count_launch(1);
    return e != cudaSuccess ? e : cudaGetLastError();
}

cudaError_t launch_repack_bf16(void* dst, const void* src, int64_t rows, int64_t cols, int64_t ld_src,
                               int64_t ld_dst, int64_t batch, int64_t stride_src, int64_t stride_dst,
                               cudaStream_t stream) {
    const int64_t total = batch * rows * (ld_dst / 8);   // ld_dst is a multiple of 8
    int64_t grid = (total + 255) / 256;
    if (grid > 148 * 32) grid = 148 * 32;
    if (grid < 1) grid = 1;
    repack_bf16_kernel<<<static_cast<unsigned>(grid), 256, 0, stream>>>(
        static_cast<uint16_t*>(dst), static_cast<const uint16_t*>(src), rows, cols, ld_src, ld_dst, batch,
        stride_src, stride_dst);
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_fp32_gemm(const Fp32GemmParams& p, cudaStream_t stream) {
    dim3 grid(static_cast<unsigned>((p.n + TN - 1) / TN), static_cast<unsigned>((p.m + TM - 1) / TM),
              static_cast<unsigned>(p.batch));
    fp32_gemm_kernel<<<grid, 256, 0, stream>>>(p);
    count_launch(1);
    return cudaGetLastError();
}

namespace {
int64_t copy_grid(int64_t total) {
    int64_t grid = (total + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    return grid < 1 ? 1 : grid;
}
bool vec16_ok(std::initializer_list<const void*> ptrs, int64_t hd, int elem_bytes) {
    if ((hd * elem_bytes) % 16 != 0) return false;
    for (const void* p : ptrs)
        if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
    return true;
}
}  // namespace

cudaError_t launch_head_merge(void* y, const void* x, int64_t B, int64_t H, int64_t T, int64_t hd, int elem_bytes,
                              cudaStream_t stream) {
    if (vec16_ok({y, x}, hd, elem_bytes)) {
        const int64_t hdv = hd * elem_bytes / 16;
        head_merge_kernel<uint4><<<static_cast<unsigned>(copy_grid(B * H * T * hdv)), 256, 0, stream>>>(
            static_cast<uint4*>(y), static_cast<const uint4*>(x), B, H, T, hdv);
    } else if (elem_bytes == 4) {
        head_merge_kernel<uint32_t><<<static_cast<unsigned>(copy_grid(B * H * T * hd)), 256, 0, stream>>>(
            static_cast<uint32_t*>(y), static_cast<const uint32_t*>(x), B, H, T, hd);
    } else {
        head_merge_kernel<uint16_t><<<static_cast<unsigned>(copy_grid(B * H * T * hd)), 256, 0, stream>>>(
            static_cast<uint16_t*>(y), static_cast<const uint16_t*>(x), B, H, T, hd);
    }
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_head_split(void* q, void* k, void* v, const void* qkv, int64_t B, int64_t H, int64_t T, int64_t hd,
                              int elem_bytes, cudaStream_t stream) {
    if (vec16_ok({q, k, v, qkv}, hd, elem_bytes)) {
        const int64_t hdv = hd * elem_bytes / 16;
        head_split_kernel<uint4><<<static_cast<unsigned>(copy_grid(3 * B * H * T * hdv)), 256, 0, stream>>>(
            static_cast<uint4*>(q), static_cast<uint4*>(k), static_cast<uint4*>(v), static_cast<const uint4*>(qkv), B, H,
            T, hdv);
    } else if (elem_bytes == 4) {
        head_split_kernel<uint32_t><<<static_cast<unsigned>(copy_grid(3 * B * H * T * hd)), 256, 0, stream>>>(
            static_cast<uint32_t*>(q), static_cast<uint32_t*>(k), static_cast<uint32_t*>(v),
            static_cast<const uint32_t*>(qkv), B, H, T, hd);
    } else {
        head_split_kernel<uint16_t><<<static_cast<unsigned>(copy_grid(3 * B * H * T * hd)), 256, 0, stream>>>(
            static_cast<uint16_t*>(q), static_cast<uint16_t*>(k), static_cast<uint16_t*>(v),
            static_cast<const uint16_t*>(qkv), B, H, T, hd);
    }
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_fp32_rowsum(const Fp32GemmParams& p, float* dbias, float dbias_beta, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>((p.m + 127) / 128);
    fp32_rowsum_kernel<<<grid, 128, 0, stream>>>(p, dbias, dbias_beta);
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_softmax_fwd(void* y, const void* x, int64_t rows, int64_t tq, int64_t tk,
                               int is_bf16, int causal, cudaStream_t stream) {
    constexpr int kRowsPerBlock = 4;  // one warp per row
    const unsigned grid = static_cast<unsigned>((rows + kRowsPerBlock - 1) / kRowsPerBlock);
    if (is_bf16)
        softmax_rows_kernel<__nv_bfloat16><<<grid, kRowsPerBlock * 32, 0, stream>>>(
            static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(x), rows, tq, tk, causal);
    else
        softmax_rows_kernel<float><<<grid, kRowsPerBlock * 32, 0, stream>>>(
            static_cast<float*>(y), static_cast<const float*>(x), rows, tq, tk, causal);
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_softmax_bwd(void* ds, const void* p, const void* dp, int64_t rows, int64_t tk,
                               int is_bf16, cudaStream_t stream) {
    constexpr int kRowsPerBlock = 4;
    const unsigned grid = static_cast<unsigned>((rows + kRowsPerBlock - 1) / kRowsPerBlock);
    if (is_bf16)
        softmax_rows_bwd_kernel<__nv_bfloat16><<<grid, kRowsPerBlock * 32, 0, stream>>>(
            static_cast<__nv_bfloat16*>(ds), static_cast<const __nv_bfloat16*>(p),
            static_cast<const __nv_bfloat16*>(dp), rows, tk);
    else
        softmax_rows_bwd_kernel<float><<<grid, kRowsPerBlock * 32, 0, stream>>>(
            static_cast<float*>(ds), static_cast<const float*>(p), static_cast<const float*>(dp),
            rows, tk);
    count_launch(1);
    return cudaGetLastError();
}

}  // namespace llmt_b200
