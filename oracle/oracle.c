/*
 * TEST INFRASTRUCTURE, NOT PRODUCT.  CPU restatement of the arithmetic that
 * llmt's matrix-multiply path performs, used only as the checker in tests/,
 * in the smoke check and as the timed CPU leg of the benchmark.  Nothing in
 * the shipped library links, loads or calls this file.
 *
 * What it restates (paths are relative to the llmt source tree):
 *   - kernels::matmul semantics,        include/llmt/kernels/matmul.h:12-24
 *     and the shape derivation in       src/kernels/matmul.cpp:175-214
 *   - Linear forward / backward,        src/layers/linear.cpp:16-30
 *   - MLP forward,                      src/layers/mlp.cpp:14-18
 *   - tanh-GELU formula,                src/kernels/gelu.cu:19-27
 *   - attention GEMM composition,       src/kernels/attention.cpp:54-62
 *   - masked row softmax,               src/kernels/softmax.cu:25-51
 *   - attention backward products,      docs/TODO.md:226-228
 *
 * llmt has no host GEMM of its own; its CPU oracle is PyTorch-on-CPU frozen
 * into golden files (tools/gen_golden.py).  This file is pinned against those
 * golden files by tests/test_oracle_goldens.py.
 *
 * All GEMMs here accumulate in double.  Inputs are float (bf16 values are
 * passed widened to float, which is exact).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Element (i, j) of op(X) where X is a row-major buffer with row pitch ld. */
static inline double op_at(const float* x, int64_t ld, int trans, int64_t i, int64_t j) {
    return trans ? (double)x[j * ld + i] : (double)x[i * ld + j];
}

/*
 * C[b] = alpha * op(A[b]) * op(B[b]) + beta * C[b]        (matmul.h:12-22)
 * op(A) is [m,k], op(B) is [k,n]; buffers are row-major with explicit pitches
 * so that padded layouts can be checked too.  batch strides are in elements.
 * The product is accumulated in double and written to a double C.
 */
ORACLE_API void oracle_gemm_f64(int64_t m, int64_t n, int64_t k, int64_t batch,
                                const float* a, int64_t lda, int64_t stride_a, int trans_a,
                                const float* b, int64_t ldb, int64_t stride_b, int trans_b,
                                double* c, int64_t ldc, int64_t stride_c,
                                double alpha, double beta) {
    for (int64_t bi = 0; bi < batch; ++bi) {
        const float* ab = a + bi * stride_a;
        const float* bb = b + bi * stride_b;
        double* cb = c + bi * stride_c;
        /* Pack op(A) rows and op(B) columns contiguously so the inner loop
         * streams; this is only a speed matter, the sum order is k ascending. */
        double* ap = (double*)malloc(sizeof(double) * (size_t)m * (size_t)k);
        double* bp = (double*)malloc(sizeof(double) * (size_t)n * (size_t)k);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < m; ++i)
            for (int64_t p = 0; p < k; ++p) ap[i * k + p] = op_at(ab, lda, trans_a, i, p);
#pragma omp parallel for schedule(static)
        for (int64_t j = 0; j < n; ++j)
            for (int64_t p = 0; p < k; ++p) bp[j * k + p] = op_at(bb, ldb, trans_b, p, j);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < m; ++i) {
            const double* ar = ap + i * k;
            for (int64_t j = 0; j < n; ++j) {
                const double* bc = bp + j * k;
                double acc = 0.0;
                for (int64_t p = 0; p < k; ++p) acc += ar[p] * bc[p];
                double prev = (beta == 0.0) ? 0.0 : beta * cb[i * ldc + j];
                cb[i * ldc + j] = alpha * acc + prev;
            }
        }
        free(ap);
        free(bp);
    }
}

/*
 * The same contraction in plain fp32 arithmetic with a blocked loop nest: the
 * timed CPU baseline ("port").  It is what a straightforward multi-threaded
 * host implementation of kernels::matmul costs; only NT / NN / TN / TT via
 * packing, fp32 accumulate.
 */
ORACLE_API void oracle_gemm_f32(int64_t m, int64_t n, int64_t k,
                                const float* a, int64_t lda, int trans_a,
                                const float* b, int64_t ldb, int trans_b,
                                float* c, int64_t ldc, float alpha, float beta) {
    /* pack B as [n][k] so both operands stream along k */
    float* bp = (float*)malloc(sizeof(float) * (size_t)n * (size_t)k);
    float* ap = NULL;
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j)
        for (int64_t p = 0; p < k; ++p)
            bp[j * k + p] = trans_b ? b[j * ldb + p] : b[p * ldb + j];
    if (trans_a) {
        ap = (float*)malloc(sizeof(float) * (size_t)m * (size_t)k);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < m; ++i)
            for (int64_t p = 0; p < k; ++p) ap[i * k + p] = a[p * lda + i];
    }
    const int64_t a_ld = trans_a ? k : lda;
    const float* a_use = trans_a ? ap : a;
    enum { BI = 4, BJ = 4 };
#pragma omp parallel for schedule(static)
    for (int64_t i0 = 0; i0 < m; i0 += BI) {
        for (int64_t j0 = 0; j0 < n; j0 += BJ) {
            float acc[BI][BJ];
            memset(acc, 0, sizeof acc);
            const int64_t ie = (i0 + BI < m) ? BI : (m - i0);
            const int64_t je = (j0 + BJ < n) ? BJ : (n - j0);
            if (ie == BI && je == BJ) {
                const float* a0 = a_use + (i0 + 0) * a_ld;
                const float* a1 = a_use + (i0 + 1) * a_ld;
                const float* a2 = a_use + (i0 + 2) * a_ld;
                const float* a3 = a_use + (i0 + 3) * a_ld;
                const float* b0 = bp + (j0 + 0) * k;
                const float* b1 = bp + (j0 + 1) * k;
                const float* b2 = bp + (j0 + 2) * k;
                const float* b3 = bp + (j0 + 3) * k;
                for (int64_t p = 0; p < k; ++p) {
                    const float x0 = a0[p], x1 = a1[p], x2 = a2[p], x3 = a3[p];
                    const float y0 = b0[p], y1 = b1[p], y2 = b2[p], y3 = b3[p];
                    acc[0][0] += x0 * y0; acc[0][1] += x0 * y1; acc[0][2] += x0 * y2; acc[0][3] += x0 * y3;
                    acc[1][0] += x1 * y0; acc[1][1] += x1 * y1; acc[1][2] += x1 * y2; acc[1][3] += x1 * y3;
                    acc[2][0] += x2 * y0; acc[2][1] += x2 * y1; acc[2][2] += x2 * y2; acc[2][3] += x2 * y3;
                    acc[3][0] += x3 * y0; acc[3][1] += x3 * y1; acc[3][2] += x3 * y2; acc[3][3] += x3 * y3;
                }
            } else {
                for (int64_t i = 0; i < ie; ++i)
                    for (int64_t j = 0; j < je; ++j) {
                        float s = 0.f;
                        for (int64_t p = 0; p < k; ++p)
                            s += a_use[(i0 + i) * a_ld + p] * bp[(j0 + j) * k + p];
                        acc[i][j] = s;
                    }
            }
            for (int64_t i = 0; i < ie; ++i)
                for (int64_t j = 0; j < je; ++j) {
                    float* dst = c + (i0 + i) * ldc + (j0 + j);
                    *dst = alpha * acc[i][j] + (beta == 0.f ? 0.f : beta * *dst);
                }
        }
    }
    free(bp);
    free(ap);
}

/* tanh-GELU, gelu.cu:23-26, evaluated in double. */
ORACLE_API double oracle_gelu_f64(double v) {
    const double k0 = 0.7978845608028654, k1 = 0.044715;
    return 0.5 * v * (1.0 + tanh(k0 * (v + k1 * v * v * v)));
}

/* The same expression in the arithmetic the llmt kernel uses (float, tanhf). */
ORACLE_API float oracle_gelu_f32(float v) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * v * (1.0f + tanhf(k0 * (v + k1 * v * v * v)));
}

/*
 * Fused-epilogue extension, defined as the composition
 *   matmul (alpha, beta) -> + bias[j] broadcast over rows -> tanh-GELU
 * applied in place on a double matrix.  flags: bit0 = bias, bit1 = gelu.
 */
ORACLE_API void oracle_epilogue_f64(double* c, int64_t m, int64_t n, int64_t ldc,
                                    const float* bias, int flags) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            double v = c[i * ldc + j];
            if (flags & 1) v += (double)bias[j];
            if (flags & 2) v = oracle_gelu_f64(v);
            c[i * ldc + j] = v;
        }
}

/*
 * dbias extension: out[i] = dbias_beta * out[i] + sum_p op(A)[i, p].
 * For the Linear dW call op(A) = dy^T, so i runs over output features and the
 * sum runs over tokens (linear.cpp:27-29 gives the operand roles).
 */
ORACLE_API void oracle_rowsum_f64(int64_t m, int64_t k, const float* a, int64_t lda, int trans_a,
                                  double* out, double out_beta) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i) {
        double s = 0.0;
        for (int64_t p = 0; p < k; ++p) s += op_at(a, lda, trans_a, i, p);
        out[i] = (out_beta == 0.0 ? 0.0 : out_beta * out[i]) + s;
    }
}

/*
 * Row softmax with llmt's masking rule (softmax.cu:33-50): row r of a
 * [rows, tk] matrix belongs to query q = r % tq; under the causal mask only
 * columns < q+1 take part and the rest are written as exact zeros.
 */
ORACLE_API void oracle_softmax_f64(const double* x, double* y, int64_t rows, int64_t tq,
                                   int64_t tk, int causal) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const int64_t q = r % tq;
        const int64_t limit = causal ? q + 1 : tk;
        const double* xr = x + r * tk;
        double* yr = y + r * tk;
        double mx = -INFINITY;
        for (int64_t i = 0; i < limit; ++i) mx = xr[i] > mx ? xr[i] : mx;
        double sum = 0.0;
        for (int64_t i = 0; i < limit; ++i) sum += exp(xr[i] - mx);
        for (int64_t i = 0; i < tk; ++i) yr[i] = i < limit ? exp(xr[i] - mx) / sum : 0.0;
    }
}

/* dS = P * (dP - rowsum(dP * P)) per row (docs/TODO.md:227). */
ORACLE_API void oracle_softmax_bwd_f64(const double* p, const double* dp, double* ds,
                                       int64_t rows, int64_t tk) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const double* pr = p + r * tk;
        const double* dr = dp + r * tk;
        double dot = 0.0;
        for (int64_t i = 0; i < tk; ++i) dot += pr[i] * dr[i];
        for (int64_t i = 0; i < tk; ++i) ds[r * tk + i] = pr[i] * (dr[i] - dot);
    }
}

/* Round-to-nearest-even float -> bf16 bit pattern (NaN kept quiet). */
ORACLE_API uint16_t oracle_f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    const uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

ORACLE_API void oracle_round_bf16(const float* in, float* out, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint32_t u = ((uint32_t)oracle_f32_to_bf16_bits(in[i])) << 16;
        memcpy(&out[i], &u, 4);
    }
}
