// TEST / BASELINE INFRASTRUCTURE, NOT PRODUCT.
//
// C entry points over the UNMODIFIED llmt library, compiled from the llmt
// sources where they lie (see oracle/Makefile, target `ref`).  The functions
// here only marshal device pointers into llmt's own Tensor/RunCtx types and
// call llmt's public API: kernels::matmul (include/llmt/kernels/matmul.h:23),
// kernels::gelu_fwd, kernels::softmax_fwd, Linear::forward/backward
// (include/llmt/layers/linear.h:29-30).  llmt's matmul path is cuBLASLt in
// strict fp32 (src/kernels/matmul.cpp:72-77,185-188), so everything is fp32.
//
// Used by the parity tests (llmt itself as a second checker on the GPU) and by
// the benchmark's reference arm.  Nothing in llmt_b200 links this.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <memory>

#include "llmt/core/arena.h"
#include "llmt/core/device.h"
#include "llmt/core/error.h"
#include "llmt/kernels/gelu.h"
#include "llmt/kernels/matmul.h"
#include "llmt/kernels/softmax.h"
#include "llmt/layers/linear.h"
#include "llmt/model/param_store.h"

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {
struct Handle {
    std::unique_ptr<llmt::Device> dev;
    llmt::RunCtx ctx;
};
llmt::Tensor view(void* p, int rank, const int64_t* dims) {
    llmt::Tensor t;
    t.data = p;
    t.dtype = llmt::DType::FP32;
    t.shape.rank = rank;
    for (int i = 0; i < rank; ++i) t.shape.d[i] = dims[i];
    return t;
}
}  // namespace

REF_API void* ref_create(int device) {
    auto* h = new Handle;
    h->dev = std::make_unique<llmt::Device>(device);
    h->ctx = h->dev->make_ctx(0, llmt::KernelBackend::Naive, llmt::PrecisionPolicy::fp32());
    return h;
}

REF_API void ref_destroy(void* hv) { delete static_cast<Handle*>(hv); }

// Runs on the caller's stream when `stream` is non-null, else on llmt's Device stream.
REF_API void ref_matmul(void* hv, void* c, const void* a, const void* b, int rank,
                        const int64_t* c_dims, const int64_t* a_dims, const int64_t* b_dims,
                        int trans_a, int trans_b, float alpha, float beta, void* stream) {
    auto* h = static_cast<Handle*>(hv);
    llmt::RunCtx ctx = h->ctx;
    if (stream) ctx.stream = static_cast<cudaStream_t>(stream);
    llmt::Tensor tc = view(c, rank, c_dims);
    const llmt::Tensor ta = view(const_cast<void*>(a), rank, a_dims);
    const llmt::Tensor tb = view(const_cast<void*>(b), rank, b_dims);
    llmt::kernels::matmul(ctx, tc, ta, tb, trans_a != 0, trans_b != 0, alpha, beta);
}

REF_API void ref_gelu(void* hv, void* y, const void* x, int64_t n, void* stream) {
    auto* h = static_cast<Handle*>(hv);
    const int64_t dims[1] = {n};
    llmt::Tensor ty = view(y, 1, dims);
    const llmt::Tensor tx = view(const_cast<void*>(x), 1, dims);
    llmt::kernels::gelu_fwd(stream ? static_cast<cudaStream_t>(stream) : h->ctx.stream, ty, tx);
}

REF_API void ref_softmax(void* hv, void* y, const void* x, int64_t batch, int64_t tq, int64_t tk,
                         int causal, void* stream) {
    auto* h = static_cast<Handle*>(hv);
    llmt::RunCtx ctx = h->ctx;
    if (stream) ctx.stream = static_cast<cudaStream_t>(stream);
    const int64_t dims[3] = {batch, tq, tk};
    llmt::Tensor ty = view(y, 3, dims);
    const llmt::Tensor tx = view(const_cast<void*>(x), 3, dims);
    llmt::kernels::softmax_fwd(ctx, ty, tx,
                               llmt::kernels::MaskSpec{causal ? llmt::kernels::MaskKind::Causal
                                                              : llmt::kernels::MaskKind::None});
}

// One Linear layer through llmt's own class: y = x W^T, dx = dy W, dW += dy^T x
// (twice when `backward_calls` is 2, to show the accumulation contract).
REF_API void ref_linear(void* hv, int64_t m, int64_t in_f, int64_t out_f, const void* w,
                        const void* x, const void* dy, void* y, void* dx, void* dw_out,
                        int backward_calls) {
    auto* h = static_cast<Handle*>(hv);
    llmt::ParamStore ps(llmt::StateDtypes::uniform(llmt::DType::FP32));
    const llmt::Linear lin(ps, "w", in_f, out_f, llmt::Role::Matrix);
    ps.finalize();
    CUDA_CHECK(cudaMemcpyAsync(lin.param().weight.data, w, sizeof(float) * in_f * out_f,
                               cudaMemcpyDeviceToDevice, h->ctx.stream));
    const int64_t xd[2] = {m, in_f}, yd[2] = {m, out_f};
    const llmt::Tensor tx = view(const_cast<void*>(x), 2, xd);
    const llmt::Tensor tdy = view(const_cast<void*>(dy), 2, yd);
    llmt::Tensor ty = view(y, 2, yd), tdx = view(dx, 2, xd);
    lin.forward(h->ctx, ty, tx);
    for (int i = 0; i < backward_calls; ++i) lin.backward(h->ctx, tdx, tdy, tx);
    CUDA_CHECK(cudaMemcpyAsync(dw_out, lin.param().grad.data, sizeof(float) * in_f * out_f,
                               cudaMemcpyDeviceToDevice, h->ctx.stream));
    h->dev->synchronize();
}

REF_API void ref_synchronize(void* hv) { static_cast<Handle*>(hv)->dev->synchronize(); }
