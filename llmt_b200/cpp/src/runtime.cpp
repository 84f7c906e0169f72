// Arena, Device and ParamStore: the small runtime llmt's layers expect around
// the GEMM path (llmt src/core/arena.cu, src/core/device.cu,
// src/model/param_store.cpp), without any cuBLASLt state.
#include <cuda_runtime.h>

#include <utility>

#include "llmt/core/arena.h"
#include "llmt/core/device.h"
#include "llmt/core/error.h"
#include "llmt/kernels/algo_cache.h"
#include "llmt/model/param_store.h"

namespace llmt {

// ------------------------------------------------------------------- Arena ---

Arena::Arena(size_t capacity, const char* name) noexcept : capacity_(capacity), name_(name) {
    CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&base_), capacity_ ? capacity_ : kAlign));
}

Arena::~Arena() {
    if (base_ != nullptr) cudaFree(base_);
}

void* Arena::alloc_bytes(size_t bytes) noexcept {
    const size_t start = (used_ + kAlign - 1) & ~(kAlign - 1);
    if (start + bytes > capacity_)
        detail::fatal("arena", "'%s' exhausted: request %zu B at offset %zu, capacity %zu B", name_,
                      bytes, start, capacity_);
    used_ = start + bytes;
    peak_ = used_ > peak_ ? used_ : peak_;
    return base_ + start;
}

Tensor Arena::alloc(const Shape& shape, DType dtype) noexcept {
    Tensor t;
    t.dtype = dtype;
    t.shape = shape;
    t.data = alloc_bytes(t.bytes());
    return t;
}

// ------------------------------------------------------------------ Device ---

Device::Device(int index) noexcept : index_(index) {
    CUDA_CHECK(cudaSetDevice(index_));
    cudaDeviceProp p{};
    CUDA_CHECK(cudaGetDeviceProperties(&p, index_));
    props_.name = p.name;
    props_.sm_major = p.major;
    props_.sm_minor = p.minor;
    props_.sm_count = p.multiProcessorCount;
    props_.vram_bytes = p.totalGlobalMem;
    props_.l2_bytes = static_cast<size_t>(p.l2CacheSize);
    CUDA_CHECK(cudaStreamCreate(&stream_));
    CUDA_CHECK(cudaMalloc(&workspace_, kBlasWorkspaceBytes));
    cache_ = std::make_unique<kernels::AlgoCache>();
}

Device::~Device() {
    if (workspace_ != nullptr) cudaFree(workspace_);
    if (stream_ != nullptr) cudaStreamDestroy(stream_);
}

RunCtx Device::make_ctx(uint64_t seed, KernelBackend backend, PrecisionPolicy precision) const noexcept {
    RunCtx ctx;
    ctx.stream = stream_;
    ctx.blas_workspace = workspace_;
    ctx.blas_workspace_bytes = kBlasWorkspaceBytes;
    ctx.algo_cache = cache_.get();
    ctx.precision = precision;
    ctx.backend = backend;
    ctx.seed = seed;
    return ctx;
}

void Device::synchronize() const noexcept { CUDA_CHECK(cudaStreamSynchronize(stream_)); }

// -------------------------------------------------------------- ParamStore ---

Param& ParamStore::add(std::string name, const Shape& shape, Role role) noexcept {
    if (finalized()) detail::fatal("param_store", "add('%s') after finalize()", name.c_str());
    if (index_.count(name) != 0) detail::fatal("param_store", "duplicate parameter '%s'", name.c_str());
    index_[name] = params_.size();
    Param p;
    p.name = std::move(name);
    p.shape = shape;
    p.role = role;
    params_.push_back(std::move(p));
    return params_.back();
}

void ParamStore::finalize() noexcept {
    if (finalized()) detail::fatal("param_store", "finalize() called twice");
    const DType dts[2] = {dtypes_.weight, dtypes_.grad};
    auto padded = [](size_t b) { return (b + Arena::kAlign - 1) / Arena::kAlign * Arena::kAlign; };
    for (int k = 0; k < 2; ++k) {
        span_bytes_[k] = 0;
        for (const Param& p : params_)
            span_bytes_[k] += padded(static_cast<size_t>(p.shape.numel()) * dtype_size(dts[k]));
    }
    mem_.emplace(span_bytes_[0] + span_bytes_[1] + 2 * Arena::kAlign, "params");
    for (int k = 0; k < 2; ++k) {
        base_[k] = static_cast<char*>(mem_->alloc_bytes(span_bytes_[k] ? span_bytes_[k] : 1));
        CUDA_CHECK(cudaMemset(base_[k], 0, span_bytes_[k]));
        size_t off = 0;
        for (Param& p : params_) {
            Tensor& t = k == 0 ? p.weight : p.grad;
            t.data = base_[k] + off;
            t.dtype = dts[k];
            t.shape = p.shape;
            off += padded(t.bytes());
        }
    }
}

Param& ParamStore::at(const std::string& name) noexcept {
    auto it = index_.find(name);
    if (it == index_.end()) detail::fatal("param_store", "unknown parameter '%s'", name.c_str());
    return params_[it->second];
}

Tensor ParamStore::flat(StateKind k) const noexcept {
    if (!finalized()) detail::fatal("param_store", "flat() before finalize()");
    const int i = k == StateKind::Weight ? 0 : 1;
    const DType dt = i == 0 ? dtypes_.weight : dtypes_.grad;
    Tensor t;
    t.data = base_[i];
    t.dtype = dt;
    t.shape = Shape{static_cast<int64_t>(span_bytes_[i] / dtype_size(dt))};
    return t;
}

void ParamStore::zero_grad(cudaStream_t s) noexcept {
    CUDA_CHECK(cudaMemsetAsync(base_[1], 0, span_bytes_[1], s));
}

}  // namespace llmt
