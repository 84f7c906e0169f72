// Arena, Device and ParamStore: the small runtime llmt's layers expect around
// the GEMM path (llmt src/core/arena.cu, src/core/device.cu,
// src/model/param_store.cpp), without any cuBLASLt state.
#include <cuda_runtime.h>

#include <utility>

#include "llmt/core/arena.h"
#include "llmt/core/device.h"
#include "llmt/core/error.h"
#include "llmt/kernels/algo_cache.h"
#include "llmt/dist/peer_exchange.h"
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
    param_numel_ += shape.numel();
    params_.push_back(std::move(p));
    return params_.back();
}

void ParamStore::alias(const std::string& alias_name, const std::string& target) noexcept {
    if (finalized()) detail::fatal("param_store", "alias('%s') after finalize()", alias_name.c_str());
    if (index_.count(alias_name) != 0) detail::fatal("param_store", "duplicate parameter '%s'", alias_name.c_str());
    auto it = index_.find(target);
    if (it == index_.end()) detail::fatal("param_store", "alias target '%s' is unknown", target.c_str());
    index_[alias_name] = it->second;  // one Param, two names; no storage is added
}

namespace {
size_t padded_bytes(size_t b) { return (b + Arena::kAlign - 1) / Arena::kAlign * Arena::kAlign; }
}  // namespace

size_t ParamStore::span_bytes_of(StateKind k) const noexcept {
    size_t total = 0;
    for (const Param& p : params_) total += padded_bytes(static_cast<size_t>(p.shape.numel()) * dtype_size(dtypes_[k]));
    return total;
}

void ParamStore::carve(void* external_grad, size_t external_bytes) noexcept {
    if (finalized()) detail::fatal("param_store", "finalize() called twice");
    constexpr int kGrad = static_cast<int>(StateKind::Grad);
    size_t own = 0;
    for (int k = 0; k < kNumStateKinds; ++k) {
        span_bytes_[k] = span_bytes_of(static_cast<StateKind>(k));
        if (!(k == kGrad && external_grad != nullptr)) own += span_bytes_[k] + Arena::kAlign;
    }
    if (external_grad != nullptr) {
        if (external_bytes < span_bytes_[kGrad])
            detail::fatal("param_store", "external gradient span too small: %zu B given, %zu B needed",
                          external_bytes, span_bytes_[kGrad]);
        if (reinterpret_cast<uintptr_t>(external_grad) % Arena::kAlign != 0)
            detail::fatal("param_store", "external gradient span is not %zu-byte aligned", Arena::kAlign);
    }
    mem_.emplace(own + Arena::kAlign, "params");
    for (int k = 0; k < kNumStateKinds; ++k) {
        const StateKind kind = static_cast<StateKind>(k);
        base_[k] = (k == kGrad && external_grad != nullptr)
                       ? static_cast<char*>(external_grad)
                       : static_cast<char*>(mem_->alloc_bytes(span_bytes_[k] ? span_bytes_[k] : 1));
        CUDA_CHECK(cudaMemset(base_[k], 0, span_bytes_[k]));  // padding stays zero: inert under sums
        size_t off = 0;
        for (Param& p : params_) {
            Tensor& t = p.state(kind);
            t.data = base_[k] + off;
            t.dtype = dtypes_[kind];
            t.shape = p.shape;
            off += padded_bytes(t.bytes());
        }
    }
}

void ParamStore::finalize() noexcept { carve(nullptr, 0); }

void ParamStore::finalize(void* grad_span, size_t bytes) noexcept {
    if (grad_span == nullptr) detail::fatal("param_store", "finalize(span): null span");
    carve(grad_span, bytes);
}

Param& ParamStore::at(const std::string& name) noexcept {
    auto it = index_.find(name);
    if (it == index_.end()) detail::fatal("param_store", "unknown parameter '%s'", name.c_str());
    return params_[it->second];
}

const Param& ParamStore::at(const std::string& name) const noexcept {
    auto it = index_.find(name);
    if (it == index_.end()) detail::fatal("param_store", "unknown parameter '%s'", name.c_str());
    return params_[it->second];
}

Tensor ParamStore::flat(StateKind k) const noexcept {
    if (!finalized()) detail::fatal("param_store", "flat() before finalize()");
    const int i = static_cast<int>(k);
    Tensor t;
    t.data = base_[i];
    t.dtype = dtypes_[k];
    t.shape = Shape{static_cast<int64_t>(span_bytes_[i] / dtype_size(dtypes_[k]))};
    return t;
}

void ParamStore::zero_grad(cudaStream_t s) noexcept {
    constexpr int kGrad = static_cast<int>(StateKind::Grad);
    CUDA_CHECK(cudaMemsetAsync(base_[kGrad], 0, span_bytes_[kGrad], s));
}

void ParamStore::allreduce_grads(dist::PeerExchange& ex, cudaStream_t stream) noexcept {
    constexpr int kGrad = static_cast<int>(StateKind::Grad);
    if (!finalized()) detail::fatal("param_store", "allreduce_grads() before finalize()");
    if (dtypes_[StateKind::Grad] != DType::FP32) detail::fatal("param_store", "allreduce_grads: gradients must be fp32");
    if (base_[kGrad] != reinterpret_cast<char*>(ex.span()))
        detail::fatal("param_store", "allreduce_grads: the gradient span does not live in this exchange "
                                     "(finalize(ex.span(), ex.span_bytes()))");
    ex.allreduce(0, static_cast<int64_t>(span_bytes_[kGrad] / sizeof(float)), stream);
}

}  // namespace llmt
