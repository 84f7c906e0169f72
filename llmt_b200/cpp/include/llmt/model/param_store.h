// Parameter container with llmt's registration API
// (llmt include/llmt/model/param_store.h:107-195): parameters are registered (add / alias),
// then finalize() carves four spans - weights, gradients and Adam's two moments - out of ONE
// allocation, zero-filled, every parameter at the same offset in spans of one dtype.  The
// gradient span is contiguous so that ONE exchange covers every dW/dbias of a step
// (llmt param_store.h:131-135: "future NCCL - one transfer each instead of one per tensor").
//
// Data-parallel extension: the gradient span may live in memory that the caller provides
// (finalize(span, bytes)), e.g. inside a dist::PeerExchange allocation that the other ranks
// can address; allreduce_grads() then sums it over the ranks in place.
#pragma once

#include <cuda_runtime.h>

#include <deque>
#include <optional>
#include <string>
#include <string_view>
#include <unordered_map>

#include "llmt/core/arena.h"
#include "llmt/core/types.h"

namespace llmt {

namespace dist {
class PeerExchange;
}

// First four values as in llmt (param_store.h: Role); Bias is the extension.
enum class Role : uint8_t { Embedding, Matrix, ResidualProj, Norm, Bias };
enum class StateKind : uint8_t { Weight, Grad, AdamM, AdamV };
constexpr int kNumStateKinds = 4;

// Storage dtype of each state kind.
struct StateDtypes {
    DType of[kNumStateKinds] = {DType::FP32, DType::FP32, DType::FP32, DType::FP32};

    static constexpr StateDtypes uniform(DType d) noexcept {
        StateDtypes s;
        for (DType& x : s.of) x = d;
        return s;
    }
    // bf16 (or any other) weights with fp32 gradients and moments: the mixed-precision setting.
    static constexpr StateDtypes mixed(DType weight, DType rest = DType::FP32) noexcept {
        StateDtypes s = uniform(rest);
        s.of[0] = weight;
        return s;
    }
    constexpr DType operator[](StateKind k) const noexcept { return of[static_cast<int>(k)]; }
};

struct Param {
    std::string name;
    Shape shape;
    Role role = Role::Matrix;
    Tensor weight, grad, adam_m, adam_v;  // one view per state kind; grad ACCUMULATES (+=)

    const Tensor& state(StateKind k) const noexcept {
        const Tensor* const t[kNumStateKinds] = {&weight, &grad, &adam_m, &adam_v};
        return *t[static_cast<int>(k)];
    }
    Tensor& state(StateKind k) noexcept {
        Tensor* const t[kNumStateKinds] = {&weight, &grad, &adam_m, &adam_v};
        return *t[static_cast<int>(k)];
    }
    // Identity of the parameter's random stream: a hash of its name (FNV-1a, 64 bit), so that
    // initial values do not depend on registration order (llmt param_store.h:36-43).
    uint64_t stream_id() const noexcept {
        uint64_t h = 14695981039346656037ull;
        for (const char c : std::string_view(name)) h = (h ^ static_cast<unsigned char>(c)) * 1099511628211ull;
        return h;
    }
};

class ParamStore {
   public:
    explicit ParamStore(StateDtypes dtypes) noexcept : dtypes_(dtypes) {}
    Param& add(std::string name, const Shape& shape, Role role) noexcept;
    // Weight tying: alias_name resolves to the existing parameter `target`; no storage is
    // added, and the shared gradient receives one += from each consumer's backward.
    void alias(const std::string& alias_name, const std::string& target) noexcept;
    void finalize() noexcept;
    // The same, with the gradient span placed in caller-provided device memory of at least
    // grad_span_bytes() bytes (256-byte aligned); the store zero-fills it but does not own it.
    void finalize(void* grad_span, size_t bytes) noexcept;
    bool finalized() const noexcept { return mem_.has_value(); }
    Param& at(const std::string& name) noexcept;
    const Param& at(const std::string& name) const noexcept;
    const std::deque<Param>& params() const noexcept { return params_; }
    int64_t param_numel() const noexcept { return param_numel_; }   // real elements, no padding
    // Size the gradient span will have (valid before finalize, once every add() is done).
    size_t grad_span_bytes() const noexcept { return span_bytes_of(StateKind::Grad); }
    Tensor flat(StateKind k) const noexcept;  // whole span incl. alignment padding (kept zero)
    void zero_grad(cudaStream_t s) noexcept;
    // Sums the gradient span over the ranks of `ex`, in place, on `stream` (one call per step,
    // after the last backward; never on a span that already holds a reduced value).  The span
    // must have been placed in ex's memory: finalize(ex.span(), ex.span_bytes()).
    void allreduce_grads(dist::PeerExchange& ex, cudaStream_t stream) noexcept;

   private:
    size_t span_bytes_of(StateKind k) const noexcept;
    void carve(void* external_grad, size_t external_bytes) noexcept;

    StateDtypes dtypes_;
    std::deque<Param> params_;
    std::unordered_map<std::string, size_t> index_;   // real names and aliases
    int64_t param_numel_ = 0;
    size_t span_bytes_[kNumStateKinds] = {0, 0, 0, 0};
    char* base_[kNumStateKinds] = {nullptr, nullptr, nullptr, nullptr};
    std::optional<Arena> mem_;
};

}  // namespace llmt
