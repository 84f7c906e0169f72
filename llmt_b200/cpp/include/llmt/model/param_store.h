// Minimal parameter container with llmt's registration API
// (include/llmt/model/param_store.h:107-195): parameters are registered, then
// finalize() carves one weight span and one gradient span out of a single
// allocation, zero-filled.  The gradient span is contiguous so that one
// all-reduce covers every dW/dbias of a step.
#pragma once

#include <deque>
#include <optional>
#include <string>
#include <unordered_map>

#include "llmt/core/arena.h"
#include "llmt/core/types.h"

namespace llmt {

// First four values as in llmt (param_store.h: Role); Bias is the extension.
enum class Role : uint8_t { Embedding, Matrix, ResidualProj, Norm, Bias };
enum class StateKind : uint8_t { Weight, Grad };

struct StateDtypes {
    DType weight = DType::FP32, grad = DType::FP32;
    static StateDtypes uniform(DType d) noexcept { return {d, d}; }
};

struct Param {
    std::string name;
    Shape shape;
    Role role = Role::Matrix;
    Tensor weight, grad;
};

class ParamStore {
   public:
    explicit ParamStore(StateDtypes dtypes) noexcept : dtypes_(dtypes) {}
    Param& add(std::string name, const Shape& shape, Role role) noexcept;
    void finalize() noexcept;
    bool finalized() const noexcept { return mem_.has_value(); }
    Param& at(const std::string& name) noexcept;
    const std::deque<Param>& params() const noexcept { return params_; }
    Tensor flat(StateKind k) const noexcept;  // whole span incl. alignment padding (kept zero)
    void zero_grad(cudaStream_t s) noexcept;

   private:
    StateDtypes dtypes_;
    std::deque<Param> params_;
    std::unordered_map<std::string, size_t> index_;
    size_t span_bytes_[2] = {0, 0};
    char* base_[2] = {nullptr, nullptr};
    std::optional<Arena> mem_;
};

}  // namespace llmt
