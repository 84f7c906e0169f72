// Bump allocator over one cudaMalloc (llmt arena.h:21-55, src/core/arena.cu).
#pragma once

#include <cstddef>

#include "llmt/core/types.h"

namespace llmt {

class Arena {
   public:
    static constexpr size_t kAlign = 256;

    explicit Arena(size_t capacity, const char* name = "arena") noexcept;
    ~Arena();
    Arena(const Arena&) = delete;
    Arena& operator=(const Arena&) = delete;

    void* alloc_bytes(size_t bytes) noexcept;            // aborts when exhausted
    Tensor alloc(const Shape& shape, DType dtype) noexcept;
    void reset() noexcept { used_ = 0; }

    size_t used() const noexcept { return used_; }
    size_t capacity() const noexcept { return capacity_; }
    size_t high_water() const noexcept { return peak_; }
    const char* name() const noexcept { return name_; }

   private:
    char* base_ = nullptr;
    size_t capacity_ = 0, used_ = 0, peak_ = 0;
    const char* name_;
};

}  // namespace llmt
