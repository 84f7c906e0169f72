// Value types at the GEMM boundary: element type, shape, tensor view and the
// precision policy.  Same names, fields and meaning as llmt's
// include/llmt/core/{dtype,shape,tensor,precision}.h so code written against
// llmt compiles against this tree; the implementation is independent.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>
#include <initializer_list>

#if defined(__CUDACC__)
#define LLMT_HD __host__ __device__
#else
#define LLMT_HD
#endif

namespace llmt {

// Codes match llmt's DType (dtype.h:15) and its golden-file header.
enum class DType : uint8_t { FP32 = 0, BF16 = 1, I32 = 2 };

constexpr size_t dtype_size(DType d) noexcept {
    return d == DType::BF16 ? 2 : (d == DType::FP32 || d == DType::I32) ? 4 : 0;
}
constexpr const char* dtype_name(DType d) noexcept {
    return d == DType::FP32 ? "fp32" : d == DType::BF16 ? "bf16" : d == DType::I32 ? "i32" : "?";
}

// Opaque 16-bit storage for bf16 elements on the host side of the boundary.
struct bf16_bits {
    uint16_t v;
};

template <typename T> struct dtype_of;
template <> struct dtype_of<float>     { static constexpr DType value = DType::FP32; };
template <> struct dtype_of<int32_t>   { static constexpr DType value = DType::I32; };
template <> struct dtype_of<bf16_bits> { static constexpr DType value = DType::BF16; };

// Up to four extents, row-major (llmt shape.h:18-53).
struct Shape {
    static constexpr int kMaxRank = 4;
    std::array<int64_t, kMaxRank> d{{0, 0, 0, 0}};
    int rank = 0;

    Shape() = default;
    Shape(std::initializer_list<int64_t> dims) noexcept {
        for (int64_t e : dims)
            if (rank < kMaxRank) d[static_cast<size_t>(rank++)] = e;
    }
    int64_t operator[](int i) const noexcept { return d[static_cast<size_t>(i)]; }
    int64_t numel() const noexcept {
        int64_t n = rank > 0 ? 1 : 0;
        for (int i = 0; i < rank; ++i) n *= d[static_cast<size_t>(i)];
        return n;
    }
    bool operator==(const Shape& o) const noexcept {
        if (rank != o.rank) return false;
        for (int i = 0; i < rank; ++i)
            if (d[static_cast<size_t>(i)] != o.d[static_cast<size_t>(i)]) return false;
        return true;
    }
    bool operator!=(const Shape& o) const noexcept { return !(*this == o); }
};

// Non-owning view of contiguous row-major device memory (llmt tensor.h:17-35).
struct Tensor {
    void* data = nullptr;
    DType dtype = DType::FP32;
    Shape shape;

    int64_t numel() const noexcept { return shape.numel(); }
    size_t bytes() const noexcept { return static_cast<size_t>(numel()) * dtype_size(dtype); }
    bool valid() const noexcept { return data != nullptr && shape.rank > 0; }
    template <typename T>
    T* ptr() const noexcept { return static_cast<T*>(data); }
};

// {master, gemm_compute, reduce} (llmt precision.h:16-22).  Two settings have
// kernels: fp32() = strict fp32 FMA, and bf16_mixed() = bf16 tensor-core
// multiply with fp32 accumulation.
struct PrecisionPolicy {
    DType master = DType::FP32;
    DType gemm_compute = DType::FP32;
    DType reduce = DType::FP32;
    static PrecisionPolicy fp32() noexcept { return {}; }
    static PrecisionPolicy bf16_mixed() noexcept { return {DType::FP32, DType::BF16, DType::FP32}; }
};

using kernel_compute_t = float;
using host_result_t = float;

}  // namespace llmt
