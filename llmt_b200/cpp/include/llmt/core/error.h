// Print-and-abort error convention of llmt (include/llmt/core/error.h:16-54):
// contract violations and CUDA failures write "[llmt] <where>: <message>" to
// stderr and abort; nothing throws.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>

namespace llmt::detail {

[[noreturn]] inline void fatal(const char* where, const char* fmt, ...) noexcept {
    std::fputs("[llmt] ", stderr);
    std::fputs(where, stderr);
    std::fputs(": ", stderr);
    va_list ap;
    va_start(ap, fmt);
    std::vfprintf(stderr, fmt, ap);
    va_end(ap);
    std::fputc('\n', stderr);
    std::abort();
}

inline void cuda_check(cudaError_t e, const char* expr, const char* file, int line) noexcept {
    if (e == cudaSuccess) return;
    std::fprintf(stderr, "[llmt] CUDA error %s:%d: %s (%s)\n", file, line, cudaGetErrorString(e), expr);
    std::abort();
}

}  // namespace llmt::detail

#define CUDA_CHECK(call) ::llmt::detail::cuda_check((call), #call, __FILE__, __LINE__)
#define CUDA_CHECK_LAST() CUDA_CHECK(cudaGetLastError())
