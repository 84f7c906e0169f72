// Per-call context threaded through every launch (llmt run_ctx.h:32-43).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "llmt/core/types.h"

namespace llmt::kernels {
struct AlgoCache;
}

namespace llmt {

class Arena;

enum class KernelBackend : uint8_t { Naive, Fused };

struct RunCtx {
    cudaStream_t stream = nullptr;
    void* blas = nullptr;             // llmt keeps a cuBLASLt handle here; unused, kept for layout parity
    void* blas_workspace = nullptr;   // Device-owned scratch, used for split-K partial sums
    size_t blas_workspace_bytes = 0;
    kernels::AlgoCache* algo_cache = nullptr;  // Device-owned record of the plans used
    Arena* activations = nullptr;
    PrecisionPolicy precision;
    KernelBackend backend = KernelBackend::Naive;
    uint64_t seed = 0;
    int64_t step = 0;
    // Data-parallel extension: rank / world size of the process that owns this
    // context and an opaque communicator (ncclComm_t) for gradient reduction.
    int rank = 0;
    int world = 1;
    void* comm = nullptr;
};

}  // namespace llmt
