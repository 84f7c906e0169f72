// Per-GPU runtime state (llmt device.h:37-70): one explicit stream, the GEMM
// scratch buffer and the plan record.  There is no cuBLASLt handle.
#pragma once

#include <cuda_runtime.h>

#include <memory>
#include <string>

#include "llmt/core/run_ctx.h"

namespace llmt {

struct DeviceProps {
    std::string name;
    int sm_major = 0, sm_minor = 0;
    int sm_count = 0;
    size_t vram_bytes = 0;
    size_t l2_bytes = 0;
};

class Device {
   public:
    // Sized for the largest split-K plan of the GPT-2 shapes (fp32 partial sums).
    static constexpr size_t kBlasWorkspaceBytes = 256ull << 20;

    explicit Device(int index = 0) noexcept;
    ~Device();
    Device(const Device&) = delete;
    Device& operator=(const Device&) = delete;

    const DeviceProps& props() const noexcept { return props_; }
    cudaStream_t stream() const noexcept { return stream_; }
    int index() const noexcept { return index_; }
    RunCtx make_ctx(uint64_t seed, KernelBackend backend, PrecisionPolicy precision) const noexcept;
    void synchronize() const noexcept;

   private:
    int index_ = 0;
    DeviceProps props_;
    cudaStream_t stream_ = nullptr;
    void* workspace_ = nullptr;
    std::unique_ptr<kernels::AlgoCache> cache_;
};

}  // namespace llmt
