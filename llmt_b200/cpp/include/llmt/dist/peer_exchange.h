// Host side of the gradient exchange for a C++ program: one process per GPU, the flat fp32
// gradient span of every rank in memory the other ranks can address (CUDA IPC), and the
// library's exchange kernel (llmt_b200_grad_allreduce, peer-copy form) over it.
//
// llmt has no multi-GPU code; the seam it documents for it is the flat gradient span of its
// ParamStore (llmt include/llmt/model/param_store.h:131-135,185).  Typical use:
//
//     ParamStore ps(dtypes);  ... add() every parameter ...
//     dist::PeerExchange ex(rank, world, ps.grad_span_bytes() / 4, allgather);
//     ps.finalize(ex.span(), ex.span_bytes());
//     ... backward passes accumulate into the gradient views ...
//     ps.allreduce_grads(ex, stream);        // or ex.allreduce(offset, count, stream) per layer
//
// The ranks exchange their IPC handles through `allgather`, which the host program supplies
// from whatever it already has between its processes (MPI_Allgather, a socket, a shared file).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <functional>

#include "llmt_b200.h"

namespace llmt::dist {

// allgather(send, recv, n): every rank contributes n bytes; recv receives world * n bytes,
// rank r's contribution at offset r * n.  Blocking; also serves as a barrier.
using AllGatherFn = std::function<void(const void* send, void* recv, size_t n)>;

// Byte layout of one rank's peer-visible allocation: the span, then `world` staging slots of
// one shard each, then the flag words.
struct ExchangeLayout {
    int64_t slot_elems = 0;
    size_t grad_off = 0, stage_off = 0, flags_off = 0, total = 0;
};
ExchangeLayout exchange_layout(int64_t numel, int world) noexcept;

class PeerExchange {
   public:
    // Collective over all ranks: allocates, exchanges IPC handles, maps the peers' buffers.
    // The current device must be this rank's GPU, and every pair of GPUs must have peer
    // access to each other (NVLink or PCIe).  numel: floats in the span, a multiple of 4.
    PeerExchange(int rank, int world, int64_t numel, const AllGatherFn& allgather, int ctas = 16) noexcept;
    ~PeerExchange();
    PeerExchange(const PeerExchange&) = delete;
    PeerExchange& operator=(const PeerExchange&) = delete;

    float* span() const noexcept { return span_; }
    size_t span_bytes() const noexcept { return static_cast<size_t>(numel_) * sizeof(float); }
    int rank() const noexcept { return rank_; }
    int world() const noexcept { return world_; }
    // Sums floats [offset, offset + count) of the span over all ranks, in place, on `stream`.
    // Every rank makes the same calls in the same order; calls of one exchange must not
    // overlap (keep them on one stream).  Aborts with llmt's message convention on a status.
    void allreduce(int64_t offset, int64_t count, cudaStream_t stream) noexcept;
    const llmt_b200_comm_desc& desc() const noexcept { return desc_; }

   private:
    int rank_ = 0, world_ = 1, ctas_ = 16;
    int64_t numel_ = 0;
    char* local_ = nullptr;                      // this rank's allocation
    char* peer_[LLMT_B200_COMM_MAX_RANKS] = {};  // every rank's allocation as this rank addresses it
    void* epoch_ = nullptr;
    float* span_ = nullptr;
    llmt_b200_comm_desc desc_{};
};

}  // namespace llmt::dist
