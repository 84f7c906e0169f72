// dist::PeerExchange: the peers' buffers mapped with CUDA IPC, the exchange itself is the
// library's kernel (llmt_b200_grad_allreduce, peer-copy form: plain peer loads and stores,
// no multicast object).  llmt has no counterpart (single GPU); the seam is the flat gradient
// span of its ParamStore (llmt include/llmt/model/param_store.h:131-135).
#include "llmt/dist/peer_exchange.h"

#include <cstring>
#include <vector>

#include "llmt/core/error.h"

namespace llmt::dist {

ExchangeLayout exchange_layout(int64_t numel, int world) noexcept {
    ExchangeLayout lay;
    const int64_t shard = (numel / 4 + world - 1) / world * 4;          // floats per rank, whole float4s
    lay.slot_elems = (shard + 63) / 64 * 64;                             // 256-byte slots
    const size_t grad_bytes = (static_cast<size_t>(numel) * 4 + 255) / 256 * 256;
    const size_t stage_bytes = static_cast<size_t>(world) * static_cast<size_t>(lay.slot_elems) * 4;
    lay.grad_off = 0;
    lay.stage_off = grad_bytes;
    lay.flags_off = grad_bytes + stage_bytes;
    lay.total = lay.flags_off + LLMT_B200_COMM_FLAG_BYTES;
    return lay;
}

PeerExchange::PeerExchange(int rank, int world, int64_t numel, const AllGatherFn& allgather, int ctas) noexcept
    : rank_(rank), world_(world), ctas_(ctas), numel_(numel) {
    if (world < 1 || world > LLMT_B200_COMM_MAX_RANKS || rank < 0 || rank >= world)
        detail::fatal("peer_exchange", "rank %d / world %d out of range (1..%d ranks)", rank, world,
                      LLMT_B200_COMM_MAX_RANKS);
    if (numel <= 0 || numel % 4 != 0) detail::fatal("peer_exchange", "span length must be a positive multiple of 4 floats");
    if (ctas < 1 || ctas > LLMT_B200_COMM_MAX_CTAS) detail::fatal("peer_exchange", "ctas must be 1..%d", LLMT_B200_COMM_MAX_CTAS);
    const ExchangeLayout lay = exchange_layout(numel, world);
    CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&local_), lay.total));
    CUDA_CHECK(cudaMemset(local_, 0, lay.total));
    CUDA_CHECK(cudaMalloc(&epoch_, LLMT_B200_COMM_EPOCH_BYTES));
    CUDA_CHECK(cudaMemset(epoch_, 0, LLMT_B200_COMM_EPOCH_BYTES));
    CUDA_CHECK(cudaDeviceSynchronize());
    peer_[rank] = local_;
    if (world > 1) {
        if (!allgather) detail::fatal("peer_exchange", "an allgather function is required for world > 1");
        cudaIpcMemHandle_t mine;
        CUDA_CHECK(cudaIpcGetMemHandle(&mine, local_));
        std::vector<cudaIpcMemHandle_t> all(static_cast<size_t>(world));
        allgather(&mine, all.data(), sizeof mine);
        for (int r = 0; r < world; ++r) {
            if (r == rank) continue;
            void* p = nullptr;
            CUDA_CHECK(cudaIpcOpenMemHandle(&p, all[static_cast<size_t>(r)], cudaIpcMemLazyEnablePeerAccess));
            peer_[r] = static_cast<char*>(p);
        }
        // nobody raises a flag before every rank has zeroed its own and mapped everybody's
        char token = 0;
        std::vector<char> tokens(static_cast<size_t>(world));
        allgather(&token, tokens.data(), 1);
    }
    span_ = reinterpret_cast<float*>(local_ + lay.grad_off);
    desc_.rank = rank;
    desc_.world = world;
    desc_.slot_elems = lay.slot_elems;
    for (int r = 0; r < world; ++r) {
        desc_.grad[r] = peer_[r] + lay.grad_off;
        desc_.stage[r] = peer_[r] + lay.stage_off;
        desc_.flags[r] = peer_[r] + lay.flags_off;
    }
    desc_.epoch = epoch_;
    desc_.grad_mc = nullptr;
}

PeerExchange::~PeerExchange() {
    cudaDeviceSynchronize();
    for (int r = 0; r < world_; ++r)
        if (r != rank_ && peer_[r] != nullptr) cudaIpcCloseMemHandle(peer_[r]);
    if (epoch_ != nullptr) cudaFree(epoch_);
    if (local_ != nullptr) cudaFree(local_);
}

void PeerExchange::allreduce(int64_t offset, int64_t count, cudaStream_t stream) noexcept {
    const int st = llmt_b200_grad_allreduce(&desc_, offset, count, ctas_, stream);
    if (st != LLMT_B200_OK) detail::fatal("peer_exchange", "%s", llmt_b200_last_error());
}

}  // namespace llmt::dist
