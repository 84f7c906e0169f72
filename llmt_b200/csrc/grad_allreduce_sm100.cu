// Sum of the flat fp32 gradient span over the data-parallel ranks, written for NVLink peer
// memory: one kernel per call, a handful of CTAs, bulk asynchronous copies (cp.async.bulk)
// between HBM, shared memory and the peers' HBM (no multimem, no multicast), deterministic.
//
// llmt has no multi-GPU code; the span is its designed seam for it (llmt
// include/llmt/model/param_store.h:131-135,185).  The GEMM kernels are persistent and fill
// the SMs they are given, so the exchange has to run beside them on few SMs; that is what a
// streaming copy over peer pointers does well and what a channel-per-CTA library does badly.
//
// Algorithm for a range of the span, W ranks, G CTAs per rank (CTA g of every rank works on
// slice g of every shard, so CTAs only ever wait for the CTA of the same index on the peers):
//   1. push   : rank r copies its partial sums of shard s into slot r of rank s's staging
//               area, for every s != r, then raises flag (push, r, g) on rank s.
//   2. reduce : rank r waits for the W-1 push flags, adds the W partial sums of its own shard
//               in rank order 0..W-1 (own span + staging slots), writes the sum to its own
//               span and to the same place of every peer's span, then raises flag (sum, r, g)
//               on every peer.
//   3. join   : rank r waits for the W-1 sum flags: its span now holds every shard's sum.
// Every shard is summed once, by its owner, in a fixed order, and then copied: all ranks end
// with the same bits and reruns reproduce them.  Flags are call counters (kept per CTA in the
// rank's own memory), so a captured launch can be replayed; staging slots are free again when
// the call returns because the join of a rank follows every peer's reduce.
// Every wait gives up after AllreduceParams::wait_limit_ns, records kDevWaitPeer and lets the
// kernel finish.
//
// Data movement: one thread per CTA drives the copy engine.  Push is a ring of 16 KB buffers
// (bulk load from the own span, bulk store into the peer's staging slot, eight loads in
// flight).  Reduce reads the W partial sums of 16 KB of output with plain loads (up to 2 W
// float4 in flight per thread), adds them in rank order into a shared-memory buffer, and W
// bulk stores carry that buffer to the own span and to every peer's.
#include "common.h"
#include "ptx_sm100.cuh"

namespace llmt_b200 {

namespace {

using namespace ptx;

constexpr uint32_t kPushChunk = 16384;                 // bytes per ring buffer
constexpr int kPushBufs = 12, kPushAhead = 8;          // ring size, loads in flight
constexpr uint32_t kSumChunk = 16384;                  // bytes per output buffer of the reduce phase
constexpr int kSumBufs = 4;
constexpr uint32_t kCommSmemBytes = kPushChunk * kPushBufs;  // 192 KB; the reduce phase reuses the first 64 KB

// Staging slots are written by the peers: read them past L1.
__device__ __forceinline__ float4 ld_stage(const float4* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// global -> shared bulk copy; completes `bytes` on the mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// shared -> global bulk copy (the destination may be a peer's memory); joins the current bulk group
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
                 : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void record_failure(const CommRank& c, int detail, int g, int* s_ok) {
    if (atomicCAS(&c.status->code, 0, kDevWaitPeer) == 0) {
        c.status->detail = detail;
        c.status->block = g;
    }
    *s_ok = 0;
}

// Bounded wait on a local mbarrier (bulk loads from this GPU's own memory land on it).
__device__ __forceinline__ bool wait_full(uint32_t bar, uint32_t parity, const CommRank& c, int g, int* s_ok,
                                          uint64_t limit_ns) {
    // the wall clock is slow to read: it is first looked at after 256 failed polls
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0u) {
            if (*reinterpret_cast<volatile int*>(s_ok) == 0) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                record_failure(c, 1024, g, s_ok);
                return false;
            }
        }
    }
    return true;
}

// Thread `tid` < world (tid != me) waits until the flag written by rank tid reaches `e`.
__device__ __forceinline__ void wait_peers(const CommRank& c, int phase, int g, uint32_t e, int* s_ok,
                                           uint64_t limit_ns) {
    const int tid = threadIdx.x;
    if (tid < c.world && tid != c.rank) {
        const uint32_t* f = c.flags[c.rank] + (phase * kMaxCommRanks + tid) * kMaxCommCtas + g;
        uint64_t t0 = 0;
        uint32_t spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys(f) - e) < 0) {
            if ((++spins & 31u) == 0u) {
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > limit_ns) {
                    record_failure(c, phase * 256 + tid, g, s_ok);
                    break;
                }
            }
        }
    }
    __syncthreads();
    // what the peers wrote is read by the copy engine next, on thread 0's behalf
    if (tid == 0) fence_proxy_async_all();
}

// Called by thread 0 after its bulk stores have completed (bulk_wait_group0): publishes them.
__device__ __forceinline__ void raise_flags(const CommRank& c, int phase, int g, uint32_t e) {
    __threadfence_system();
    for (int r = 0; r < c.world; ++r)
        if (r != c.rank) st_release_sys(c.flags[r] + (phase * kMaxCommRanks + c.rank) * kMaxCommCtas + g, e);
}

// Sequence of push chunks of one CTA: for every foreign shard s = me+1, me+2, ... its slice
// [lo, hi_s) cut into kPushChunk pieces.
struct PushCursor {
    int d;          // 1 .. W-1: shard (me + d) % W
    int64_t pos;    // float4 index within the shard
};

__global__ void __launch_bounds__(kCommThreads)
grad_allreduce_kernel(const AllreduceParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) uint64_t full_bar[kPushBufs];
    __shared__ uint32_t s_epoch;
    __shared__ int s_ok;

    const CommRank& c = P.ctx[blockIdx.y];
    const int g = blockIdx.x, G = gridDim.x, W = c.world, me = c.rank;
    const int tid = threadIdx.x;
    if (tid == 0) {
        s_epoch = c.epoch[g] + 1u;
        s_ok = 1;
        for (int i = 0; i < kPushBufs; ++i) mbar_init(smem_u32(&full_bar[i]), 1);
        fence_barrier_init();
    }
    __syncthreads();
    const uint32_t e = s_epoch;
    const uint32_t smem_base = smem_u32(smem);

    // geometry in float4 units: W shards of shard4, each cut into G slices of slice4
    const int64_t n4 = P.count / 4;
    const int64_t shard4 = (n4 + W - 1) / W;
    const int64_t slice4 = (shard4 + G - 1) / G;
    const int64_t lo = g * slice4;
    const int64_t hi_slice = lo + slice4 < shard4 ? lo + slice4 : shard4;
    float4* own = reinterpret_cast<float4*>(c.grad[me] + P.offset);
    const int64_t slot4 = c.slot_elems / 4;
    // ---- 1. push my partial sums of every foreign shard to its owner -------------------------
    if (tid == 0) {
        constexpr int64_t kChunk4 = kPushChunk / 16;
        auto hi_of = [&](int d) {
            const int64_t rest = n4 - static_cast<int64_t>((me + d) % W) * shard4;
            return rest < hi_slice ? rest : hi_slice;
        };
        auto settle = [&](PushCursor& cur) {  // skip exhausted or empty shards
            while (cur.d < W && cur.pos >= hi_of(cur.d)) { ++cur.d; cur.pos = lo; }
        };
        PushCursor lc{1, lo}, sc{1, lo};
        settle(lc); settle(sc);
        int64_t n_loaded = 0, n_stored = 0;
        auto load_next = [&]() {
            const int s = (me + lc.d) % W;
            const int64_t hi = hi_of(lc.d);
            const int64_t len4 = hi - lc.pos < kChunk4 ? hi - lc.pos : kChunk4;
            const int b = static_cast<int>(n_loaded % kPushBufs);
            const uint32_t bar = smem_u32(&full_bar[b]);
            mbar_arrive_expect_tx(bar, static_cast<uint32_t>(len4 * 16));
            bulk_load(smem_base + b * kPushChunk, own + s * shard4 + lc.pos, static_cast<uint32_t>(len4 * 16), bar);
            lc.pos += len4; ++n_loaded;
            settle(lc);
        };
        for (int i = 0; i < kPushAhead && lc.d < W; ++i) load_next();
        bool ok = true;
        while (sc.d < W) {
            const int s = (me + sc.d) % W;
            const int64_t hi = hi_of(sc.d);
            const int64_t len4 = hi - sc.pos < kChunk4 ? hi - sc.pos : kChunk4;
            const int b = static_cast<int>(n_stored % kPushBufs);
            ok = wait_full(smem_u32(&full_bar[b]), static_cast<uint32_t>((n_stored / kPushBufs) & 1), c, g, &s_ok,
                           P.wait_limit_ns);
            if (!ok) break;
            bulk_store(reinterpret_cast<float4*>(c.stage[s]) + me * slot4 + sc.pos, smem_base + b * kPushChunk,
                       static_cast<uint32_t>(len4 * 16));
            bulk_commit_group();
            sc.pos += len4; ++n_stored;
            settle(sc);
            if (lc.d < W) {
                // the buffer of load n_loaded was last read by the store kPushBufs chunks earlier
                bulk_wait_read<kPushBufs - kPushAhead>();
                load_next();
            }
        }
        bulk_wait_group0();
        raise_flags(c, 0, g, e);
    }
    // ---- 2. sum my own shard in rank order and hand the result to everybody ------------------
    wait_peers(c, 0, g, e, &s_ok, P.wait_limit_ns);
    {
        const int64_t base = me * shard4;
        int64_t hi = n4 - base;
        if (hi > hi_slice) hi = hi_slice;
        constexpr int64_t kOut4 = kSumChunk / 16;
        const int64_t n_chunks = hi > lo ? (hi - lo + kOut4 - 1) / kOut4 : 0;
        const float4* st = reinterpret_cast<const float4*>(c.stage[me]);
        for (int64_t k = 0; k < n_chunks; ++k) {
            const int b = static_cast<int>(k % kSumBufs);
            const int64_t pos = lo + k * kOut4;
            const int64_t len4 = hi - pos < kOut4 ? hi - pos : kOut4;
            float4* out = reinterpret_cast<float4*>(smem + b * kSumChunk);
            // two float4 per thread and pass: up to 2 * W loads in flight per thread
            for (int64_t i0 = tid; i0 < len4; i0 += 2 * kCommThreads) {
                const int64_t i1 = i0 + kCommThreads;
                const bool two = i1 < len4;
                float4 p0[kMaxCommRanks], p1[kMaxCommRanks];
#pragma unroll
                for (int r = 0; r < kMaxCommRanks; ++r)
                    if (r < W) {
                        p0[r] = r == me ? own[base + pos + i0] : ld_stage(st + r * slot4 + pos + i0);
                        if (two) p1[r] = r == me ? own[base + pos + i1] : ld_stage(st + r * slot4 + pos + i1);
                    }
                float4 a0 = p0[0], a1 = p1[0];
#pragma unroll
                for (int r = 1; r < kMaxCommRanks; ++r)
                    if (r < W) {
                        a0.x += p0[r].x; a0.y += p0[r].y; a0.z += p0[r].z; a0.w += p0[r].w;
                        a1.x += p1[r].x; a1.y += p1[r].y; a1.z += p1[r].z; a1.w += p1[r].w;
                    }
                out[i0] = a0;
                if (two) out[i1] = a1;
            }
            fence_proxy_async_smem();  // the sums are read by the copy engine next
            // thread 0: the next output buffer must have been drained by the stores that used it
            if (tid == 0) bulk_wait_read<kSumBufs - 2>();
            __syncthreads();
            if (tid == 0) {
                const uint32_t bytes = static_cast<uint32_t>(len4 * 16);
                for (int d = 0; d < W; ++d) {
                    const int s = (me + d) % W;
                    bulk_store(reinterpret_cast<float4*>(c.grad[s] + P.offset) + base + pos, smem_base + b * kSumChunk,
                               bytes);
                }
                bulk_commit_group();
            }
        }
    }
    if (tid == 0) {
        bulk_wait_group0();
        raise_flags(c, 1, g, e);
    }

    // ---- 3. my span is complete once every peer has delivered its shard ----------------------
    wait_peers(c, 1, g, e, &s_ok, P.wait_limit_ns);
    if (tid == 0) c.epoch[g] = e;
}

// ---- the same sum through NVSwitch multicast ------------------------------------------------
// With the span mapped through a multicast object, one multimem.ld_reduce fetches the sum of
// all ranks' values (added inside the switch) and one multimem.st writes it to every rank:
// rank r moves 1/W of the range in and out instead of pushing and copying W-1 shards, so the
// SM-side traffic drops by about 2W.  No shared memory and few registers: the CTAs fit on SMs
// that a resident GEMM CTA already occupies.  Every element is summed once (by its owner) and
// broadcast, so all ranks hold the same bits; the order of the additions is the switch's.
constexpr int kMcThreads = 256;

__global__ void __launch_bounds__(kMcThreads, 2)
grad_allreduce_mc_kernel(const AllreduceParams P) {
    const CommRank& c = P.ctx[0];
    const int g = blockIdx.x, G = gridDim.x, W = c.world, me = c.rank;
    const int tid = threadIdx.x;
    // no shared memory at all: the CTA must fit beside a GEMM CTA that owns the SM's
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(c.epoch + g) + 1u;
    int s_ok = 1;
    const int64_t n4 = P.count / 4;
    const int64_t shard4 = (n4 + W - 1) / W;
    const int64_t slice4 = (shard4 + G - 1) / G;
    const int64_t lo = g * slice4;
    int64_t hi = lo + slice4 < shard4 ? lo + slice4 : shard4;
    if (hi > n4 - me * shard4) hi = n4 - me * shard4;

    // 0. every rank's partial sums are in place (they were written by earlier kernels)
    if (tid < W && tid != me) st_release_sys(c.flags[tid] + (0 * kMaxCommRanks + me) * kMaxCommCtas + g, e);
    wait_peers(c, 0, g, e, &s_ok, P.wait_limit_ns);

    // 1. my shard: sum in the switch, broadcast to everybody
    float4* mc = reinterpret_cast<float4*>(c.grad_mc + P.offset) + me * shard4;
    int64_t i = lo + tid;
    constexpr int kU = 8;  // switch round trips are long: eight 16-byte reductions in flight per thread
    for (; i + (kU - 1) * kMcThreads < hi; i += kU * kMcThreads) {
        float4 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) v[u] = multimem_ld_reduce_add(mc + i + u * kMcThreads);
#pragma unroll
        for (int u = 0; u < kU; ++u) multimem_st(mc + i + u * kMcThreads, v[u]);
    }
    for (; i < hi; i += kMcThreads) multimem_st(mc + i, multimem_ld_reduce_add(mc + i));

    // 2. everybody's shard has reached me
    __threadfence_system();
    __syncthreads();
    if (tid < W && tid != me) st_release_sys(c.flags[tid] + (1 * kMaxCommRanks + me) * kMaxCommCtas + g, e);
    wait_peers(c, 1, g, e, &s_ok, P.wait_limit_ns);
    if (tid == 0) c.epoch[g] = e;
}

}  // namespace

// Ride-along exchanges number themselves step * kMaxRidesPerStep + index; the step counter lives
// on the device so that a captured step can be replayed.
__global__ void exchange_begin_step_kernel(uint32_t* step_word) { *step_word = *step_word + 1u; }

cudaError_t launch_exchange_begin_step(uint32_t* step_word, cudaStream_t stream) {
    exchange_begin_step_kernel<<<1, 1, 0, stream>>>(step_word);
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_grad_allreduce_mc(const AllreduceParams& p, int ctas, cudaStream_t stream) {
    grad_allreduce_mc_kernel<<<dim3(ctas, 1), kMcThreads, 0, stream>>>(p);
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_grad_allreduce(const AllreduceParams& p, int ctas, int emulated_ranks, cudaStream_t stream) {
    static bool configured[64];  // the attribute is per device
    int dev = 0;
    cudaError_t e0 = cudaGetDevice(&dev);
    if (e0 != cudaSuccess) return e0;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(grad_allreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kCommSmemBytes));
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    cudaError_t e;
    if (emulated_ranks > 0) {
        // All ranks in one grid on one device: the blocks wait on one another, so the launch
        // must be cooperative (refused unless every block is resident at once).
        AllreduceParams copy = p;
        void* args[] = {&copy};
        e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(grad_allreduce_kernel),
                                        dim3(ctas, emulated_ranks), dim3(kCommThreads), args, kCommSmemBytes, stream);
    } else {
        grad_allreduce_kernel<<<dim3(ctas, 1), kCommThreads, kCommSmemBytes, stream>>>(p);
        e = cudaGetLastError();
    }
    count_launch(1);
    return e;
}

}  // namespace llmt_b200
