// bf16 x bf16 -> fp32-accumulate GEMM for sm_100a as ONE persistent kernel over
// a list of problems ("group"): tcgen05 MMA with the accumulator in tensor
// memory, operands staged in 128-byte-swizzled shared memory by TMA, results
// leaving through swizzled shared-memory buffers and TMA stores.
//
// One CTA per SM, 352 threads, warp-specialised:
//   warp 0      scheduler + TMA producer: draws the next ticket from a global counter,
//               publishes it to the other roles through a small ring in shared memory,
//               then streams the even k-blocks of that tile's operands
//   warp 10     second TMA producer (the odd k-blocks; CTA pairs only)
//   warp 1      MMA issuer (one lane issues tcgen05.mma / tcgen05.commit; the warp
//               owns the TMEM allocation)
//   warps 2-9   epilogue: tcgen05.ld, alpha/beta/bias/GELU/cast, store C.  Two warps per
//               TMEM lane quarter; each warp drains every other 128-byte-wide column unit of
//               its 32 rows through staging buffers of its own and issues its own TMA
//               stores, so no epilogue warp ever waits for another one.
//
// Every problem of the group is llmt's row-major  C = alpha*op(A)*op(B) + beta*C
// (llmt include/llmt/kernels/matmul.h:12-24) with its own shape, transposes, tile
// width and epilogue; tiles of all problems share one queue, longest first, so
// the tail of one problem overlaps the head of the next and e.g. the dX and dW
// products of Linear::backward (llmt src/layers/linear.cpp:22-30) run as one launch.
//
// A transposed operand is not copied: the tile is loaded as stored and described
// to the tensor core as MN-major.
//
// The fused bias gradient (dbias[i] = sum_p op(A)[i, p]; for the dW product of a linear
// layer: the column sums of dy) is part of the same launch: its reductions are extra
// tickets at the head of the queue, each 16 values of i per CTA, that the epilogue warps of
// whichever CTA draws them carry out with plain loads (dy is in L2: the dX and dW tiles of the
// launch stream it), in a fixed order, while that CTA's producer and MMA warps already work
// on the next tile.  Narrow tickets put every SM to work on them: the reduction is bound by
// the bytes one SM can keep in flight, not by arithmetic.  The tensor pipe never sees them.
//
// No wait is unbounded: every mbarrier wait gives up after GroupParams::wait_limit_ns,
// records why in the DeviceStatus word and makes the CTA drain and exit.
#include <cuda_bf16.h>

#include <type_traits>

#include "common.h"
#include "ptx_sm100.cuh"

namespace llmt_b200 {

using namespace ptx;

namespace {

constexpr int BM = 128;  // UMMA M (cta_group::1)
constexpr int BK = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 352;
constexpr int kEpilogueWarps = 8;
constexpr int kProducerHelperWarp = 10;  // second TMA producer warp
constexpr int kMaxStages = 6;
constexpr int kRing = 4;                             // scheduler ring entries
constexpr uint32_t kATileBytes = BM * BK * 2;        // 16 KB
constexpr uint32_t kStoreBufBytes = 32 * 128;        // one staging buffer: 32 rows x 128 bytes
// Per CTA and stage: the A tile plus room for the widest B tile.  A CTA pair (CG = 2)
// splits B between its two CTAs, so a stage is smaller: five of them and two staging
// buffers per epilogue warp fit where a single CTA has four stages and one buffer.
template <int CG> struct Geo {
    static constexpr uint32_t kBRegionBytes = (256 / CG) * BK * 2;
    static constexpr uint32_t kStageBytes = kATileBytes + kBRegionBytes;
    static constexpr int kStages = CG == 2 ? 5 : 4;
    static constexpr int kStoreBufs = CG == 2 ? 2 : 1;
    static constexpr uint32_t kStagingBytes = kEpilogueWarps * kStoreBufs * kStoreBufBytes;
};
constexpr uint32_t kBlock64Bytes = 64 * BK * 2;      // one 64-wide MN-major block
constexpr uint32_t kAccStride = 256;                 // TMEM columns per accumulator buffer
constexpr uint32_t kTmemCols = 512;
constexpr int kDbiasColsPerCta = 16;                 // rows of op(A) whose sums one CTA forms per dbias ticket
constexpr uint32_t kDbiasScratchBytes = kRing * kEpilogueWarps * kDbiasColsPerCta * 4;  // 2 KB

struct __align__(8) Control {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t sched_full[kRing];
    uint64_t sched_empty[kRing];
    int32_t ring[kRing];
    int32_t dbias_arrivals[kRing];  // epilogue warps that have delivered their part of a dbias ticket, per ring slot
    uint32_t tmem_base;
    int abort_flag;
};

// The template flag only marks barriers that the peer CTA of a pair also signals; those
// signals carry no generic-proxy data (ring entries arrive by st.async, operands by TMA,
// accumulators through tcgen05 fences), so the default CTA-scope acquire is enough.
template <bool CLUSTER = false>
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             DeviceStatus* st, int code, int detail, uint64_t limit_ns) {
    auto poll = [&]() { return mbar_try_wait(bar, parity); };
    if (poll()) return true;
    // The wall clock is slow to read: it is first looked at after 256 failed polls, so a wait
    // of ordinary length never touches it.
    uint64_t t0 = 0;
    uint32_t spins = 0;
    for (;;) {
        if (poll()) return true;
        if ((++spins & 255u) == 0u) {
            if (*abort_flag) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > limit_ns) {
                if (atomicCAS(&st->code, 0, code) == 0) {
                    st->detail = detail;
                    st->block = static_cast<int32_t>(blockIdx.x);
                }
                *abort_flag = 1;
                return false;
            }
        }
    }
}

struct TileCoord {
    int prob;
    int m_tile, n_tile, split, batch;
    int kb0, kb1;
};

__device__ __forceinline__ TileCoord decode_tile(const GroupParams& gp, int t) {
    TileCoord tc;
    int pi = 0;
#pragma unroll 1
    for (int i = 1; i < gp.num_problems; ++i)
        if (t >= gp.prob[i].tile_begin) pi = i;
    const GroupProblem& p = gp.prob[pi];
    tc.prob = pi;
    int r = t - p.tile_begin;
    tc.m_tile = r % p.tiles_m;
    r /= p.tiles_m;
    tc.n_tile = r % p.tiles_n;
    r /= p.tiles_n;
    tc.split = r % p.splits;
    tc.batch = r / p.splits;
    tc.kb0 = tc.split * p.kblocks_per_split;
    tc.kb1 = min(tc.kb0 + p.kblocks_per_split, p.kblocks_total);
    return tc;
}

__device__ __forceinline__ void store_chunk_f32(float* dst, const float* v, int valid) {
    if (valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0u) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < valid) dst[j] = v[j];
    }
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void store_chunk_bf16(__nv_bfloat16* dst, const float* v, int valid) {
    if (valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0u) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            uint4 u;
            u.x = pack_bf16(v[j + 0], v[j + 1]);
            u.y = pack_bf16(v[j + 2], v[j + 3]);
            u.z = pack_bf16(v[j + 4], v[j + 5]);
            u.w = pack_bf16(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(dst + j) = u;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < valid) dst[j] = __float2bfloat16_rn(v[j]);
    }
}

__device__ __forceinline__ void load_chunk_f32(const float* src, float* dst, int valid) {
    if (valid >= 32 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0u) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
            const float4 t = *reinterpret_cast<const float4*>(src + j);
            dst[j] = t.x; dst[j + 1] = t.y; dst[j + 2] = t.z; dst[j + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[j] = j < valid ? src[j] : 0.0f;
    }
}

__device__ __forceinline__ void load_chunk_bf16(const __nv_bfloat16* src, float* dst, int valid) {
    if (valid >= 32 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0u) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            const uint4 u = *reinterpret_cast<const uint4*>(src + j);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                dst[j + 2 * q] = __uint_as_float(w[q] << 16);
                dst[j + 2 * q + 1] = __uint_as_float(w[q] & 0xFFFF0000u);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) dst[j] = j < valid ? __bfloat162float(src[j]) : 0.0f;
    }
}

// 16 bytes of an operand that this kernel only reads.
__device__ __forceinline__ uint4 ld_operand16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void add_bf16x8(float* acc, const uint4& u) {
    acc[0] += __uint_as_float(u.x << 16); acc[1] += __uint_as_float(u.x & 0xFFFF0000u);
    acc[2] += __uint_as_float(u.y << 16); acc[3] += __uint_as_float(u.y & 0xFFFF0000u);
    acc[4] += __uint_as_float(u.z << 16); acc[5] += __uint_as_float(u.z & 0xFFFF0000u);
    acc[6] += __uint_as_float(u.w << 16); acc[7] += __uint_as_float(u.w & 0xFFFF0000u);
}
// Sum over the 32 lanes in a fixed tree (the same on every run and every machine).
__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One dbias ticket as one of the eight epilogue warps (ew = 0..7) of a CTA sees it:
// dbias[i] (+)= sum over p in this split's k range of op(A)[i, p] for the kDbiasColsPerCta
// values of i starting at i0.  The order of the additions depends only on the problem's
// shape.  `scratch` (8 x 16 floats) and `arrivals` belong to the ring slot the ticket came in.
__device__ __noinline__ void dbias_ticket_warp(const GroupProblem& p, int64_t i0, int split, int ew, int lane,
                                               float* scratch, int32_t* arrivals) {
    if (i0 >= p.m) return;  // CTA-uniform: all eight warps skip together
    const int64_t kbeg = static_cast<int64_t>(split) * p.kblocks_per_split * BK;
    int64_t kend = kbeg + static_cast<int64_t>(p.kblocks_per_split) * BK;
    if (kend > p.k) kend = p.k;
    const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(p.a_raw);
    if (p.a_mn) {
        // A is stored [k, m]: the sums run down columns i0 .. i0+15 (32 bytes of every row).
        // The eight warps share the rows: warp w, lane L reads 16 bytes (columns i0 + 8 (L & 1) ..)
        // of rows kbeg + 16 w + L / 2, + 128, ...; sixteen rows in flight per lane.  A warp then
        // folds its sixteen row-lanes in a fixed tree and leaves 16 partial sums in shared memory;
        // the warp that arrives last adds the eight partial sums of every column in warp order.
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
        const int64_t c = i0 + 8 * (lane & 1);
        if (c < p.m) {  // the row pitch covers whole groups of 8 columns
            const __nv_bfloat16* col = A + c;
            int64_t r = kbeg + 16 * ew + (lane >> 1);
            for (; r + 15 * 128 < kend; r += 16 * 128) {
                uint4 q[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) q[u] = ld_operand16(col + (r + 128 * u) * p.lda);
#pragma unroll
                for (int u = 0; u < 16; ++u) add_bf16x8(acc, q[u]);
            }
            for (; r < kend; r += 128) add_bf16x8(acc, ld_operand16(col + r * p.lda));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int o = 16; o > 1; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
        }
        if (lane < 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) scratch[ew * kDbiasColsPerCta + 8 * lane + j] = acc[j];
        }
        __syncwarp();
        int last = 0;
        if (lane == 0) {
            __threadfence_block();
            last = (atomicAdd(arrivals, 1) & (kEpilogueWarps - 1)) == kEpilogueWarps - 1;
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (!last) return;
        __threadfence_block();
        const int64_t i = i0 + lane;
        if (lane < kDbiasColsPerCta && i < p.m) {
            const volatile float* sc = scratch;
            float out = 0.0f;
#pragma unroll
            for (int w = 0; w < kEpilogueWarps; ++w) out += sc[w * kDbiasColsPerCta + lane];
            if (p.splits > 1) {
                p.ws_dbias[static_cast<int64_t>(split) * p.m + i] = out;
            } else {
                const float prev = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i] : 0.0f;
                p.dbias[i] = prev + out;
            }
        }
    } else {
        // A is stored [m, k]: the sums run along rows; warp w takes rows i0 + 2 w and i0 + 2 w + 1.
        // Lane L takes the 8 elements at kbeg + 8 L, + 256, ... of a row; lane 0 also takes the
        // ragged end of the range.
        const int64_t span = kend - kbeg;
        const int64_t vec_end = kbeg + span / 8 * 8;
#pragma unroll 1
        for (int j = 0; j < 2; ++j) {
            const int64_t i = i0 + 2 * ew + j;
            if (i >= p.m) break;  // warp-uniform
            const __nv_bfloat16* row = A + i * p.lda;
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
            int64_t q = kbeg + 8 * lane;
            for (; q + 3 * 256 < vec_end; q += 4 * 256) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = ld_operand16(row + q + 256 * u);
#pragma unroll
                for (int u = 0; u < 4; ++u) add_bf16x8(acc, v[u]);
            }
            for (; q < vec_end; q += 256) add_bf16x8(acc, ld_operand16(row + q));
            float t = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
            if (lane == 0)
                for (int64_t e = vec_end; e < kend; ++e) t += __bfloat162float(row[e]);
            t = lanes_sum(t);
            if (lane == 0) {
                if (p.splits > 1) {
                    p.ws_dbias[static_cast<int64_t>(split) * p.m + i] = t;
                } else {
                    const float prev = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i] : 0.0f;
                    p.dbias[i] = prev + t;
                }
            }
        }
    }
}

// tcgen05.ld fills its destination registers asynchronously until tcgen05.wait::ld.  The
// compiler must not schedule a read of them ahead of the wait: this empty statement, placed
// after the wait, makes every later use depend on it.
__device__ __forceinline__ void after_tmem_ld_wait(uint32_t (&r)[32]) {
#pragma unroll
    for (int j = 0; j < 32; j += 8)
        asm volatile("" : "+r"(r[j]), "+r"(r[j + 1]), "+r"(r[j + 2]), "+r"(r[j + 3]), "+r"(r[j + 4]), "+r"(r[j + 5]),
                          "+r"(r[j + 6]), "+r"(r[j + 7]) :: "memory");
}

template <int N> __device__ __forceinline__ void bulk_wait_group_read_n() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int CG>
__device__ __forceinline__ void tc_grouped_body(const GroupParams& gp) {
    constexpr int kStages = Geo<CG>::kStages;
    constexpr uint32_t kStageBytes = Geo<CG>::kStageBytes;
    constexpr int kStoreBufs = Geo<CG>::kStoreBufs;
    constexpr bool kPair = CG == 2;
    constexpr int kTileRows = BM * CG;  // rows of C one scheduled tile covers
    // A pair's leader (cluster rank 0) runs the scheduler and issues the MMAs for both CTAs.
    const uint32_t rank = kPair ? cluster_ctarank() : 0u;
    const bool leader = rank == 0;
    const int n_sched = static_cast<int>(gridDim.x) / CG;  // CTAs (pairs) drawing tickets
    const int sched_id = static_cast<int>(blockIdx.x) / CG;
    const uint64_t wait_ns = gp.wait_limit_ns;

    extern __shared__ uint8_t smem_raw[];
    // Layout: control block, then (1024-byte aligned, as swizzled tiles need) the operand
    // stages and the epilogue warps' staging buffers.
    Control* ctl = reinterpret_cast<Control*>(smem_raw);
    const uint32_t smem_base = (smem_u32(smem_raw) + static_cast<uint32_t>(sizeof(Control)) + 1023u) & ~1023u;
    const uint32_t staging_base = smem_base + kStages * kStageBytes;
    float* dbias_scratch = reinterpret_cast<float*>(smem_raw + (staging_base - smem_u32(smem_raw)) + Geo<CG>::kStagingBytes);
    volatile int* abort_flag = &ctl->abort_flag;
    DeviceStatus* status = gp.status;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctl->tmem_empty[a]), CG * kEpilogueWarps);      // both CTAs' epilogues
        }
        for (int r = 0; r < kRing; ++r) {
            mbar_init(smem_u32(&ctl->sched_full[r]), 1);
            mbar_init(smem_u32(&ctl->sched_empty[r]), kPair ? 2 * (2 + kEpilogueWarps) : 1 + kEpilogueWarps);  // every ring reader
        }
        for (int r = 0; r < kRing; ++r) ctl->dbias_arrivals[r] = 0;
        ctl->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc_cg<CG>(smem_u32(&ctl->tmem_base), kTmemCols);
        tmem_relinquish_cg<CG>();
    }
    tc_fence_before_thread_sync();
    __syncthreads();
    if (kPair) cluster_sync_all();  // the peer's barriers exist before anything is sent to them
    tc_fence_after_thread_sync();
    const uint32_t tmem_base = ctl->tmem_base;
    // Still independent of the previous kernel in the stream: the first ticket (this
    // launch's counter was re-armed by the launch that used it 64 launches ago) and the tensor
    // maps, which the host encoded.
    int first_ticket = 0;
    if (warp == 0 && leader) {
        if (lane == 0) first_ticket = gp.static_schedule == 0 ? atomicAdd(gp.sched_counter, 1) : sched_id;
        else if (lane <= 3 * gp.num_problems && lane <= 24) {
            const GroupProblem& q = gp.prob[(lane - 1) / 3];
            const int which = (lane - 1) % 3;
            if (which < 2 || q.c_tma) prefetch_tensormap(which == 0 ? &q.map_a : which == 1 ? &q.map_b : &q.map_c);
        }
    } else if (warp == 0 && lane >= 1 && lane <= 2 * gp.num_problems && lane <= 16) {
        const GroupProblem& q = gp.prob[(lane - 1) / 2];
        prefetch_tensormap((lane - 1) % 2 == 0 ? &q.map_a : &q.map_b);
    }
    // Everything above touched only this CTA's own state, so it may overlap the tail of the
    // previous kernel in the stream; nothing below may start before that kernel is done.
    grid_launch_dependents();
    grid_dependency_wait();

    // Barriers that live in the leader CTA of a pair, as cluster addresses usable from both.
    auto on_leader = [&](const void* bar) { return kPair ? mapa_shared(smem_u32(bar), 0u) : smem_u32(bar); };
    // A ring reader releases its slot to the scheduler (the leader's barrier).
    auto release_ring_slot = [&](int slot) {
        if (kPair) mbar_arrive_cluster(on_leader(&ctl->sched_empty[slot]));
        else mbar_arrive(smem_u32(&ctl->sched_empty[slot]));
    };

    if (warp == 0 || (kPair && warp == kProducerHelperWarp)) {
        // ------------------------------------------- scheduler + TMA producers
        // Two producer warps share the k-blocks (even ones to warp 0, odd ones to the helper
        // warp): one iteration costs a few hundred cycles of barrier and issue latency, which
        // a single warp cannot hide and which would otherwise cap how far loads run ahead.
        // In each the whole warp walks the loop; lane 0 does the barrier bookkeeping and
        // lane L issues the L-th box of a stage, so the up to six TMA boxes of a k-block
        // (MN-major operands come in 64-wide blocks) leave in one issue slot.  Warp 0 of the
        // leader also runs the scheduler.
        const bool scheduler = warp == 0 && leader;
        // A single CTA streams 48 KB per k-block and is bound by that, not by issue latency:
        // there the helper stays idle and warp 0 takes every k-block.
        const uint32_t my_parity = warp == 0 ? 0u : 1u;
        const uint32_t parity_mask = kPair ? 1u : 0u;
        uint32_t seq = 0;  // k-blocks streamed so far by this CTA; k-block `seq` uses stage seq % kStages
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        // A ticket is drawn only when the producer is ready to stream that tile (the first one
        // before the dependency wait).  Drawing one tile ahead would hide the atomic's round trip,
        // but every CTA busy with a long tile would then sit on a short one that idle CTAs could
        // have taken (measured on the QKV backward: the dX CTAs idle from 35 us of an 84 us launch).
        // The operand stages already in shared memory cover the round trip instead.
        const bool dynamic = gp.static_schedule == 0;
        int prev_ticket = 0;
        for (int it = 0; ok; ++it) {
            const int slot = it % kRing;
            const uint32_t sphase = static_cast<uint32_t>(it / kRing) & 1u;
            int t = -1;
            if (lane == 0) {
                if (scheduler) {
                    ok = bounded_wait<kPair>(smem_u32(&ctl->sched_empty[slot]), sphase ^ 1u, abort_flag, status,
                                             kDevWaitSched, slot, wait_ns);
                    if (ok) {
                        t = it == 0 ? first_ticket
                                    : (dynamic ? atomicAdd(gp.sched_counter, 1) : prev_ticket + n_sched);
                        prev_ticket = t;
                        if (t >= gp.total_tiles) {
                            // Every drawer takes exactly one out-of-range ticket; the last re-arms the counter.
                            if (dynamic && t == gp.total_tiles + n_sched - 1) *gp.sched_counter = 0;
                            t = -1;
                        }
                        ctl->ring[slot] = t;
                        mbar_arrive(smem_u32(&ctl->sched_full[slot]));
                        // The peer's copy travels as an async store that completes its barrier.
                        if (kPair)
                            st_async_cluster_u32(mapa_shared(smem_u32(&ctl->ring[slot]), 1u), static_cast<uint32_t>(t),
                                                 mapa_shared(smem_u32(&ctl->sched_full[slot]), 1u));
                    }
                } else {
                    // In the peer CTA warp 0 arms the ring barrier for the leader's 4-byte store.
                    if (kPair && warp == 0) mbar_arrive_expect_tx(smem_u32(&ctl->sched_full[slot]), 4u);
                    ok = bounded_wait<kPair>(smem_u32(&ctl->sched_full[slot]), sphase, abort_flag, status,
                                             kDevWaitSched, 48 + slot, wait_ns);
                    if (ok) {
                        t = ctl->ring[slot];
                        release_ring_slot(slot);
                    }
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            t = __shfl_sync(0xffffffffu, t, 0);
            if (!ok || t < 0) break;
            if (t < gp.colsum_total) continue;  // a dbias ticket: work for the epilogue warps only
            const TileCoord tc = decode_tile(gp, t);
            const GroupProblem& p = gp.prob[tc.prob];
            const int bn = p.bn, a_mn = p.a_mn, b_mn = p.b_mn;
            const int bn_cta = bn / CG;                         // B columns this CTA stages
            const int m0 = tc.m_tile * kTileRows + static_cast<int>(rank) * BM;
            const int n0 = tc.n_tile * bn + static_cast<int>(rank) * bn_cta;
            const uint32_t tx = kATileBytes + static_cast<uint32_t>(bn_cta) * (BK * 2);
            // This lane's box: destination offset inside the stage, tensor map, and the
            // coordinates (the k coordinate advances with the k-block).
            const int n_a = a_mn ? 2 : 1, n_b = b_mn ? (bn_cta >> 6) : 1;
            const CUtensorMap* my_map = nullptr;
            uint32_t my_off = 0;
            int my_x = 0, my_y = 0;
            bool k_is_x = false, k_is_y = false;
            if (lane < n_a) {
                my_map = &p.map_a;
                if (a_mn) { my_off = lane * kBlock64Bytes; my_x = m0 + 64 * lane; k_is_y = true; }
                else      { my_y = m0; k_is_x = true; }
            } else if (lane < n_a + n_b) {
                const int j = lane - n_a;
                my_map = &p.map_b;
                my_off = kATileBytes;
                if (b_mn) { my_off += j * kBlock64Bytes; my_x = n0 + 64 * j; k_is_y = true; }
                else      { my_y = n0; k_is_x = true; }
            }
            for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++seq) {
                if ((seq & parity_mask) == my_parity) {
                    if (lane == 0) {
                        ok = bounded_wait<kPair>(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag, status,
                                                 kDevWaitSmemEmpty, stage, wait_ns);
                        // The leader's barrier counts the bytes of both CTAs of a pair.
                        if (ok && leader) mbar_arrive_expect_tx(smem_u32(&ctl->full[stage]), tx * CG);
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    if (my_map != nullptr) {
                        const int k0 = kb * BK;
                        const uint32_t dst = smem_base + static_cast<uint32_t>(stage) * kStageBytes + my_off;
                        const int x = my_x + (k_is_x ? k0 : 0), y = my_y + (k_is_y ? k0 : 0);
                        if (kPair) tma_load_3d_pair(dst, my_map, on_leader(&ctl->full[stage]), x, y, tc.batch);
                        else tma_load_3d(dst, my_map, smem_u32(&ctl->full[stage]), x, y, tc.batch);
                    }
                }
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0 && leader) {
            // Shared-memory descriptor, 128-byte swizzle: K-major = k-step 32 bytes along the
            // row, LBO unused (16), SBO 1024; MN-major = k-step 16 k-rows of 128 bytes, LBO =
            // one 64-wide block, SBO 1024.  Only the 14-bit start-address field changes between
            // k-steps and stages, so the issuing thread does one add per operand.
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            int stage = 0;
            uint32_t phase = 0;
            // Accumulator slot q lives in TMEM buffer q & 1 and is on its (q >> 1)-th use.
            uint32_t acc_seq = 0;
            bool ok = true;
            for (int it = 0; ok; ++it) {
                const int slot = it % kRing;
                const uint32_t sphase = static_cast<uint32_t>(it / kRing) & 1u;
                ok = bounded_wait(smem_u32(&ctl->sched_full[slot]), sphase, abort_flag, status,
                                  kDevWaitSched, 16 + slot, wait_ns);
                if (!ok) break;
                const int t = ctl->ring[slot];
                release_ring_slot(slot);
                if (t < 0) break;
                if (t < gp.colsum_total) continue;
                const TileCoord tc = decode_tile(gp, t);
                const GroupProblem& p = gp.prob[tc.prob];
                const uint32_t idesc = make_idesc_bf16(kTileRows, p.bn, p.a_mn, p.b_mn);
                const uint32_t step_a = (p.a_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
                const uint32_t step_b = (p.b_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
                const uint32_t a_lo_base = (smem_base >> 4) | (((p.a_mn ? kBlock64Bytes : 16u) >> 4) << 16);
                const uint32_t b_lo_base = ((smem_base + kATileBytes) >> 4) |
                                           (((p.b_mn ? kBlock64Bytes : 16u) >> 4) << 16);
                const int acc = static_cast<int>(acc_seq & 1u);
                ok = bounded_wait<kPair>(smem_u32(&ctl->tmem_empty[acc]), ((acc_seq >> 1) & 1u) ^ 1u, abort_flag,
                                         status, kDevWaitTmemEmpty, acc, wait_ns);
                if (!ok) break;
                tc_fence_after_thread_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * kAccStride;
                for (int kb = tc.kb0; kb < tc.kb1; ++kb) {
                    ok = bounded_wait<kPair>(smem_u32(&ctl->full[stage]), phase, abort_flag, status,
                                             kDevWaitSmemFull, stage, wait_ns);
                    if (!ok) break;
                    tc_fence_after_thread_sync();
                    const uint32_t stage_off = static_cast<uint32_t>(stage) * (kStageBytes >> 4);
                    const uint32_t a_lo = a_lo_base + stage_off;
                    const uint32_t b_lo = b_lo_base + stage_off;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t da = (static_cast<uint64_t>(kDescHi) << 32) |
                                            static_cast<uint64_t>(a_lo + kk * step_a);
                        const uint64_t db = (static_cast<uint64_t>(kDescHi) << 32) |
                                            static_cast<uint64_t>(b_lo + kk * step_b);
                        umma_bf16_cg<CG>(d_tmem, da, db, idesc, (kb > tc.kb0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit_cg<CG>(smem_u32(&ctl->empty[stage]));  // frees the stage when the MMAs retire
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit_cg<CG>(smem_u32(&ctl->tmem_full[acc]));
                ++acc_seq;
            }
        }
    } else if (warp < 2 + kEpilogueWarps) {
        // ---------------------------------------------------------- epilogue
        const int quarter = warp & 3;        // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
        const int half = (warp - 2) >> 2;    // this warp takes the column units u with u % 2 == half
        const int ew = warp - 2;             // 0..7
        const uint32_t my_bufs = staging_base + static_cast<uint32_t>(ew * kStoreBufs) * kStoreBufBytes;
        uint32_t buf_seq = 0;  // TMA stores this warp has issued so far
        uint32_t acc_seq = 0;  // accumulator slot counter, in step with the MMA issuer's
        bool ok = true;
        for (int it = 0; ok; ++it) {
            const int slot = it % kRing;
            const uint32_t sphase = static_cast<uint32_t>(it / kRing) & 1u;
            ok = bounded_wait<kPair>(smem_u32(&ctl->sched_full[slot]), sphase, abort_flag, status,
                                     kDevWaitSched, 32 + slot, wait_ns);
            if (!ok) break;
            const int t = ctl->ring[slot];
            __syncwarp();
            if (t >= 0 && t < gp.colsum_total) {
                // A dbias ticket: (block of rows of op(A), split) of the problem that owns it.  The
                // ring slot is released only afterwards: its scratch area is in use until then.
                int pi = 0;
#pragma unroll 1
                for (int i = 0; i < gp.num_problems; ++i)
                    if (gp.prob[i].colsum_tiles > 0 && t >= gp.prob[i].colsum_begin) pi = i;
                const GroupProblem& p = gp.prob[pi];
                const int r = t - p.colsum_begin;
                const int blk = r % p.colsum_blocks, split = r / p.colsum_blocks;
                dbias_ticket_warp(p, (static_cast<int64_t>(blk) * CG + rank) * kDbiasColsPerCta, split, ew, lane,
                                  dbias_scratch + slot * (kEpilogueWarps * kDbiasColsPerCta), &ctl->dbias_arrivals[slot]);
                __syncwarp();
                if (lane == 0) release_ring_slot(slot);
                continue;
            }
            if (lane == 0) release_ring_slot(slot);
            if (t < 0) break;
            const TileCoord tc = decode_tile(gp, t);
            const GroupProblem& p = gp.prob[tc.prob];
            const int acc = static_cast<int>(acc_seq & 1u);
            const int row0 = tc.m_tile * kTileRows + static_cast<int>(rank) * BM + quarter * 32;  // this warp's first row
            const int64_t row = static_cast<int64_t>(row0) + lane;
            const bool row_ok = row < p.m;
            const int64_t n0 = static_cast<int64_t>(tc.n_tile) * p.bn;
            const bool partial = p.splits > 1;
            const bool out_bf16 = !partial && p.c_is_bf16;
            // A column unit is what one TMA store carries: 32 rows x 128 bytes.
            const int unit_cols = out_bf16 ? 64 : 32;
            const int spu = out_bf16 ? 2 : 1;  // 32-column steps (one tcgen05.ld each) per unit
            const bool tma_ok = partial ? p.ws_tma != 0 : p.c_tma != 0;
            const CUtensorMap* out_map = partial ? &p.map_ws : &p.map_c;
            const int out_z = partial ? tc.batch * p.splits + tc.split : tc.batch;
            // Column (inside the tile) of this warp's s-th step.
            auto step_col = [&](int s) { return (half + 2 * (s / spu)) * unit_cols + (s % spu) * 32; };
            int ns = ((p.bn / unit_cols + 1 - half) / 2) * spu;
            while (ns > 0 && n0 + step_col(ns - 1) >= p.n) --ns;
            if (row0 >= p.m) ns = 0;  // the whole warp lies below the matrix
            if (p.beta != 0.0f && !partial && row_ok) {
                // beta * C_in is read row by row (one row per thread): ask L2 for this thread's
                // lines now, while the tile's main loop is still running.
                const int esz = p.c_is_bf16 ? 2 : 4;
                const char* base = static_cast<const char*>(p.c) +
                                   (static_cast<int64_t>(tc.batch) * p.stride_c + row * p.ldc + n0) * esz;
                for (int s = 0; s < ns; s += spu)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(base + static_cast<int64_t>(step_col(s)) * esz));
            }
            ok = bounded_wait(smem_u32(&ctl->tmem_full[acc]), (acc_seq >> 1) & 1u, abort_flag, status,
                              kDevWaitTmemFull, acc, wait_ns);
            if (!ok) break;
            tc_fence_after_thread_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc) * kAccStride;
            // The accumulator goes back to the MMA issuer (in the leader CTA) as soon as this
            // warp's last tcgen05.ld has completed.
            auto release_acc = [&]() {
                tc_fence_before_thread_sync();
                __syncwarp();
                if (lane == 0) {
                    if (kPair) mbar_arrive_cluster(on_leader(&ctl->tmem_empty[acc]));
                    else mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
                }
            };
            // One 32-column step: epilogue arithmetic on the values of this thread's row, then
            // into the staging buffer (and out by TMA once the unit is complete) or, for a
            // ragged unit or a C that TMA cannot address, straight to global memory.
            auto emit = [&](const uint32_t (&r)[32], int s) {
                const int c0 = step_col(s);
                const int64_t col = n0 + c0;
                const int valid = static_cast<int>(min(static_cast<int64_t>(32), p.n - col));
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                const int64_t c_off = static_cast<int64_t>(tc.batch) * p.stride_c + row * p.ldc + col;
                if (!partial) {
                    if (p.alpha != 1.0f) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
                    }
                    if (p.beta != 0.0f && row_ok) {
                        float cin[32];
                        if (p.c_is_bf16)
                            load_chunk_bf16(static_cast<const __nv_bfloat16*>(p.c) + c_off, cin, valid);
                        else
                            load_chunk_f32(static_cast<const float*>(p.c) + c_off, cin, valid);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = fmaf(p.beta, cin[j], v[j]);
                    }
                    if (p.epi_flags & kEpiBias) {
                        float bv[32];
                        if (p.bias_is_bf16)
                            load_chunk_bf16(static_cast<const __nv_bfloat16*>(p.bias) + col, bv, valid);
                        else
                            load_chunk_f32(static_cast<const float*>(p.bias) + col, bv, valid);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] += bv[j];
                    }
                    if (p.epi_flags & kEpiGelu) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_fast(v[j]);
                    }
                }
                const int sub = s % spu;
                const int64_t unit_col = col - sub * 32;
                if (tma_ok && unit_col + unit_cols <= p.n) {
                    const uint32_t buf = my_bufs + (buf_seq % kStoreBufs) * kStoreBufBytes;
                    if (sub == 0) {
                        // The buffer is free once the store that last read it has done so.
                        if (lane == 0) bulk_wait_group_read_n<kStoreBufs - 1>();
                        __syncwarp();
                    }
                    const uint32_t row_addr = buf + static_cast<uint32_t>(lane) * 128u;
                    const uint32_t sw = static_cast<uint32_t>(lane) & 7u;
                    if (out_bf16) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(row_addr + ((static_cast<uint32_t>(sub * 4 + q) ^ sw) << 4)),
                                           "r"(pack_bf16(v[8 * q + 0], v[8 * q + 1])),
                                           "r"(pack_bf16(v[8 * q + 2], v[8 * q + 3])),
                                           "r"(pack_bf16(v[8 * q + 4], v[8 * q + 5])),
                                           "r"(pack_bf16(v[8 * q + 6], v[8 * q + 7])) : "memory");
                    } else {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(row_addr + ((static_cast<uint32_t>(q) ^ sw) << 4)),
                                           "r"(__float_as_uint(v[4 * q + 0])), "r"(__float_as_uint(v[4 * q + 1])),
                                           "r"(__float_as_uint(v[4 * q + 2])), "r"(__float_as_uint(v[4 * q + 3]))
                                         : "memory");
                    }
                    if (sub == spu - 1) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(out_map, buf, static_cast<int32_t>(unit_col), row0, out_z);
                            bulk_commit_group();
                        }
                        ++buf_seq;
                    }
                } else if (row_ok) {
                    if (partial) {
                        float* dst = p.ws +
                                     ((static_cast<int64_t>(tc.batch) * p.splits + tc.split) * p.m + row) * p.n + col;
                        store_chunk_f32(dst, v, valid);
                    } else if (p.c_is_bf16) {
                        store_chunk_bf16(static_cast<__nv_bfloat16*>(p.c) + c_off, v, valid);
                    } else {
                        store_chunk_f32(static_cast<float*>(p.c) + c_off, v, valid);
                    }
                }
            };
            // Software pipeline over the steps: the tcgen05.ld of step s+1 is in flight while
            // step s is converted and staged.
            if (ns == 0) {
                release_acc();
            } else {
                uint32_t ra[32], rb[32];
                tmem_ld_32x32(t_row + static_cast<uint32_t>(step_col(0)), ra);
#pragma unroll 1
                for (int s = 0; s < ns; s += 2) {
                    tmem_ld_wait();
                    after_tmem_ld_wait(ra);
                    if (s + 1 < ns) tmem_ld_32x32(t_row + static_cast<uint32_t>(step_col(s + 1)), rb);
                    else release_acc();
                    emit(ra, s);
                    if (s + 1 < ns) {
                        tmem_ld_wait();
                        after_tmem_ld_wait(rb);
                        if (s + 2 < ns) tmem_ld_32x32(t_row + static_cast<uint32_t>(step_col(s + 2)), ra);
                        else release_acc();
                        emit(rb, s + 1);
                    }
                }
            }
            ++acc_seq;
        }
        // Outstanding TMA stores must complete before the shared memory goes away.
        if (lane == 0) bulk_wait_group0();
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag) {
        // A wait ran out somewhere: give copies still in flight time to land
        // before the shared memory and TMEM are released.
        __nanosleep(200000);
    }
    tc_fence_before_thread_sync();
    __syncthreads();
    // Neither CTA of a pair may leave while the other can still signal its barriers,
    // read its operand tiles or use the pair's TMEM allocation.
    if (kPair) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_thread_sync();
        tmem_dealloc_cg<CG>(tmem_base, kTmemCols);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
tc_grouped_kernel(const __grid_constant__ GroupParams gp) {
    tc_grouped_body<1>(gp);
}

// The same kernel over CTA pairs: clusters of two CTAs, each pair computing 256-row tiles
// with cta_group::2 MMAs, every CTA staging its own 128 rows of A and half of the B tile.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
tc_grouped_pair_kernel(const __grid_constant__ GroupParams gp) {
    tc_grouped_body<2>(gp);
}

// C = epilogue(alpha * sum_s ws[s] + beta * C): fixed summation order s = 0..splits-1.
// Four consecutive columns per thread when the row length allows it.
__global__ void splitk_reduce_kernel(const GroupProblem p) {
    grid_launch_dependents();
    grid_dependency_wait();
    const int64_t n4 = (p.n + 3) / 4;
    const int64_t total4 = static_cast<int64_t>(p.batch) * p.m * n4;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < total4) {
        const int64_t col = (i % n4) * 4;
        const int64_t row = (i / n4) % p.m;
        const int64_t b = i / (n4 * p.m);
        const int cnt = static_cast<int>(min(static_cast<int64_t>(4), p.n - col));
        const float* src = p.ws + (b * p.splits * p.m + row) * p.n + col;
        const int64_t sstride = p.m * p.n;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (cnt == 4 && ((reinterpret_cast<uintptr_t>(src) | (static_cast<uintptr_t>(sstride) * 4u)) & 15u) == 0u) {
            for (int s = 0; s < p.splits; ++s) {
                const float4 t = *reinterpret_cast<const float4*>(src + s * sstride);
                acc[0] += t.x; acc[1] += t.y; acc[2] += t.z; acc[3] += t.w;
            }
        } else {
            for (int s = 0; s < p.splits; ++s)
                for (int j = 0; j < cnt; ++j) acc[j] += src[s * sstride + j];
        }
        const int64_t c_off = b * p.stride_c + row * p.ldc + col;
        for (int j = 0; j < cnt; ++j) {
            float v = p.alpha * acc[j];
            if (p.beta != 0.0f)
                v += p.beta * (p.c_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.c)[c_off + j])
                                           : static_cast<const float*>(p.c)[c_off + j]);
            if (p.epi_flags & kEpiBias)
                v += p.bias_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col + j])
                                    : static_cast<const float*>(p.bias)[col + j];
            if (p.epi_flags & kEpiGelu) v = gelu_tanh_fast(v);
            if (p.c_is_bf16)
                static_cast<__nv_bfloat16*>(p.c)[c_off + j] = __float2bfloat16_rn(v);
            else
                static_cast<float*>(p.c)[c_off + j] = v;
        }
    }
    if (p.dbias != nullptr && i < p.m) {
        float acc = 0.0f;
        for (int s = 0; s < p.splits; ++s) acc += p.ws_dbias[static_cast<int64_t>(s) * p.m + i];
        const float prev = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i] : 0.0f;
        p.dbias[i] = prev + acc;
    }
}

}  // namespace

size_t tc_grouped_smem_bytes() {
    // Both geometries use the same amount: 4 x 48 KB of operand stages + 32 KB of staging,
    // or 5 x 32 KB + 64 KB; then 2 KB for the dbias tickets.  227 KB in all.
    static_assert(Geo<1>::kStages * Geo<1>::kStageBytes + Geo<1>::kStagingBytes ==
                  Geo<2>::kStages * Geo<2>::kStageBytes + Geo<2>::kStagingBytes, "shared-memory budget");
    static_assert(sizeof(Control) <= 1024, "control block must fit below the first aligned KB");
    return 1024 /* control block + alignment */ + Geo<1>::kStages * Geo<1>::kStageBytes + Geo<1>::kStagingBytes +
           kDbiasScratchBytes;
}

int tc_dbias_rows_per_cta() { return kDbiasColsPerCta; }

// Per-device record of what has been configured (cudaFuncSetAttribute is per device).
static bool g_configured[64];

static cudaError_t configure_device(int dev) {
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (g_configured[dev]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(tc_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tc_grouped_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess) g_configured[dev] = true;
    return e;
}

cudaError_t launch_tc_grouped(const GroupParams& gp, int grid, bool pairs, cudaStream_t stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = configure_device(dev);
    if (e != cudaSuccess) return e;
    // Programmatic dependent launch: the kernel's prologue (barriers, TMEM) overlaps the tail
    // of the previous kernel in the stream; the kernel itself waits before touching memory.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = tc_grouped_smem_bytes();
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = pairs ? cudaLaunchKernelEx(&cfg, tc_grouped_pair_kernel, gp)
              : cudaLaunchKernelEx(&cfg, tc_grouped_kernel, gp);
    count_launch(1);
    return e != cudaSuccess ? e : cudaGetLastError();
}

// How many CTA pairs can be resident at once on the current device (1 CTA per SM, pairs
// share a cluster); -1 when the query fails.
int max_resident_pairs() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
    if (cached[dev] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2, 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = tc_grouped_smem_bytes();
        int n = 0;
        if (configure_device(dev) == cudaSuccess &&
            cudaOccupancyMaxActiveClusters(&n, tc_grouped_pair_kernel, &cfg) == cudaSuccess && n > 0)
            cached[dev] = n;
        else
            cached[dev] = -1;
    }
    return cached[dev];
}

cudaError_t launch_splitk_reduce(const GroupProblem& p, cudaStream_t stream) {
    const int64_t n4 = (p.n + 3) / 4;
    const int64_t total = static_cast<int64_t>(p.batch) * p.m * n4;
    const int64_t work = total > p.m ? total : p.m;
    const int block = 256;
    const int64_t grid = (work + block - 1) / block;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, p);
    count_launch(1);
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace llmt_b200
