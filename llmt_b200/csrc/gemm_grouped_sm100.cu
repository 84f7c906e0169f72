// bf16 x bf16 -> fp32-accumulate GEMM for sm_100a as ONE persistent kernel over
// a list of problems ("group"): tcgen05 MMA with the accumulator in tensor
// memory, operands staged in 128-byte-swizzled shared memory by TMA, results
// leaving through swizzled shared-memory buffers and TMA stores.
//
// One CTA per SM, 384 threads, warp-specialised:
//   warp 0      scheduler + TMA producer: draws the next ticket from a global counter,
//               publishes it to the other roles through a small ring in shared memory,
//               then streams the even k-blocks of that tile's operands
//   warp 10     helper TMA producer (CTA pairs only): the two producer warps take the k-blocks
//               in turn
//   warp 11     side warp: when the launch carries a gradient exchange (see RideExchange), it
//               sums chunks of that range over the ranks through the NVSwitch while the other
//               warps run the launch's tiles; idle otherwise
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
// layer: the column sums of dy) is part of the same launch, as extra tickets that only the
// epilogue warps of whichever CTA draws them work on, with plain loads, while that CTA's
// producer and MMA warps go straight on to the next tile; the tensor pipe never sees them.
// For A stored [k, m] (the dW case) the reduction runs in two phases, both in a fixed order:
// tickets at the head of the queue each sum a chunk of rows of A over ALL columns (whole rows,
// so every load instruction reads 512 contiguous bytes and every byte of dy is read once) into
// a row of partial sums in the workspace; tickets at the tail of the queue, drawn by the CTAs
// that run out of tiles first, add the partial sums in chunk order.  The tail tickets wait
// (bounded) on a counter of finished head tickets; the wait can never block progress, since
// head tickets are drawn first and wait for nothing.
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
constexpr int kThreads = 384;
constexpr int kEpilogueWarps = 8;
constexpr int kProducerHelperWarp = 10;  // first of the helper TMA producer warps (CTA pairs only)
constexpr int kProducerHelpers = 1;
constexpr int kSideWarp = 11;            // works on the exchange that rides along, nothing else
constexpr int kMaxStages = 6;
constexpr int kRing = 4;                             // scheduler ring entries
constexpr uint32_t kATileBytes = BM * BK * 2;        // 16 KB
constexpr uint32_t kStoreBufBytes = 32 * 128;        // one staging buffer: 32 rows x 128 bytes
// Per CTA and stage: the A tile plus room for the widest B tile.  A CTA pair (CG = 2)
// splits B between its two CTAs, so a stage is smaller: six of them fit where a single CTA
// has four.  The main loop is bound by the bytes in flight: a stage is refilled about 1.7 us
// after its MMAs retire (commit -> producer -> TMA -> L2 -> shared memory -> MMA issuer), and a
// pair consumes 32 KB per CTA every 0.3 us, so anything below ~180 KB of stages starves the
// tensor pipe (measured with five stages: 0.34-0.43 us per k-block).
#ifndef LLMT_B200_PAIR_STAGES
#define LLMT_B200_PAIR_STAGES 6
#endif
// 16-byte sums one lane of a side warp keeps in flight.  More is slower, not faster: at 16 the
// exchange's requests crowd the GEMM's own loads out of the memory system (two GPUs, GPT-2 step:
// 0.427 ms at 8, 0.435 at 4, 0.453 at 16, 0.550 at 32).
#ifndef LLMT_B200_RIDE_UNROLL
#define LLMT_B200_RIDE_UNROLL 8
#endif
#ifndef LLMT_B200_PAIR_STORE_BUFS
#define LLMT_B200_PAIR_STORE_BUFS 1
#endif
template <int CG> struct Geo {
    static constexpr uint32_t kBRegionBytes = (256 / CG) * BK * 2;
    static constexpr uint32_t kStageBytes = kATileBytes + kBRegionBytes;
    static constexpr int kStages = CG == 2 ? LLMT_B200_PAIR_STAGES : 4;
    static constexpr int kStoreBufs = CG == 2 ? LLMT_B200_PAIR_STORE_BUFS : 1;   // staging buffers per epilogue warp
    static constexpr uint32_t kStagingBytes = kEpilogueWarps * kStoreBufs * kStoreBufBytes;
    static constexpr uint32_t kScalarBytes = kMaxGroupProblems * static_cast<uint32_t>(sizeof(ProblemScalars));
    static constexpr uint32_t kSmemBytes = 1024 /* control block + alignment */ + kStages * kStageBytes + kStagingBytes + kScalarBytes;
};
static_assert(Geo<1>::kSmemBytes <= 227 * 1024 && Geo<2>::kSmemBytes <= 227 * 1024, "shared-memory budget");
constexpr uint32_t kBlock64Bytes = 64 * BK * 2;      // one 64-wide MN-major block
constexpr uint32_t kAccStride = 256;                 // TMEM columns per accumulator buffer
constexpr uint32_t kTmemCols = 512;
constexpr int kDbiasRowsPerCta = 16;                 // mode 2: rows of op(A) one CTA sums per dbias ticket
constexpr int kDbiasFinishPerCta = 256;              // mode 1: values of i one CTA finishes per ticket

// A ticket as the scheduler publishes it: already decoded, so that the warps that read it
// (producers, MMA issuer, epilogue) go from one tile to the next on a few shared-memory reads.
// The decode runs once, in the scheduler, ahead of need.
struct __align__(16) TileCoord {
    int t;                 // the ticket; -1: no more work
    int prob;
    int kb0, kb1;
    int m_tile, n_tile;
    int bz, bw;            // the batch item as (index inside its group, group): (batch, 0) for a plain batch
    int split, batch;
    int pad0, pad1;
};
static_assert(sizeof(TileCoord) == 48, "three 16-byte words");

struct __align__(16) Control {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t landed[kMaxStages];   // peer CTA of a pair: "this stage's operands are in" (the full barrier lives in the leader)
    uint64_t sum_bar[2];           // the epilogue warps among themselves, around the cross-warp dbias sum
    uint64_t sched_full[kRing];
    uint64_t sched_empty[kRing];
    TileCoord ring[kRing];
    uint4 mma_consts[kMaxGroupProblems];    // per problem: instruction descriptor, operand descriptor bases, k-steps
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


// n / d with the reciprocal of d at hand.  One thread of the MMA warp decodes a ticket between
// two tiles, where a hardware-emulated integer division (a long dependent chain) is exposed:
// below 2^24 the float product is within one of the quotient and two compares fix it.
__device__ __forceinline__ uint32_t div_by(uint32_t n, uint32_t d, float inv_d) {
    if (n >= (1u << 24)) return n / d;
    uint32_t q = static_cast<uint32_t>(__uint2float_rz(n) * inv_d);
    const uint32_t prod = q * d;
    if (prod > n) --q;
    else if (n - prod >= d) ++q;
    return q;
}

__device__ __forceinline__ TileCoord decode_tile(const ProblemScalars* sp, int num_problems, int t) {
    TileCoord tc;
    tc.t = t;
    tc.pad0 = tc.pad1 = 0;
    int pi = 0;
#pragma unroll 1
    for (int i = 1; i < num_problems; ++i)
        if (t >= sp[i].tile_begin) pi = i;
    const ProblemScalars& p = sp[pi];
    tc.prob = pi;
    // The common cases (one split, one batch item) need one quotient only.
    const uint32_t r = static_cast<uint32_t>(t - p.tile_begin);
    const uint32_t q1 = div_by(r, static_cast<uint32_t>(p.tiles_m), p.inv_tiles_m);
    tc.m_tile = static_cast<int>(r - q1 * static_cast<uint32_t>(p.tiles_m));
    if (p.splits == 1 && p.batch <= 1) {
        tc.n_tile = static_cast<int>(q1);
        tc.split = 0;
        tc.batch = 0;
    } else {
        const uint32_t q2 = div_by(q1, static_cast<uint32_t>(p.tiles_n), p.inv_tiles_n);
        tc.n_tile = static_cast<int>(q1 - q2 * static_cast<uint32_t>(p.tiles_n));
        const uint32_t q3 = div_by(q2, static_cast<uint32_t>(p.splits), p.inv_splits);
        tc.split = static_cast<int>(q2 - q3 * static_cast<uint32_t>(p.splits));
        tc.batch = static_cast<int>(q3);
    }
    tc.bz = tc.batch;
    tc.bw = 0;
    if (p.batch_inner > 0) {
        tc.bw = static_cast<int>(div_by(static_cast<uint32_t>(tc.batch), static_cast<uint32_t>(p.batch_inner), p.inv_batch_inner));
        tc.bz = tc.batch - tc.bw * p.batch_inner;
    }
    tc.kb0 = tc.split * p.kblocks_per_split;
    tc.kb1 = min(tc.kb0 + p.kblocks_per_split, p.kblocks_total);
    return tc;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void load_chunk_f32(const float* src, float* dst, int valid) {
    if (__builtin_expect(valid >= 32 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0u, 1)) {
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
    if (__builtin_expect(valid >= 32 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0u, 1)) {
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

// One thread's 32 consecutive values of a row to global memory (the second result of an epilogue
// that has two): 16-byte stores where the row allows them.
__device__ __forceinline__ void store_chunk_bf16(__nv_bfloat16* dst, const float* v, int valid) {
    if (__builtin_expect(valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0u, 1)) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(pack_bf16(v[8 * q + 0], v[8 * q + 1]), pack_bf16(v[8 * q + 2], v[8 * q + 3]),
                                                                pack_bf16(v[8 * q + 4], v[8 * q + 5]), pack_bf16(v[8 * q + 6], v[8 * q + 7]));
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < valid) dst[j] = __float2bfloat16_rn(v[j]);
    }
}
__device__ __forceinline__ void store_chunk_f32(float* dst, const float* v, int valid) {
    if (__builtin_expect(valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0u, 1)) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(dst + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < valid) dst[j] = v[j];
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

// dbias, A stored [k, m], first phase.  Ticket j covers rows [j R, (j+1) R) of A and every
// column: warp `wid` of the `nw` warps that share the ticket takes the 256-column chunks wid,
// wid + nw, ...; lane L sums columns c + 8 L .. + 7 of the chunk down the rows (sixteen rows in
// flight) and leaves eight partial sums in row j of the workspace.
__device__ __noinline__ void dbias_partial_warp(const ProblemScalars& p, int j, int wid, int nw, int lane) {
    const int64_t r0 = static_cast<int64_t>(j) * p.dbias_rows;
    int64_t r1 = r0 + p.dbias_rows;
    if (r1 > p.k) r1 = p.k;
    const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(p.a_raw);
    float* out = p.ws_dbias + static_cast<int64_t>(j) * p.m;
    for (int64_t c = static_cast<int64_t>(wid) * 256 + 8 * lane; c - 8 * lane < p.m; c += static_cast<int64_t>(nw) * 256) {
        if (c >= p.m) continue;  // the row pitch covers whole groups of 8 columns
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        const __nv_bfloat16* col = A + c;
        int64_t r = r0;
        for (; r + 16 <= r1; r += 16) {
            uint4 q[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) q[u] = ld_operand16(col + (r + u) * p.lda);
#pragma unroll
            for (int u = 0; u < 16; ++u) add_bf16x8(acc, q[u]);
        }
        for (; r < r1; ++r) add_bf16x8(acc, ld_operand16(col + r * p.lda));
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (c + e < p.m) out[c + e] = acc[e];
    }
}

// dbias, A stored [k, m], second phase: dbias[i] = dbias_beta * dbias[i] + sum_j partial[j][i],
// j ascending, for the 32 values of i starting at i0 (one per lane).
// One value: partial sums j = 0 .. colsum_tiles-1 in that order, many loads in flight (the
// loop is a chain of L2 round trips otherwise).
__device__ __forceinline__ void dbias_finish_one(const ProblemScalars& p, int64_t i) {
    const float* src = p.ws_dbias + i;
    float acc = 0.0f;
    int j = 0;
    for (; j + 16 <= p.colsum_tiles; j += 16) {
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = __ldcg(src + static_cast<int64_t>(j + u) * p.m);  // written by other SMs: read from L2
#pragma unroll
        for (int u = 0; u < 16; ++u) acc += v[u];
    }
    for (; j < p.colsum_tiles; ++j) acc += __ldcg(src + static_cast<int64_t>(j) * p.m);
    const float prev = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i] : 0.0f;
    p.dbias[i] = prev + acc;
}
__device__ __noinline__ void dbias_finish_warp(const ProblemScalars& p, int64_t i0, int lane) {
    const int64_t i = i0 + lane;
    if (i < p.m) dbias_finish_one(p, i);
}

// dbias, A stored [m, k]: the sums run along rows, nothing to combine.  The warp takes rows
// i0 and i0 + 1; lane L takes the 8 elements at 8 L, + 256, ... of a row; lane 0 also takes
// the ragged end.
__device__ __noinline__ void dbias_rows_warp(const ProblemScalars& p, int64_t i0, int lane) {
    const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(p.a_raw);
    const int64_t vec_end = p.k / 8 * 8;
#pragma unroll 1
    for (int j = 0; j < 2; ++j) {
        const int64_t i = i0 + j;
        if (i >= p.m) break;  // warp-uniform
        const __nv_bfloat16* row = A + i * p.lda;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.0f;
        int64_t q = 8 * lane;
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
            for (int64_t e = vec_end; e < p.k; ++e) t += __bfloat162float(row[e]);
        t = lanes_sum(t);
        if (lane == 0) {
            const float prev = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i] : 0.0f;
            p.dbias[i] = prev + t;
        }
    }
}

// The exchange that rides along, as one warp per CTA sees it: this rank's share of the range is
// cut into `tiles` chunks that the side warps of all CTAs draw from a counter of their own (the
// tile queue and the warps that serve it never see them, so a slow round trip through the switch
// cannot hold up an epilogue).  A chunk is summed inside the switch (multimem.ld_reduce) and
// written into every rank's copy by it (multimem.st).  First every other rank must have
// announced that its partial sums of the range are complete; the wait is bounded.
__device__ __noinline__ void ride_exchange_side_warp(const RideExchange& x, int32_t* counter, int lane,
                                                     uint64_t wait_ns, DeviceStatus* status) {
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(x.local + kRideStep) * kMaxRidesPerStep +
                       static_cast<uint32_t>(x.index);
    int ok = 1;
    if (lane < x.world && lane != x.rank) {
        const uint32_t* f = x.local + kRideReady + lane;
        uint64_t t0 = 0;
        uint32_t spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys(f) - e) < 0) {
            if ((++spins & 31u) == 0u) {
                const uint64_t now = globaltimer_ns();
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > wait_ns) {
                    if (atomicCAS(&status->code, 0, kDevWaitPeer) == 0) {
                        status->detail = 2048 + lane;
                        status->block = static_cast<int32_t>(blockIdx.x);
                    }
                    ok = 0;
                    break;
                }
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    const int64_t shard4 = (x.n4 + x.world - 1) / x.world;
    const int64_t lo = static_cast<int64_t>(x.rank) * shard4;
    const int64_t hi = lo + shard4 < x.n4 ? lo + shard4 : x.n4;
    const int64_t chunk4 = (shard4 + x.tiles - 1) / x.tiles;
    float4* mc = reinterpret_cast<float4*>(x.mc);
    constexpr int kU = LLMT_B200_RIDE_UNROLL;  // sums of 16 bytes in flight per lane
    const int n_side = static_cast<int>(gridDim.x);
    for (;;) {
        // Every side warp draws until it gets a ticket past the end; the last such draw re-arms the counter.
        int j = 0;
        if (lane == 0) j = atomicAdd(counter, 1);
        j = __shfl_sync(0xffffffffu, j, 0);
        if (j >= x.tiles) {
            if (lane == 0 && j == x.tiles + n_side - 1) *counter = 0;
            break;
        }
        if (!ok) continue;  // gave up on a peer: the tickets are still drawn, so that the counter re-arms
        const int64_t c_lo = lo + static_cast<int64_t>(j) * chunk4;
        const int64_t c_hi = c_lo + chunk4 < hi ? c_lo + chunk4 : hi;
        int64_t i = c_lo + lane;
        for (; i + (kU - 1) * 32 < c_hi; i += kU * 32) {
            float4 v[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) v[u] = multimem_ld_reduce_add(mc + i + u * 32);
#pragma unroll
            for (int u = 0; u < kU; ++u) multimem_st(mc + i + u * 32, v[u]);
        }
        for (; i < c_hi; i += 32) multimem_st(mc + i, multimem_ld_reduce_add(mc + i));
    }
    __threadfence_system();
}

// Copies a staged unit (up to 32 rows x 128 bytes, 128-byte swizzle) to a destination that TMA
// cannot address or that is ragged: one row per store instruction (up to 128 contiguous bytes),
// eight rows in flight.  `dst` is the unit's first element, `ld` the row pitch in elements,
// `valid` the unit's columns that lie inside the matrix.
template <typename T>
__device__ __noinline__ void copy_out_rows(uint32_t buf, T* dst, int64_t ld, int rows, int valid, int lane) {
    const uint32_t word = ((static_cast<uint32_t>(lane) >> 2) << 4) | ((static_cast<uint32_t>(lane) & 3u) << 2);
    constexpr int kPer = sizeof(T) == 4 ? 1 : 2;  // elements per 32-bit word
    for (int r0 = 0; r0 < rows; r0 += 8) {
        uint32_t w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t rr = static_cast<uint32_t>(r0 + u);
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w[u]) : "r"(buf + (rr & 31u) * 128u + (word ^ ((rr & 7u) << 4))));
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (r0 + u >= rows) break;
            T* row = dst + static_cast<int64_t>(r0 + u) * ld + kPer * lane;
            if (kPer == 1) {
                if (lane < valid) *reinterpret_cast<uint32_t*>(row) = w[u];
            } else if (2 * lane + 1 < valid && (reinterpret_cast<uintptr_t>(row) & 3u) == 0u) {
                *reinterpret_cast<uint32_t*>(row) = w[u];
            } else {
                uint16_t* h = reinterpret_cast<uint16_t*>(row);
                if (2 * lane < valid) h[0] = static_cast<uint16_t>(w[u] & 0xFFFFu);
                if (2 * lane + 1 < valid) h[1] = static_cast<uint16_t>(w[u] >> 16);
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

// kLse: the extended, row-wise epilogue, a kernel of its own so that the code costs the other
// launches nothing.  Which of its parts run is in the problem's epi_flags:
//   kEpiLse     beside (or instead of) storing C, every epilogue warp keeps, per row, the maximum and
//               the sum of exponentials of the columns it produces and leaves them in
//               ProblemScalars::ext_stats; the warp that meets the row's target column leaves that
//               value in ext_rowvec (the LM head feeding a cross-entropy; the first pass of a
//               softmax over the rows of the product)
//   kEpiCausal  columns beyond the row's own index count as absent and are stored as exact zeros
//   kEpiExpSub  C = exp(v - ext_rowvec[row]): with the rows' log-sum-exp, the softmax itself
//   kEpiMulAux  C = aux ⊙ (v - ext_rowvec[row]): the softmax backward dS = P ⊙ (dP - D) as the
//               epilogue of the product that makes dP
//   kEpiSavePre the value before the GELU (after alpha, beta, bias) is stored as a second result
//   kEpiGeluBwd C = v * gelu'(aux): the dX product of the layer after a GELU, leaving as the gradient
//               with respect to the GELU's input (aux = the saved pre-activation)
//   kEpiCeGrad  C = (exp(v - lse[row]) - [col = target[row]]) * g[row]: the cross-entropy's gradient
//               with respect to the logits, from the LM-head product made a second time
template <uint32_t V> struct Sig { static constexpr uint32_t value = V; };

template <int CG, bool kLse>
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
    // The problems' scalars, copied from the kernel parameters (see ProblemScalars).
    ProblemScalars* sp = reinterpret_cast<ProblemScalars*>(smem_raw + (staging_base - smem_u32(smem_raw)) + Geo<CG>::kStagingBytes);
    volatile int* abort_flag = &ctl->abort_flag;
    DeviceStatus* status = gp.status;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            // A stage is released by the MMAs that read it (one commit) and by the eight epilogue
            // warps, which read it too when the tile sums its A operand for a bias gradient; for
            // every other tile the producer arrives in their place.
            mbar_init(smem_u32(&ctl->empty[s]), 1 + kEpilogueWarps);
            mbar_init(smem_u32(&ctl->landed[s]), 1);
        }
        mbar_init(smem_u32(&ctl->sum_bar[0]), kEpilogueWarps);
        mbar_init(smem_u32(&ctl->sum_bar[1]), kEpilogueWarps);
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctl->tmem_empty[a]), CG * kEpilogueWarps);      // both CTAs' epilogues
        }
        for (int r = 0; r < kRing; ++r) {
            mbar_init(smem_u32(&ctl->sched_full[r]), 1);
            mbar_init(smem_u32(&ctl->sched_empty[r]), kPair ? 2 * (1 + kProducerHelpers + kEpilogueWarps) : 1 + kEpilogueWarps);  // every ring reader
        }
        ctl->abort_flag = 0;
        fence_barrier_init();
    }
    // The peer must see these barriers before anything is sent to them: arrive now, wait after the
    // rest of the set-up (the cluster barrier's round trip overlaps it).
    __syncwarp();  // (thread 0 is back with its warp: the arrive is a warp-wide instruction)
    if (kPair) cluster_arrive_all();
    // Independent of everything else, and slow: the tensor maps' descriptors on their way to the
    // TMA unit.  (The first ticket needs no round trip at all: see the scheduler.)
    if (warp == 0 && leader) {
        if (lane >= 1 && lane <= 3 * gp.num_problems && lane <= 24) {
            const GroupProblem& q = gp.prob[(lane - 1) / 3];
            const int which = (lane - 1) % 3;
            if (which < 2 || q.c_tma) prefetch_tensormap(which == 0 ? &q.map_a : which == 1 ? &q.map_b : &q.map_c);
        }
    } else if (warp == 0 && lane >= 1 && lane <= 2 * gp.num_problems && lane <= 16) {
        const GroupProblem& q = gp.prob[(lane - 1) / 2];
        prefetch_tensormap((lane - 1) % 2 == 0 ? &q.map_a : &q.map_b);
    }
    if (static_cast<int>(threadIdx.x) < gp.num_problems) {
        // Shared-memory descriptors, 128-byte swizzle: K-major = k-step 32 bytes along the
        // row, LBO unused (16), SBO 1024; MN-major = k-step 16 k-rows of 128 bytes, LBO =
        // one 64-wide block, SBO 1024.  Only the 14-bit start-address field changes between
        // k-steps and stages, so the issuing thread does one add per operand.
        const ProblemScalars& q = gp.prob[threadIdx.x];
        uint4 c;
        c.x = make_idesc_bf16(kTileRows, q.bn, q.a_mn, q.b_mn);
        c.y = (smem_base >> 4) | (((q.a_mn ? kBlock64Bytes : 16u) >> 4) << 16);
        c.z = ((smem_base + kATileBytes) >> 4) | (((q.b_mn ? kBlock64Bytes : 16u) >> 4) << 16);
        c.w = ((q.a_mn ? UMMA_K * 128u : UMMA_K * 2u) >> 4) | (((q.b_mn ? UMMA_K * 128u : UMMA_K * 2u) >> 4) << 16);
        ctl->mma_consts[threadIdx.x] = c;
    }
    {
        constexpr int kWords = static_cast<int>(sizeof(ProblemScalars) / 4);
        for (int i = threadIdx.x; i < gp.num_problems * kWords; i += kThreads) {
            const int pi = i / kWords, wi = i - pi * kWords;
            reinterpret_cast<uint32_t*>(&sp[pi])[wi] =
                reinterpret_cast<const uint32_t*>(static_cast<const ProblemScalars*>(&gp.prob[pi]))[wi];
        }
    }
    if (warp == 1) {
        tmem_alloc_cg<CG>(smem_u32(&ctl->tmem_base), kTmemCols);
        tmem_relinquish_cg<CG>();
    }
    tc_fence_before_thread_sync();
    __syncthreads();
    if (kPair) cluster_wait_all();
    tc_fence_after_thread_sync();
    const uint32_t tmem_base = ctl->tmem_base;
    // The first ticket of every drawer is its own index (any order of arrival would hand the
    // first n_sched tickets to the n_sched drawers anyway); the queue's counter serves the tickets
    // from n_sched on, so no atomic's round trip stands before the first load.
    const int first_ticket = sched_id;
    // Everything above touched only this CTA's own state, so it may overlap the tail of the
    // previous kernel in the stream.  What depends on that kernel is global memory, and every
    // warp that touches any waits for it itself, as late as it can: the producers only before
    // their first load, so that the first tile's ticket, its decoding and the boxes' set-up (some
    // two microseconds of code that runs from a cold instruction cache at this point) are done
    // by the time the previous kernel's results are visible; the MMA issuer touches none.
    grid_launch_dependents();
    if (gp.ride.tiles > 0 && blockIdx.x == 0 && static_cast<int>(threadIdx.x) < gp.ride.world) {
        grid_dependency_wait();
        if (static_cast<int>(threadIdx.x) != gp.ride.rank) {
            // Everything earlier in this stream is complete, so this rank's partial sums of the range
            // that rides along are: tell the other ranks.
            const uint32_t e = *reinterpret_cast<volatile uint32_t*>(gp.ride.local + kRideStep) * kMaxRidesPerStep +
                               static_cast<uint32_t>(gp.ride.index);
            __threadfence_system();
            st_release_sys(gp.ride.peer_ready[threadIdx.x], e);
        }
    }

    // Barriers that live in the leader CTA of a pair, as cluster addresses usable from both.
    auto on_leader = [&](const void* bar) { return kPair ? mapa_shared(smem_u32(bar), 0u) : smem_u32(bar); };
    // A ring reader releases its slot to the scheduler (the leader's barrier).
    auto release_ring_slot = [&](int slot) {
        if (kPair) mbar_arrive_cluster(on_leader(&ctl->sched_empty[slot]));
        else mbar_arrive(smem_u32(&ctl->sched_empty[slot]));
    };

    if (warp == 0 || (kPair && warp >= kProducerHelperWarp && warp < kProducerHelperWarp + kProducerHelpers)) {
        // ------------------------------------------- scheduler + TMA producers
        // Two producer warps take the k-blocks in turn.  The operand pipeline is bound by bytes
        // in flight (six stages against a load latency of about six k-block times), so a load
        // that is issued late is a bubble in the tensor pipe later: a producer must be waiting at
        // a stage's barrier when the stage frees.  One iteration costs a few hundred cycles of
        // barrier and issue latency, which a single warp cannot hide (a third warp measured no
        // further gain).  In each warp the whole warp walks the loop; lane 0 does the barrier
        // bookkeeping and lane L issues the L-th box of a stage, so the up to six TMA boxes of a k-block
        // (MN-major operands come in 64-wide blocks) leave in one issue slot.  Warp 0 of the
        // leader also runs the scheduler.
        const bool scheduler = warp == 0 && leader;
        // A single CTA streams 48 KB per k-block and is bound by that, not by issue latency:
        // there the helper stays idle and warp 0 takes every k-block.
        const int n_turns = kPair ? 1 + kProducerHelpers : 1;
        const int my_turn = warp == 0 ? 0 : warp - kProducerHelperWarp + 1;
        int turn = 0;      // whose k-block `seq` is: producers take them round robin, across tiles
        uint32_t seq = 0;  // k-blocks streamed so far by this CTA; k-block `seq` uses stage seq % kStages
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        // A ticket is drawn when the producer is nearly ready to stream that tile: a few k-blocks
        // before it has issued the last loads of the current one (the first ticket before the
        // dependency wait), so that the atomic's round trip (about a microsecond) overlaps those
        // loads instead of opening a bubble between two tiles.  Drawing a whole tile ahead would hide
        // it too, but every CTA busy with a long tile would then sit on a short one that idle
        // CTAs could have taken (measured on the QKV backward: the dX CTAs idle from 35 us of an
        // 84 us launch).
        const bool dynamic = gp.static_schedule == 0;
        int prev_ticket = 0;
        constexpr int kDrawAhead = 8;   // k-blocks before the end of a tile at which the next ticket is drawn
        constexpr int kNotDrawn = -2;
        int next_ticket = kNotDrawn;
        // The per-tile code of every role runs once in thousands of cycles, from a cold
        // instruction cache, on the critical path of the operand pipeline (a stage is refilled
        // about as fast as it is consumed, so a load that is issued late is a bubble in the tensor
        // pipe later).  So the ticket is decoded once, here, and on long tiles ahead of need: a few
        // k-blocks before the current tile's last loads, right after one of this warp's own
        // k-blocks (two k-block times before its next one is due), as soon as the ring slot is
        // free.  Short tiles publish at the top of the next iteration.
        constexpr int kPublishAhead = 5;     // earliest k-block, counted from the end of the tile
        constexpr int kMinEarlyKblocks = 10; // shorter tiles publish at the top (the draw has not returned yet)
        bool early = false;                  // the next iteration's ticket is already in the ring
        bool dep_waited = false;             // this warp has waited for the previous kernel in the stream
        // Ring entry `slot` <- ticket `raw`, decoded (out-of-range: the end marker).
        auto publish = [&](int slot, int raw) {
            int t = raw;
            prev_ticket = raw;
            if (t >= gp.total_tiles) {
                // Every drawer takes exactly one out-of-range ticket; the last re-arms the counter.
                if (dynamic && t == gp.total_tiles + n_sched - 1) *gp.sched_counter = 0;
                t = -1;
            }
            TileCoord e;
            if (t >= gp.colsum_total && t < gp.fin_begin) {
                e = decode_tile(sp, gp.num_problems, t);
            } else {
                e.t = t;  // the end, or a dbias ticket: the readers look at nothing else
                e.prob = e.kb0 = e.kb1 = e.m_tile = e.n_tile = e.bz = e.bw = e.split = e.batch = e.pad0 = e.pad1 = 0;
            }
            ctl->ring[slot] = e;
            mbar_arrive(smem_u32(&ctl->sched_full[slot]));
            // The peer's copy travels as async stores that complete its barrier.
            if (kPair) {
                const uint32_t dst = mapa_shared(smem_u32(&ctl->ring[slot]), 1u);
                const uint32_t bar = mapa_shared(smem_u32(&ctl->sched_full[slot]), 1u);
                const uint32_t* w = reinterpret_cast<const uint32_t*>(&e);
#pragma unroll
                for (int q = 0; q < 3; ++q) st_async_cluster_v4(dst + 16u * q, w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3], bar);
            }
        };
        for (int it = 0; ok; ++it) {
            const int slot = it % kRing;
            const uint32_t sphase = static_cast<uint32_t>(it / kRing) & 1u;
            if (lane == 0) {
                if (scheduler && early) {
                    early = false;
                } else if (scheduler) {
                    ok = bounded_wait<kPair>(smem_u32(&ctl->sched_empty[slot]), sphase ^ 1u, abort_flag, status,
                                             kDevWaitSched, slot, wait_ns);
                    if (ok) {
                        const int raw = it == 0 ? first_ticket
                                      : !dynamic ? prev_ticket + n_sched
                                      : next_ticket != kNotDrawn ? next_ticket : atomicAdd(gp.sched_counter, 1) + n_sched;
                        next_ticket = kNotDrawn;
                        publish(slot, raw);
                    }
                } else {
                    // In the peer CTA warp 0 arms the ring barrier for the leader's stores.
                    if (kPair && warp == 0)
                        mbar_arrive_expect_tx(smem_u32(&ctl->sched_full[slot]), static_cast<uint32_t>(sizeof(TileCoord)));
                    ok = bounded_wait<kPair>(smem_u32(&ctl->sched_full[slot]), sphase, abort_flag, status,
                                             kDevWaitSched, 48 + slot, wait_ns);
                }
            }
            __syncwarp();  // lane 0's ring write is visible to the warp
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const TileCoord tc = ctl->ring[slot];
            __syncwarp();
            if (!scheduler && lane == 0) release_ring_slot(slot);
            const int t = tc.t;
            if (t < 0) break;
            if (t < gp.colsum_total || t >= gp.fin_begin) continue;  // a dbias ticket: work for the epilogue warps only
            const ProblemScalars& p = sp[tc.prob];
            const GroupProblem& pm = gp.prob[tc.prob];  // for the addresses of its tensor maps only
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
                my_map = &pm.map_a;
                if (a_mn) { my_off = lane * kBlock64Bytes; my_x = m0 + 64 * lane; k_is_y = true; }
                else      { my_y = m0; k_is_x = true; }
            } else if (lane < n_a + n_b) {
                const int j = lane - n_a;
                my_map = &pm.map_b;
                my_off = kATileBytes;
                if (b_mn) { my_off += j * kBlock64Bytes; my_x = n0 + 64 * j; k_is_y = true; }
                else      { my_y = n0; k_is_x = true; }
            }
            if (!dep_waited) {   // the first loads are next: the previous kernel must be done
                grid_dependency_wait();
                dep_waited = true;
            }
            const bool tile_sums = p.dbias_mode == 3 && tc.n_tile == 0;  // the epilogue warps read this tile's A stages
            const int draw_kb = tc.kb1 - kDrawAhead > tc.kb0 ? tc.kb1 - kDrawAhead : tc.kb0;
            const int publish_kb = tc.kb1 - tc.kb0 >= kMinEarlyKblocks ? tc.kb1 - kPublishAhead : 0x7fffffff;
            const int after_own = n_turns > 1 ? 1 : 0;
            for (int kb = tc.kb0; kb < tc.kb1; ++kb, ++seq) {
                if (kb >= draw_kb && scheduler && lane == 0) {  // (the first test is warp-uniform and false on most k-blocks)
                    if (dynamic && kb == draw_kb) next_ticket = atomicAdd(gp.sched_counter, 1) + n_sched;
                    if (kb >= publish_kb && !early && turn == after_own) {
                        const int nslot = (it + 1) % kRing;
                        const uint32_t nphase = static_cast<uint32_t>((it + 1) / kRing) & 1u;
                        // one poll: a ring that is still full is waited for at the top
                        if (mbar_try_wait(smem_u32(&ctl->sched_empty[nslot]), nphase ^ 1u)) {
                            publish(nslot, dynamic ? next_ticket : prev_ticket + n_sched);
                            next_ticket = kNotDrawn;
                            early = true;
                        }
                    }
                }
                if (turn == my_turn) {
                    if (lane == 0)
                        ok = bounded_wait<kPair>(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag, status,
                                                 kDevWaitSmemEmpty, stage, wait_ns);
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    // The loads leave first: the latency from "stage free" to "load issued" is part of
                    // every stage's cycle.  The bookkeeping follows; bytes that land before the
                    // barrier is armed are counted all the same (the phase cannot complete without
                    // the arming arrival).
                    if (my_map != nullptr) {
                        const int k0 = kb * BK;
                        const uint32_t dst = smem_base + static_cast<uint32_t>(stage) * kStageBytes + my_off;
                        const int x = my_x + (k_is_x ? k0 : 0), y = my_y + (k_is_y ? k0 : 0);
                        if (kPair) tma_load_4d_pair(dst, my_map, on_leader(&ctl->full[stage]), x, y, tc.bz, tc.bw);
                        else tma_load_4d(dst, my_map, smem_u32(&ctl->full[stage]), x, y, tc.bz, tc.bw);
                    }
                    if (lane == 0) {
                        // The leader's barrier counts the bytes of both CTAs of a pair.
                        if (leader) mbar_arrive_expect_tx(smem_u32(&ctl->full[stage]), tx * CG);
                        // the stage's next release: nobody but the MMAs will read it
                        if (!tile_sums) mbar_arrive_count(smem_u32(&ctl->empty[stage]), kEpilogueWarps);
                    }
                }
                if (++turn == n_turns) turn = 0;
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0 && leader) {
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
                const int4 head = *reinterpret_cast<const int4*>(&ctl->ring[slot]);  // t, prob, kb0, kb1
                release_ring_slot(slot);
                const int t = head.x;
                if (t < 0) break;
                if (t < gp.colsum_total || t >= gp.fin_begin) continue;
                const int nkb = head.w - head.z;
                const uint4 mc = ctl->mma_consts[head.y];
                const uint32_t idesc = mc.x, a_lo_base = mc.y, b_lo_base = mc.z;
                const uint32_t step_a = mc.w & 0xFFFFu, step_b = mc.w >> 16;
                const int acc = static_cast<int>(acc_seq & 1u);
                ok = bounded_wait<kPair>(smem_u32(&ctl->tmem_empty[acc]), ((acc_seq >> 1) & 1u) ^ 1u, abort_flag,
                                         status, kDevWaitTmemEmpty, acc, wait_ns);
                if (!ok) break;
                tc_fence_after_thread_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * kAccStride;
                for (int i = 0; i < nkb; ++i) {
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
                        umma_bf16_cg<CG>(d_tmem, da, db, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit_cg<CG>(smem_u32(&ctl->empty[stage]));  // frees the stage when the MMAs retire
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit_cg<CG>(smem_u32(&ctl->tmem_full[acc]));
                ++acc_seq;
            }
        }
    } else if (warp == kSideWarp) {
        // ------------------------------------------------------------ side warp
        if (gp.ride.tiles > 0) {
            grid_dependency_wait();
            ride_exchange_side_warp(gp.ride, gp.ride_counter, lane, wait_ns, status);
        }
    } else if (warp < 2 + kEpilogueWarps) {
        // ---------------------------------------------------------- epilogue
        grid_dependency_wait();              // bias, C_in, dbias tickets and the result itself are global memory
        const int quarter = warp & 3;        // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
        const int half = (warp - 2) >> 2;    // this warp takes the column units u with u % 2 == half
        const int ew = warp - 2;             // 0..7
        const uint32_t my_bufs = staging_base + static_cast<uint32_t>(ew * kStoreBufs) * kStoreBufBytes;
        uint32_t buf_seq = 0;  // TMA stores this warp has issued so far
        uint32_t acc_seq = 0;  // accumulator slot counter, in step with the MMA issuer's
        int e_stage = 0;       // stage and phase of the next tile's first k-block: the epilogue warps follow
        uint32_t e_phase = 0;  // the CTA's k-block sequence, because on some tiles they read the stages too
        uint32_t sum_phase = 0;
        uint32_t landed_bits = 0;  // peer CTA: parity of each stage's `landed` barrier (it moves on summing tiles only)
        bool ok = true;
        for (int it = 0; ok; ++it) {
            const int slot = it % kRing;
            const uint32_t sphase = static_cast<uint32_t>(it / kRing) & 1u;
            ok = bounded_wait<kPair>(smem_u32(&ctl->sched_full[slot]), sphase, abort_flag, status,
                                     kDevWaitSched, 32 + slot, wait_ns);
            if (!ok) break;
            const TileCoord tc = ctl->ring[slot];
            __syncwarp();
            if (lane == 0) release_ring_slot(slot);
            const int t = tc.t;
            if (t < 0) break;
            if (t < gp.colsum_total) {
                // A dbias reduction ticket of the problem that owns it.
                int pi = 0;
#pragma unroll 1
                for (int i = 0; i < gp.num_problems; ++i)
                    if (sp[i].colsum_tiles > 0 && t >= sp[i].colsum_begin) pi = i;
                const ProblemScalars& p = sp[pi];
                const int r = t - p.colsum_begin;
                if (p.dbias_mode == 1) {
                    dbias_partial_warp(p, r, static_cast<int>(rank) * kEpilogueWarps + ew, CG * kEpilogueWarps, lane);
                    if (gp.fin_begin < gp.total_tiles) {
                        // this warp's partial sums are written: count it for the finishing tickets
                        __syncwarp();
                        if (lane == 0) {
                            __threadfence();
                            atomicAdd(gp.dbias_sync, 1);
                        }
                    }
                } else {
                    dbias_rows_warp(p, (static_cast<int64_t>(r) * CG + rank) * kDbiasRowsPerCta + 2 * ew, lane);
                }
                continue;
            }
            if (t >= gp.fin_begin) {
                // A finishing ticket: every first-phase warp of the launch must have delivered.
                const int f = t - gp.fin_begin;
                int pi = 0;
#pragma unroll 1
                for (int i = 0; i < gp.num_problems; ++i)
                    if (sp[i].fin_tiles > 0 && f >= sp[i].fin_begin) pi = i;
                const ProblemScalars& p = sp[pi];
                int expected = 0;
#pragma unroll 1
                for (int i = 0; i < gp.num_problems; ++i)
                    if (sp[i].dbias_mode == 1) expected += sp[i].colsum_tiles;
                expected *= CG * kEpilogueWarps;
                int ready = 1;
                if (lane == 0) {
                    uint64_t t0 = 0;
                    uint32_t spins = 0;
                    while (*reinterpret_cast<volatile int32_t*>(gp.dbias_sync) < expected) {
                        if ((++spins & 63u) == 0u) {
                            const uint64_t now = globaltimer_ns();
                            if (t0 == 0) {
                                t0 = now;
                            } else if (now - t0 > wait_ns || *abort_flag) {
                                if (atomicCAS(&status->code, 0, kDevWaitSched) == 0) {
                                    status->detail = 99;
                                    status->block = static_cast<int32_t>(blockIdx.x);
                                }
                                ready = 0;
                                break;
                            }
                        }
                    }
                    __threadfence();
                }
                ready = __shfl_sync(0xffffffffu, ready, 0);
                if (ready)
                    dbias_finish_warp(p, (static_cast<int64_t>(f - p.fin_begin) * CG + rank) * kDbiasFinishPerCta + 32 * ew, lane);
                __syncwarp();
                if (lane == 0) {
                    // the last finishing warp of the launch re-arms both counters
                    const int fin_warps = (gp.total_tiles - gp.fin_begin) * CG * kEpilogueWarps;
                    if (atomicAdd(gp.dbias_sync + 1, 1) == fin_warps - 1) {
                        gp.dbias_sync[0] = 0;
                        gp.dbias_sync[1] = 0;
                    }
                }
                continue;
            }
            const ProblemScalars& p = sp[tc.prob];
            const int acc = static_cast<int>(acc_seq & 1u);
            const int nkb = tc.kb1 - tc.kb0;
            if (p.dbias_mode == 3 && tc.n_tile == 0) {
                // ---- bias gradient of a dW product: dbias[i] = sum over k of op(A)[i, k], A stored
                // [k, m].  The tile's A operand passes through shared memory anyway, and these warps
                // have nothing to do until the accumulator is complete: they add up every A stage
                // as it lands (a second reader of the stage beside the MMAs; both release it), so dy
                // is not read from memory a second time and nothing competes with the operand loads.
                // Warp w takes k-rows 8w..8w+7 of a stage; lane L the four m-columns 4 (L % 16) ..+3
                // of the 64-wide block L / 16 (one 8-byte read per row, 128-byte swizzle undone by
                // hand); rows, k-blocks and warps are added in ascending order: fixed order, no atomics.
                float dsum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t blk = static_cast<uint32_t>(lane >> 4) * kBlock64Bytes;
                const uint32_t chunk = static_cast<uint32_t>(lane & 15) >> 1, half8 = static_cast<uint32_t>(lane & 1) * 8u;
                for (int i = 0; i < nkb && ok; ++i) {
                    if (lane == 0) {
                        if (leader) {
                            ok = bounded_wait<kPair>(smem_u32(&ctl->full[e_stage]), e_phase, abort_flag, status,
                                                     kDevWaitSmemFull, 64 + e_stage, wait_ns);
                            // the peer CTA cannot see the leader's barrier: pass the news on
                            if (kPair && ok && ew == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&ctl->landed[e_stage]), 1u));
                        } else {
                            uint64_t t0 = 0;
                            uint32_t spins = 0;
                            while (!mbar_try_wait_cluster(smem_u32(&ctl->landed[e_stage]), (landed_bits >> e_stage) & 1u)) {
                                if ((++spins & 255u) == 0u) {
                                    const uint64_t now = globaltimer_ns();
                                    if (*abort_flag) { ok = false; break; }
                                    if (t0 == 0) {
                                        t0 = now;
                                    } else if (now - t0 > wait_ns) {
                                        if (atomicCAS(&status->code, 0, kDevWaitSmemFull) == 0) {
                                            status->detail = 96 + e_stage;
                                            status->block = static_cast<int32_t>(blockIdx.x);
                                        }
                                        *abort_flag = 1;
                                        ok = false;
                                        break;
                                    }
                                }
                            }
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    landed_bits ^= 1u << e_stage;
                    const uint32_t base = smem_base + static_cast<uint32_t>(e_stage) * kStageBytes + blk + half8;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const uint32_t row = static_cast<uint32_t>(8 * ew + r);
                        uint32_t lo, hi;
                        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(lo), "=r"(hi)
                                     : "r"(base + row * 128u + ((chunk ^ (row & 7u)) << 4)));
                        dsum[0] += __uint_as_float(lo << 16);
                        dsum[1] += __uint_as_float(lo & 0xFFFF0000u);
                        dsum[2] += __uint_as_float(hi << 16);
                        dsum[3] += __uint_as_float(hi & 0xFFFF0000u);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ctl->empty[e_stage]));  // this warp is done with the stage
                    if (++e_stage == kStages) { e_stage = 0; e_phase ^= 1u; }
                }
                if (!ok) break;
                // The eight warps' sums meet in the staging buffers (free once the TMA stores that
                // last read them have done so); warp 0 adds them in warp order and writes the result.
                if (lane == 0) bulk_wait_group_read_n<0>();
                __syncwarp();
                const uint32_t slot_off = static_cast<uint32_t>(64 * (lane >> 4) + 4 * (lane & 15)) * 4u;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                             ::"r"(my_bufs + slot_off), "r"(__float_as_uint(dsum[0])), "r"(__float_as_uint(dsum[1])),
                               "r"(__float_as_uint(dsum[2])), "r"(__float_as_uint(dsum[3])) : "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->sum_bar[0]));
                if (lane == 0)
                    ok = bounded_wait(smem_u32(&ctl->sum_bar[0]), sum_phase, abort_flag, status, kDevWaitSched, 80, wait_ns);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                if (ew == 0) {
                    float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int w = 0; w < kEpilogueWarps; ++w) {
                        uint32_t v0, v1, v2, v3;
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                                     : "r"(staging_base + static_cast<uint32_t>(w * kStoreBufs) * kStoreBufBytes + slot_off));
                        tot[0] += __uint_as_float(v0); tot[1] += __uint_as_float(v1);
                        tot[2] += __uint_as_float(v2); tot[3] += __uint_as_float(v3);
                    }
                    const int64_t i0 = static_cast<int64_t>(tc.m_tile) * kTileRows + static_cast<int64_t>(rank) * BM +
                                       64 * (lane >> 4) + 4 * (lane & 15);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (i0 + e >= p.m) break;
                        if (p.splits > 1) {
                            p.ws_dbias[static_cast<int64_t>(tc.split) * p.m + i0 + e] = tot[e];  // the split-K reduction adds the splits
                        } else {
                            const float prev = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i0 + e] : 0.0f;
                            p.dbias[i0 + e] = prev + tot[e];
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ctl->sum_bar[1]));  // the staging buffers may be written again
                if (lane == 0)
                    ok = bounded_wait(smem_u32(&ctl->sum_bar[1]), sum_phase, abort_flag, status, kDevWaitSched, 81, wait_ns);
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                sum_phase ^= 1u;
            } else {
                const int total = e_stage + nkb;
                e_phase ^= static_cast<uint32_t>(total / kStages) & 1u;
                e_stage = total % kStages;
            }
            // Everything a step needs is read from the problem's scalars ONCE per tile, into
            // registers: a step is a chain of dependent instructions executed by a warp that has
            // one other warp to share its scheduler with, so every shared-memory read and every
            // branch inside it costs its full latency, four times per tile.
            const int pm = p.m, pn = p.n;
            const int row0 = tc.m_tile * kTileRows + static_cast<int>(rank) * BM + quarter * 32;  // this warp's first row
            const bool row_ok = row0 + lane < pm;
            const int n0 = tc.n_tile * p.bn;
            const bool partial = p.splits > 1;
            const bool out_bf16 = !partial && p.c_is_bf16;
            // A column unit is what one TMA store carries: 32 rows x 128 bytes.  Everything per step
            // is shifts and adds: an integer division on this path costs a warp hundreds of cycles.
            const int unit_shift = out_bf16 ? 6 : 5;
            const int unit_cols = 1 << unit_shift;
            const int spu_shift = out_bf16 ? 1 : 0;
            const int spu = 1 << spu_shift;  // 32-column steps (one tcgen05.ld each) per unit
            const bool tma_ok = partial ? p.ws_tma != 0 : p.c_tma != 0;
            const CUtensorMap* out_map = partial ? &gp.prob[tc.prob].map_ws : &gp.prob[tc.prob].map_c;
            const int out_z = partial ? tc.batch * p.splits + tc.split : tc.bz;
            const int out_w = partial ? 0 : tc.bw;
            // Offset of this tile's batch item inside C, in elements.
            const int64_t c_item_off = static_cast<int64_t>(tc.bz) * p.stride_c + static_cast<int64_t>(tc.bw) * p.stride_c_outer;
            // Column (inside the tile) of this warp's s-th step.
            auto step_col = [&](int s) { return ((half + 2 * (s >> spu_shift)) << unit_shift) + ((s & (spu - 1)) << 5); };
            int ns = (((p.bn >> unit_shift) + 1 - half) >> 1) << spu_shift;
            while (ns > 0 && n0 + step_col(ns - 1) >= pn) --ns;
            if (row0 >= pm) ns = 0;  // the whole warp lies below the matrix
            // Offset of this thread's row of the tile inside C, in elements.
            const int64_t c_row_off = c_item_off + static_cast<int64_t>(row0 + lane) * p.ldc + n0;
            // The epilogue operations of this tile as bits; a split's partial sums get none.
            constexpr uint32_t kOpAlpha = 1u, kOpBeta = 2u, kOpBias = 4u, kOpGelu = 8u;
            // A signature: the operation bits, the result type, the extended epilogue's parts; or "generic".
            constexpr uint32_t kSigBf16 = 0x10u, kSigGeneric = 0x80000000u;
            constexpr uint32_t kSigExtMask = static_cast<uint32_t>(kEpiLse | kEpiExpSub | kEpiMulAux | kEpiCeGrad | kEpiGeluBwd | kEpiSavePre);
            const float alpha = p.alpha, beta = p.beta;
            const bool c_bf16 = p.c_is_bf16 != 0;
            const void* const c_ptr = p.c;
            uint32_t ops = 0;
            if (!partial) {
                if (alpha != 1.0f) ops |= kOpAlpha;
                if (beta != 0.0f && row_ok) ops |= kOpBeta;
                if (p.epi_flags & kEpiBias) ops |= kOpBias;
                if (p.epi_flags & kEpiGelu) ops |= kOpGelu;
            }
            // Every row of a step adds the same 32 bias values: lane j fetches the j-th of each of
            // the (at most four) steps now, while the tile's main loop is still running, and the
            // warp passes them round by shuffle when the step comes.
            float bias_mine[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (ops & kOpBias) {
                const bool bias_bf16 = p.bias_is_bf16 != 0;
                const void* const bias_ptr = p.bias;
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const int col = n0 + step_col(s) + lane;
                    if (s < ns && col < pn)
                        bias_mine[s] = bias_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(bias_ptr)[col])
                                                 : static_cast<const float*>(bias_ptr)[col];
                }
            }
            // Extended epilogue: this thread's row, over the columns this warp produces
            float lse_m = -INFINITY, lse_s = 0.0f;
            int lse_target = -1;
            float row_val = 0.0f, row_scale = 0.0f;
            const uint32_t ext = kLse ? static_cast<uint32_t>(p.epi_flags) : 0u;
            const int64_t ext_row = static_cast<int64_t>(tc.batch) * pm + row0 + lane;
            // Under the mask, with nothing to store, the steps beyond the diagonal for every row of
            // this warp have no work at all.
            if (kLse && (ext & kEpiCausal) && p.c == nullptr)
                while (ns > 0 && n0 + step_col(ns - 1) > row0 + 31) --ns;
            if (kLse && row_ok) {
                if ((ext & kEpiLse) && p.ext_ptr != nullptr) lse_target = static_cast<const int32_t*>(p.ext_ptr)[row0 + lane];
                if (ext & (kEpiExpSub | kEpiMulAux)) row_val = p.ext_rowvec[ext_row];
                if (ext & kEpiCeGrad) {
                    const float2 lg = p.ext_stats[row0 + lane];
                    row_val = lg.x;
                    row_scale = lg.y;
                    lse_target = static_cast<const int32_t*>(p.ext_ptr)[row0 + lane];
                }
                if (ext & (kEpiMulAux | kEpiGeluBwd)) {
                    const int esz = c_bf16 ? 2 : 4;
                    const char* base = static_cast<const char*>(p.ext_ptr) + c_row_off * esz;
                    for (int s = 0; s < ns; s += spu)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + static_cast<int64_t>(step_col(s)) * esz));
                }
            }
            if (ops & kOpBeta) {
                // beta * C_in is read row by row (one row per thread): ask L2 for this thread's
                // lines now, while the tile's main loop is still running.
                const int esz = c_bf16 ? 2 : 4;
                const char* base = static_cast<const char*>(c_ptr) + c_row_off * esz;
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
            // into the staging buffer; once the unit is complete it leaves by TMA or, for a
            // ragged unit or a C that TMA cannot address, by the warp's own row-wise stores.
            //
            // The step's code exists once per SIGNATURE (the epilogue operations and the result type
            // as compile-time constants) for the signatures that matter, plus once with everything
            // decided at run time: a step is a few hundred instructions run by a warp with one
            // other warp to hide behind, and every branch it has to resolve and every jump to a cold
            // instruction-cache line stalls it (batched scores, one k-block per tile: 5100 cycles of
            // epilogue per tile with run-time operations, 3400 with constants).  The fp32 results
            // (dW += ..., split-K partial sums) stay with the run-time form: their epilogue hides
            // behind long main loops, and constants measured slower where it does not (dW with dbias).
            auto emit = [&](auto sig_c, const uint32_t (&r)[32], int s, float my_bias) {
                constexpr uint32_t kSig = decltype(sig_c)::value;
                constexpr bool kGeneric = (kSig & kSigGeneric) != 0;
                const uint32_t e_ops = kGeneric ? ops : (kSig & 0xFu);
                const bool e_bf16 = kGeneric ? out_bf16 : (kSig & kSigBf16) != 0;
                const uint32_t e_ext = !kLse ? 0u : kGeneric ? ext : ((ext & kEpiCausal) | (kSig & kSigExtMask));
                const int c0 = step_col(s);
                const int col = n0 + c0;
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                if (e_ops != 0u) {
                    if (e_ops & kOpAlpha) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] *= alpha;
                    }
                    if (e_ops & kOpBeta) {
                        const int valid = row_ok ? min(32, pn - col) : 0;
                        const int64_t c_off = c_row_off + c0;
                        float cin[32];
                        if (c_bf16)
                            load_chunk_bf16(static_cast<const __nv_bfloat16*>(c_ptr) + c_off, cin, valid);
                        else
                            load_chunk_f32(static_cast<const float*>(c_ptr) + c_off, cin, valid);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = fmaf(beta, cin[j], v[j]);
                    }
                    if (e_ops & kOpBias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, my_bias, j);
                    }
                    if (kLse && (e_ext & kEpiSavePre)) {
                        // the value the GELU is about to see, for the backward pass
                        const int have = row_ok ? min(32, pn - col) : 0;
                        if (c_bf16) store_chunk_bf16(static_cast<__nv_bfloat16*>(const_cast<void*>(p.ext_ptr)) + c_row_off + c0, v, have);
                        else store_chunk_f32(static_cast<float*>(const_cast<void*>(p.ext_ptr)) + c_row_off + c0, v, have);
                    }
                    if (e_ops & kOpGelu) {
                        // A bf16 result rounds at 2^-9: the hardware tanh (2^-11) is exact enough for
                        // it and halves the special-function work, which bounds this step; an fp32
                        // result gets the form that is accurate to 1e-6.
                        if (e_bf16) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_hw(v[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_fast(v[j]);
                        }
                    }
                }
                if (kLse) {
                    // Columns of this step that exist for this thread's row (may be <= 0 under the mask).
                    int valid = min(32, pn - col);
                    if (e_ext & kEpiCausal) valid = min(valid, row0 + lane + 1 - col);
                    // Almost every step has all of its columns for all of its rows: that case runs
                    // without a predicate per value.  A step beyond the mask for all rows does no
                    // arithmetic at all.
                    const bool full = __all_sync(0xffffffffu, valid >= 32);
                    const bool none = !full && __all_sync(0xffffffffu, valid <= 0);
                    constexpr float kLog2e = 1.4426950408889634f;
                    if (!full && !none && (e_ext & (kEpiLse | kEpiExpSub))) {
                        // absent columns count as -inf: no part in the maximum, exp() exactly 0
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = j < valid ? v[j] : -INFINITY;
                    }
                    if ((e_ext & kEpiLse) && !none && valid > 0) {
                        float t[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) t[j] = fmaxf(v[2 * j], v[2 * j + 1]);
#pragma unroll
                        for (int w = 8; w > 0; w >>= 1) {
#pragma unroll
                            for (int j = 0; j < w; ++j) t[j] = fmaxf(t[j], t[j + w]);
                        }
                        // Exponentials relative to the running maximum itself: one rescaling of the
                        // sum so far per step instead of one per value.
                        const float nm = fmaxf(lse_m, t[0]);
                        const float nms = nm * kLog2e;
                        float acc4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc4[j & 3] += ex2_approx(fmaf(v[j], kLog2e, -nms));
                        lse_s = fmaf(lse_s, ex2_approx((lse_m - nm) * kLog2e), (acc4[0] + acc4[1]) + (acc4[2] + acc4[3]));
                        lse_m = nm;
                        if (lse_target >= col && lse_target < col + 32) {
                            float tv = 0.0f;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j == lse_target) tv = v[j];
                            p.ext_rowvec[row0 + lane] = tv;
                        }
                    }
                    if (p.c == nullptr) return;  // the product itself is not wanted
                    if (none) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = 0.0f;
                    } else if (e_ext & kEpiExpSub) {
                        const float shift = row_val * kLog2e;
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = ex2_approx(fmaf(v[j], kLog2e, -shift));
                    } else if (e_ext & kEpiGeluBwd) {
                        float aux[32];
                        const int have = row_ok ? min(32, pn - col) : 0;
                        if (c_bf16)
                            load_chunk_bf16(static_cast<const __nv_bfloat16*>(p.ext_ptr) + c_row_off + c0, aux, have);
                        else
                            load_chunk_f32(static_cast<const float*>(p.ext_ptr) + c_row_off + c0, aux, have);
                        if (e_bf16) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] *= dgelu_tanh_hw(aux[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] *= dgelu_tanh_precise(aux[j]);
                        }
                    } else if (e_ext & kEpiCeGrad) {
                        // softmax minus one-hot, times the row's weight; absent columns are not stored
                        const float shift = row_val * kLog2e;
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = ex2_approx(fmaf(v[j], kLog2e, -shift)) * row_scale;
                        if (lse_target >= col && lse_target < col + 32) {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j == lse_target) v[j] -= row_scale;
                        }
                    } else if (e_ext & kEpiMulAux) {
                        float aux[32];
                        const int64_t c_off = c_row_off + c0;
                        // aux holds exact zeros where the mask applies: whole chunks are read, so
                        // that the rows on the diagonal keep the vector loads
                        const int have = row_ok && valid > 0 ? min(32, pn - col) : 0;
                        if (c_bf16)
                            load_chunk_bf16(static_cast<const __nv_bfloat16*>(p.ext_ptr) + c_off, aux, have);
                        else
                            load_chunk_f32(static_cast<const float*>(p.ext_ptr) + c_off, aux, have);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = aux[j] * (v[j] - row_val);
                        if (!full) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = j < valid ? v[j] : 0.0f;
                        }
                    } else if (!full) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = j < valid ? v[j] : 0.0f;
                    }
                }
                const int sub = s & (spu - 1);
                const int unit_col = col - sub * 32;
                const bool by_tma = tma_ok && unit_col + unit_cols <= pn;
                const uint32_t buf = my_bufs + (buf_seq % kStoreBufs) * kStoreBufBytes;
                if (sub == 0) {
                    // The buffer is free once the TMA store that last read it has done so.
                    if (lane == 0) bulk_wait_group_read_n<kStoreBufs - 1>();
                    __syncwarp();
                }
                const uint32_t row_addr = buf + static_cast<uint32_t>(lane) * 128u;
                const uint32_t sw = static_cast<uint32_t>(lane) & 7u;
                if (e_bf16) {
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
                if (sub != spu - 1 && s != ns - 1) return;  // the unit's other half follows
                if (by_tma) {
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_4d(out_map, buf, unit_col, row0, out_z, out_w);
                        bulk_commit_group();
                    }
                    ++buf_seq;
                    return;
                }
                // A ragged unit, or a destination TMA cannot address (odd pitch or base): the warp
                // copies the staged rows out itself, one row per instruction, so that every store
                // instruction writes up to 128 contiguous bytes.
                __syncwarp();
                {
                    const int unit_valid = min(unit_cols, pn - unit_col);
                    const int rows = min(32, pm - row0);
                    if (e_bf16) {
                        copy_out_rows<uint16_t>(buf, static_cast<uint16_t*>(p.c) + c_item_off + static_cast<int64_t>(row0) * p.ldc + unit_col,
                                                p.ldc, rows, unit_valid, lane);
                    } else {
                        float* base = partial
                            ? p.ws + ((static_cast<int64_t>(tc.batch) * p.splits + tc.split) * pm + row0) * pn + unit_col
                            : static_cast<float*>(p.c) + c_item_off + static_cast<int64_t>(row0) * p.ldc + unit_col;
                        copy_out_rows<float>(buf, base, partial ? static_cast<int64_t>(pn) : p.ldc, rows, unit_valid, lane);
                    }
                }
                __syncwarp();  // the buffer may be rewritten once every lane has read its words
            };
            // Software pipeline over the steps: the tcgen05.ld of step s+1 is in flight while
            // step s is converted and staged; the prefetched values are moved into `cur` after
            // their wait.
            auto run_steps = [&](auto sig_c) {
                uint32_t cur[32], nxt[32];
                tmem_ld_32x32(t_row + static_cast<uint32_t>(step_col(0)), nxt);
#pragma unroll 1
                for (int s = 0; s < ns; ++s) {
                    tmem_ld_wait();
                    after_tmem_ld_wait(nxt);
#pragma unroll
                    for (int j = 0; j < 32; ++j) cur[j] = nxt[j];
                    if (s + 1 < ns) tmem_ld_32x32(t_row + static_cast<uint32_t>(step_col(s + 1)), nxt);
                    else release_acc();
                    emit(sig_c, cur, s, s == 0 ? bias_mine[0] : s == 1 ? bias_mine[1] : s == 2 ? bias_mine[2] : bias_mine[3]);
                }
            };
            if (ns == 0) {
                release_acc();
            } else {
                // The tile's signature: uniform over the CTA (beta counts even where this thread's
                // row lies below the matrix; the step itself looks at the row).
                uint32_t sig = (ops & ~kOpBeta) | (!partial && beta != 0.0f ? kOpBeta : 0u) | (out_bf16 ? kSigBf16 : 0u);
                if (kLse) sig |= ext & kSigExtMask;
                if (!kLse) {
                    switch (sig) {
                        case kSigBf16: run_steps(Sig<kSigBf16>{}); break;                                  // dX
                        case kSigBf16 | kOpAlpha: run_steps(Sig<kSigBf16 | kOpAlpha>{}); break;            // attention scores
                        case kSigBf16 | kOpBias: run_steps(Sig<kSigBf16 | kOpBias>{}); break;              // Linear forward
                        case kSigBf16 | kOpBias | kOpGelu: run_steps(Sig<kSigBf16 | kOpBias | kOpGelu>{}); break;  // MLP fc
                        default: run_steps(Sig<kSigGeneric>{}); break;
                    }
                } else {
                    switch (sig) {
                        case kEpiLse | kSigBf16 | kOpAlpha: run_steps(Sig<kEpiLse | kSigBf16 | kOpAlpha>{}); break;        // softmax, first pass
                        case kEpiExpSub | kSigBf16 | kOpAlpha: run_steps(Sig<kEpiExpSub | kSigBf16 | kOpAlpha>{}); break;  // softmax, second pass
                        case kEpiMulAux | kSigBf16: run_steps(Sig<kEpiMulAux | kSigBf16>{}); break;                         // softmax backward
                        case kEpiLse: run_steps(Sig<kEpiLse>{}); break;                                                     // LM head + loss
                        case kEpiCeGrad | kSigBf16: run_steps(Sig<kEpiCeGrad | kSigBf16>{}); break;                         // dLogits
                        case kEpiGeluBwd | kSigBf16: run_steps(Sig<kEpiGeluBwd | kSigBf16>{}); break;                       // dX through the GELU
                        case kEpiSavePre | kSigBf16 | kOpBias | kOpGelu: run_steps(Sig<kEpiSavePre | kSigBf16 | kOpBias | kOpGelu>{}); break;  // MLP fc, training
                        case kEpiLse | kOpBias: run_steps(Sig<kEpiLse | kOpBias>{}); break;
                        default: run_steps(Sig<kSigGeneric>{}); break;
                    }
                }
            }
            if (kLse && (ext & kEpiLse) && row_ok)
                p.ext_stats[static_cast<int64_t>(tc.n_tile * 2 + half) * p.batch * pm + ext_row] = make_float2(lse_m, lse_s);
            ++acc_seq;
        }
        // Outstanding TMA stores must have read their staging buffers before the shared memory goes
        // away; their writes complete with the grid.
        if (lane == 0) bulk_wait_group_read_n<0>();
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
    tc_grouped_body<1, false>(gp);
}

// The same kernel over CTA pairs: clusters of two CTAs, each pair computing 256-row tiles
// with cta_group::2 MMAs, every CTA staging its own 128 rows of A and half of the B tile.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
tc_grouped_pair_kernel(const __grid_constant__ GroupParams gp) {
    tc_grouped_body<2, false>(gp);
}

// C = epilogue(alpha * sum_s ws[s] + beta * C): fixed summation order s = 0..splits-1.
// Four consecutive columns per thread when the row length allows it.
// The same kernels with the log-sum-exp epilogue.
__global__ void __launch_bounds__(kThreads, 1)
tc_grouped_lse_kernel(const __grid_constant__ GroupParams gp) {
    tc_grouped_body<1, true>(gp);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
tc_grouped_pair_lse_kernel(const __grid_constant__ GroupParams gp) {
    tc_grouped_body<2, true>(gp);
}

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
        int64_t item_off = b * p.stride_c;
        if (p.batch_inner > 0) item_off = (b % p.batch_inner) * p.stride_c + (b / p.batch_inner) * p.stride_c_outer;
        const int64_t c_off = item_off + row * p.ldc + col;
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
        if (p.splits == 0) {
            // An empty reduction (k == 0) sums nothing into the bias gradient either.
            p.dbias[i] = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i] : 0.0f;
        } else if (p.dbias_mode == 3) {
            // The tiles summed their A stages per split; the splits are added here, in order.
            float acc = 0.0f;
            for (int s = 0; s < p.splits; ++s) acc += p.ws_dbias[static_cast<int64_t>(s) * p.m + i];
            p.dbias[i] = (p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i] : 0.0f) + acc;
        }
    }
}

}  // namespace

size_t tc_grouped_smem_bytes() {
    static_assert(sizeof(Control) <= 1024, "control block must fit below the first aligned KB");
    return Geo<1>::kSmemBytes > Geo<2>::kSmemBytes ? Geo<1>::kSmemBytes : Geo<2>::kSmemBytes;
}

int tc_pair_stages() { return Geo<2>::kStages; }
int tc_dbias_rows_per_cta() { return kDbiasRowsPerCta; }
int tc_dbias_finish_per_cta() { return kDbiasFinishPerCta; }

// Per-device record of what has been configured (cudaFuncSetAttribute is per device).
static bool g_configured[64];

static cudaError_t configure_device(int dev) {
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (g_configured[dev]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(tc_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tc_grouped_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tc_grouped_lse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(tc_grouped_pair_lse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess) g_configured[dev] = true;
    return e;
}

cudaError_t launch_tc_grouped(const GroupParams& gp, int grid, bool pairs, cudaStream_t stream, bool lse) {
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
    if (lse)
        e = pairs ? cudaLaunchKernelEx(&cfg, tc_grouped_pair_lse_kernel, gp)
                  : cudaLaunchKernelEx(&cfg, tc_grouped_lse_kernel, gp);
    else
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
