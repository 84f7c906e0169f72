// bf16 x bf16 -> fp32-accumulate GEMM for sm_100a as ONE persistent kernel over
// a list of problems ("group"): tcgen05 MMA with the accumulator in tensor
// memory, operands staged in 128-byte-swizzled shared memory by TMA, results
// leaving through swizzled shared-memory slabs and TMA stores.
//
// One CTA per SM, 320 threads, warp-specialised:
//   warp 0      scheduler + TMA producer (one lane): draws the next tile from a
//               global counter, publishes it to the other roles through a small
//               ring in shared memory, then streams that tile's operands
//   warp 1      MMA issuer (one lane issues tcgen05.mma / tcgen05.commit; the warp
//               owns the TMEM allocation)
//   warps 2-9   epilogue: tcgen05.ld, alpha/beta/bias/GELU/cast, store C (two warps
//               per TMEM lane quarter, each taking half of the tile's columns)
//
// Every problem of the group is llmt's row-major  C = alpha*op(A)*op(B) + beta*C
// (llmt include/llmt/kernels/matmul.h:12-24) with its own shape, transposes, tile
// width and epilogue; tiles of all problems share one queue, longest first, so
// the tail of one problem overlaps the head of the next and e.g. the dX and dW
// products of Linear::backward (llmt src/layers/linear.cpp:22-30) run as one launch.
//
// A transposed operand is not copied: the tile is loaded as stored and described
// to the tensor core as MN-major.  The fused bias gradient (row sums of op(A)) is
// an extra 64-wide block of bf16 ones loaded behind the B tile of the tiles in
// the first tile column, whose MMAs then run with N = bn + 16.
//
// No wait is unbounded: every mbarrier wait gives up after kWaitLimitNs, records
// why in the DeviceStatus word and makes the CTA drain and exit.
#include <cuda_bf16.h>

#include "common.h"
#include "ptx_sm100.cuh"

namespace llmt_b200 {

using namespace ptx;

namespace {

constexpr int BM = 128;  // UMMA M (cta_group::1)
constexpr int BK = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 320;
constexpr int kEpilogueWarps = 8;
constexpr int kStages = 4;
constexpr int kRing = 4;                             // scheduler ring entries
constexpr uint32_t kATileBytes = BM * BK * 2;        // 16 KB
constexpr uint32_t kBRegionBytes = 256 * BK * 2;     // 32 KB: widest B tile (or narrower tile + ones block)
constexpr uint32_t kStageBytes = kATileBytes + kBRegionBytes;
constexpr uint32_t kBlock64Bytes = 64 * BK * 2;      // one 64-wide MN-major block / the ones block
constexpr uint32_t kAccStride = 256;                 // TMEM columns per accumulator buffer
constexpr uint32_t kTmemCols = 512;
constexpr int kDbiasCols = 16;
constexpr uint32_t kSlabBytes = 128 * 32 * 4;        // 128 rows x 32 columns of fp32
constexpr uint32_t kStagingBytes = 2 * kSlabBytes;   // one slab per column half
constexpr uint64_t kWaitLimitNs = 2000000000ull;

struct __align__(8) Control {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t sched_full[kRing];
    uint64_t sched_empty[kRing];
    int32_t ring[kRing];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             DeviceStatus* st, int code, int detail) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63u) == 0u) {
            if (*abort_flag) return false;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
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

__device__ __forceinline__ void store_chunk_bf16(__nv_bfloat16* dst, const float* v, int valid) {
    if (valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0u) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j + 0], v[j + 1]);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
            uint4 u;
            u.x = *reinterpret_cast<uint32_t*>(&h0);
            u.y = *reinterpret_cast<uint32_t*>(&h1);
            u.z = *reinterpret_cast<uint32_t*>(&h2);
            u.w = *reinterpret_cast<uint32_t*>(&h3);
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

__global__ void __launch_bounds__(kThreads, 1)
tc_grouped_kernel(const __grid_constant__ GroupParams gp) {
    extern __shared__ uint8_t smem_raw[];
    // Swizzled tiles need 1024-byte alignment.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t staging_base = smem_base + kStages * kStageBytes;
    Control* ctl = reinterpret_cast<Control*>(smem_gen + kStages * kStageBytes + kStagingBytes);
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
            mbar_init(smem_u32(&ctl->tmem_empty[a]), kEpilogueWarps);
        }
        for (int r = 0; r < kRing; ++r) {
            mbar_init(smem_u32(&ctl->sched_full[r]), 1);
            mbar_init(smem_u32(&ctl->sched_empty[r]), 1 + kEpilogueWarps);
        }
        ctl->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
        tmem_relinquish_alloc_permit();
    }
    tc_fence_before_thread_sync();
    __syncthreads();
    tc_fence_after_thread_sync();
    const uint32_t tmem_base = ctl->tmem_base;

    if (warp == 0) {
        // ------------------------------------------- scheduler + TMA producer
        // The whole warp walks the loop; lane 0 owns the scheduler and the barrier
        // bookkeeping, and lane L issues the L-th box of a stage, so the up to seven TMA
        // boxes of a k-block (MN-major operands come in 64-wide blocks) leave in one issue
        // slot instead of queueing behind one thread.
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        // The ticket for the NEXT tile is drawn while the current tile's operands stream,
        // so the atomic's round trip stays off the critical path.
        const bool dynamic = gp.static_schedule == 0;
        int next = 0;
        if (lane == 0) next = dynamic ? atomicAdd(gp.sched_counter, 1) : static_cast<int>(blockIdx.x);
        for (int it = 0; ok; ++it) {
            const int slot = it % kRing;
            const uint32_t sphase = static_cast<uint32_t>(it / kRing) & 1u;
            int t = -1;
            if (lane == 0) {
                ok = bounded_wait(smem_u32(&ctl->sched_empty[slot]), sphase ^ 1u, abort_flag, status,
                                  kDevWaitSched, slot);
                if (ok) {
                    t = next;
                    if (t >= gp.total_tiles) {
                        // Every CTA draws exactly one out-of-range ticket; the last one re-arms the counter.
                        if (dynamic && t == gp.total_tiles + static_cast<int>(gridDim.x) - 1) *gp.sched_counter = 0;
                        t = -1;
                    } else {
                        next = dynamic ? atomicAdd(gp.sched_counter, 1) : t + static_cast<int>(gridDim.x);
                    }
                    ctl->ring[slot] = t;
                    mbar_arrive(smem_u32(&ctl->sched_full[slot]));
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            t = __shfl_sync(0xffffffffu, t, 0);
            if (!ok || t < 0) break;
            const TileCoord tc = decode_tile(gp, t);
            const GroupProblem& p = gp.prob[tc.prob];
            const int bn = p.bn, a_mn = p.a_mn, b_mn = p.b_mn;
            const int m0 = tc.m_tile * BM, n0 = tc.n_tile * bn;
            const bool ones = p.dbias != nullptr && tc.n_tile == 0;
            const uint32_t tx = kATileBytes + static_cast<uint32_t>(bn) * (BK * 2) + (ones ? kBlock64Bytes : 0u);
            // This lane's box: destination offset inside the stage, tensor map, and the
            // coordinates (the k coordinate advances with the k-block).
            const int n_a = a_mn ? 2 : 1, n_b = b_mn ? (bn >> 6) : 1;
            const CUtensorMap* my_map = nullptr;
            uint32_t my_off = 0;
            int my_x = 0, my_y = 0;
            bool k_is_x = false;
            if (lane < n_a) {
                my_map = &p.map_a;
                if (a_mn) { my_off = lane * kBlock64Bytes; my_x = m0 + 64 * lane; }
                else      { my_y = m0; k_is_x = true; }
            } else if (lane < n_a + n_b) {
                const int j = lane - n_a;
                my_map = &p.map_b;
                my_off = kATileBytes;
                if (b_mn) { my_off += j * kBlock64Bytes; my_x = n0 + 64 * j; }
                else      { my_y = n0; k_is_x = true; }
            } else if (lane == n_a + n_b && ones) {
                my_map = &gp.map_ones;
                my_off = kATileBytes + static_cast<uint32_t>(bn) * (BK * 2);
            }
            const bool k_is_y = (my_map == &p.map_a && a_mn) || (my_map == &p.map_b && b_mn);
            const int batch = my_map == &gp.map_ones ? 0 : tc.batch;
            for (int kb = tc.kb0; kb < tc.kb1; ++kb) {
                if (lane == 0) {
                    ok = bounded_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag, status,
                                      kDevWaitSmemEmpty, stage);
                    if (ok) mbar_arrive_expect_tx(smem_u32(&ctl->full[stage]), tx);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                if (my_map != nullptr) {
                    const int k0 = kb * BK;
                    tma_load_3d(smem_base + static_cast<uint32_t>(stage) * kStageBytes + my_off, my_map,
                                smem_u32(&ctl->full[stage]), my_x + (k_is_x ? k0 : 0),
                                my_y + (k_is_y ? k0 : 0), batch);
                }
                if (++stage == kStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // Shared-memory descriptor, 128-byte swizzle: K-major = k-step 32 bytes along the
            // row, LBO unused (16), SBO 1024; MN-major = k-step 16 k-rows of 128 bytes, LBO =
            // one 64-wide block, SBO 1024.  Only the 14-bit start-address field changes between
            // k-steps and stages, so the issuing thread does one add per operand.
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int it = 0; ok; ++it) {
                const int slot = it % kRing;
                const uint32_t sphase = static_cast<uint32_t>(it / kRing) & 1u;
                ok = bounded_wait(smem_u32(&ctl->sched_full[slot]), sphase, abort_flag, status,
                                  kDevWaitSched, 16 + slot);
                if (!ok) break;
                const int t = ctl->ring[slot];
                mbar_arrive(smem_u32(&ctl->sched_empty[slot]));
                if (t < 0) break;
                const TileCoord tc = decode_tile(gp, t);
                const GroupProblem& p = gp.prob[tc.prob];
                const bool ones = p.dbias != nullptr && tc.n_tile == 0;
                const uint32_t idesc = make_idesc_bf16(BM, p.bn + (ones ? kDbiasCols : 0), p.a_mn, p.b_mn);
                const uint32_t step_a = (p.a_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
                const uint32_t step_b = (p.b_mn ? UMMA_K * 128 : UMMA_K * 2) >> 4;
                const uint32_t a_lo_base = (smem_base >> 4) | (((p.a_mn ? kBlock64Bytes : 16u) >> 4) << 16);
                const uint32_t b_lo_base = ((smem_base + kATileBytes) >> 4) |
                                           (((p.b_mn ? kBlock64Bytes : 16u) >> 4) << 16);
                ok = bounded_wait(smem_u32(&ctl->tmem_empty[acc]), acc_phase ^ 1u, abort_flag, status,
                                  kDevWaitTmemEmpty, acc);
                if (!ok) break;
                tc_fence_after_thread_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * kAccStride;
                for (int kb = tc.kb0; kb < tc.kb1; ++kb) {
                    ok = bounded_wait(smem_u32(&ctl->full[stage]), phase, abort_flag, status,
                                      kDevWaitSmemFull, stage);
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
                        umma_bf16(d_tmem, da, db, idesc, (kb > tc.kb0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&ctl->empty[stage]));  // frees the stage when the MMAs retire
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                umma_commit(smem_u32(&ctl->tmem_full[acc]));
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------------------------------------------------- epilogue
        const int quarter = warp & 3;        // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
        const int half = (warp - 2) >> 2;    // which half of the tile's columns this warp drains
        const int tile_row = quarter * 32 + lane;
        const uint32_t slab = staging_base + static_cast<uint32_t>(half) * kSlabBytes;
        const bool store_leader = (warp == 2 + 4 * half) && lane == 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int it = 0; ok; ++it) {
            const int slot = it % kRing;
            const uint32_t sphase = static_cast<uint32_t>(it / kRing) & 1u;
            ok = bounded_wait(smem_u32(&ctl->sched_full[slot]), sphase, abort_flag, status,
                              kDevWaitSched, 32 + slot);
            if (!ok) break;
            const int t = ctl->ring[slot];
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->sched_empty[slot]));
            if (t < 0) break;
            const TileCoord tc = decode_tile(gp, t);
            const GroupProblem& p = gp.prob[tc.prob];
            ok = bounded_wait(smem_u32(&ctl->tmem_full[acc]), acc_phase, abort_flag, status,
                              kDevWaitTmemFull, acc);
            if (!ok) break;
            tc_fence_after_thread_sync();
            const int64_t row = static_cast<int64_t>(tc.m_tile) * BM + tile_row;
            const bool row_ok = row < p.m;
            const int64_t n0 = static_cast<int64_t>(tc.n_tile) * p.bn;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc) * kAccStride;
            const bool partial = p.splits > 1;
            const bool via_tma = p.c_tma && !partial;
            const int half_cols = p.bn >> 1;
#pragma unroll 1
            for (int c0 = half * half_cols; c0 < (half + 1) * half_cols; c0 += 32) {
                if (n0 + c0 >= p.n) break;  // warp-uniform, and the same in all warps of a half
                uint32_t r[32];
                tmem_ld_32x32(t_row + static_cast<uint32_t>(c0), r);
                tmem_ld_wait();
                const int64_t col = n0 + c0;
                const int valid = static_cast<int>(min(static_cast<int64_t>(32), p.n - col));
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                if (partial) {
                    if (row_ok) {
                        float* dst = p.ws +
                                     ((static_cast<int64_t>(tc.batch) * p.splits + tc.split) * p.m + row) * p.n + col;
                        store_chunk_f32(dst, v, valid);
                    }
                    continue;
                }
                if (p.alpha != 1.0f) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
                }
                const int64_t c_off = static_cast<int64_t>(tc.batch) * p.stride_c + row * p.ldc + col;
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
                // TMA clips a box at 16-byte granularity, so a ragged last chunk goes out
                // through registers instead.
                if (via_tma && valid == 32) {
                    // The slab is free once the previous TMA store has read it.
                    if (store_leader) bulk_wait_group_read0();
                    named_barrier_sync(1 + half, 128);
                    if (p.c_is_bf16) {
                        const uint32_t row_addr = slab + static_cast<uint32_t>(tile_row) * 64u;
                        const uint32_t sw = static_cast<uint32_t>(tile_row >> 1) & 3u;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * q + 0], v[8 * q + 1]);
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * q + 2], v[8 * q + 3]);
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * q + 4], v[8 * q + 5]);
                            __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * q + 6], v[8 * q + 7]);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(row_addr + ((static_cast<uint32_t>(q) ^ sw) << 4)),
                                           "r"(*reinterpret_cast<uint32_t*>(&h0)),
                                           "r"(*reinterpret_cast<uint32_t*>(&h1)),
                                           "r"(*reinterpret_cast<uint32_t*>(&h2)),
                                           "r"(*reinterpret_cast<uint32_t*>(&h3)) : "memory");
                        }
                    } else {
                        const uint32_t row_addr = slab + static_cast<uint32_t>(tile_row) * 128u;
                        const uint32_t sw = static_cast<uint32_t>(tile_row) & 7u;
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                         ::"r"(row_addr + ((static_cast<uint32_t>(q) ^ sw) << 4)),
                                           "r"(__float_as_uint(v[4 * q + 0])), "r"(__float_as_uint(v[4 * q + 1])),
                                           "r"(__float_as_uint(v[4 * q + 2])), "r"(__float_as_uint(v[4 * q + 3]))
                                         : "memory");
                        }
                    }
                    fence_proxy_async_smem();
                    named_barrier_sync(1 + half, 128);
                    if (store_leader) {
                        tma_store_3d(&p.map_c, slab, static_cast<int32_t>(col), tc.m_tile * BM, tc.batch);
                        bulk_commit_group();
                    }
                } else if (row_ok) {
                    if (p.c_is_bf16)
                        store_chunk_bf16(static_cast<__nv_bfloat16*>(p.c) + c_off, v, valid);
                    else
                        store_chunk_f32(static_cast<float*>(p.c) + c_off, v, valid);
                }
            }
            if (p.dbias != nullptr && tc.n_tile == 0 && half == 0) {
                // Accumulator column bn holds sum_k op(A)[row, k] (the ones block).
                uint32_t r[16];
                tmem_ld_32x16(t_row + static_cast<uint32_t>(p.bn), r);
                tmem_ld_wait();
                if (row_ok) {
                    const float s = __uint_as_float(r[0]);
                    if (partial) {
                        p.ws_dbias[static_cast<int64_t>(tc.split) * p.m + row] = s;
                    } else {
                        const float prev = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[row] : 0.0f;
                        p.dbias[row] = prev + s;
                    }
                }
            }
            tc_fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[acc]));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
        // Outstanding TMA stores must complete before the shared memory goes away.
        if (store_leader) bulk_wait_group0();
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag) {
        // A wait ran out somewhere: give copies still in flight time to land
        // before the shared memory and TMEM are released.
        __nanosleep(200000);
    }
    tc_fence_before_thread_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_thread_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// C = epilogue(alpha * sum_s ws[s] + beta * C): fixed summation order s = 0..splits-1.
// Four consecutive columns per thread when the row length allows it.
__global__ void splitk_reduce_kernel(const GroupProblem p) {
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
    return 1024 /* alignment slack */ + kStages * kStageBytes + kStagingBytes + sizeof(Control);
}

cudaError_t launch_tc_grouped(const GroupParams& gp, int grid, cudaStream_t stream) {
    static int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(tc_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024);
        if (e != cudaSuccess) return e;
        configured_device = dev;
    }
    tc_grouped_kernel<<<grid, kThreads, tc_grouped_smem_bytes(), stream>>>(gp);
    count_launch(1);
    return cudaGetLastError();
}

cudaError_t launch_splitk_reduce(const GroupProblem& p, cudaStream_t stream) {
    const int64_t n4 = (p.n + 3) / 4;
    const int64_t total = static_cast<int64_t>(p.batch) * p.m * n4;
    const int64_t work = total > p.m ? total : p.m;
    const int block = 256;
    const int64_t grid = (work + block - 1) / block;
    splitk_reduce_kernel<<<static_cast<unsigned>(grid), block, 0, stream>>>(p);
    count_launch(1);
    return cudaGetLastError();
}

}  // namespace llmt_b200
