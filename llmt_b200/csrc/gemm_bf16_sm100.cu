// bf16 x bf16 -> fp32-accumulate GEMM for sm_100a: tcgen05 MMA with the
// accumulator in tensor memory, operands staged in 128-byte-swizzled shared
// memory by TMA, one persistent CTA per SM, warp-specialised:
//
//   warp 0      TMA producer   (one lane issues cp.async.bulk.tensor loads)
//   warp 1      MMA issuer     (one lane issues tcgen05.mma / tcgen05.commit; the
//                               warp also owns the TMEM allocation)
//   warps 2-9   epilogue       (tcgen05.ld the accumulator, apply
//                               alpha/beta/bias/GELU/cast, store C; two warps per
//                               TMEM lane quarter, each taking half the columns)
//
// Two rings of mbarriers connect them: full/empty per shared-memory stage and
// full/empty per TMEM accumulator buffer (two buffers, so the epilogue of tile
// i overlaps the main loop of tile i+1).
//
// The kernel computes llmt's row-major  C = alpha*op(A)*op(B) + beta*C
// (llmt: include/llmt/kernels/matmul.h:12-24) for all four transpose
// combinations.  A transposed operand is not copied: the tile is loaded as
// stored and described to the tensor core as "MN-major".
//
// No wait in here is unbounded: every mbarrier wait gives up after
// kWaitLimitNs, records why in the DeviceStatus word and makes the CTA drain
// and exit.
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
constexpr int kMaxStages = 8;
constexpr uint32_t kATileBytes = BM * BK * 2;
constexpr uint32_t kBlock64Bytes = 64 * BK * 2;  // one 64-wide MN-major block of a stage
// Fused dbias: every pipeline stage carries one extra 64-wide block of bf16 ones
// right behind its B tile, so that a tile of the first tile column can run its
// MMAs with N = BN + 16 and receive sum_k op(A)[row, k] in accumulator column BN.
constexpr uint32_t kOnesBytes = 64 * 128;
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr int kDbiasCols = 16;
// Epilogue staging: one 128-row x 32-column slab per column half (fp32: 128-byte rows,
// 128B swizzle; bf16: 64-byte rows, 64B swizzle), written by 4 warps, stored by TMA.
constexpr uint32_t kSlabBytes = 128 * 32 * 4;
constexpr uint32_t kStagingBytes = 2 * kSlabBytes;

struct __align__(8) Control {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
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
    int m_tile, n_tile, split, batch;
    int kb0, kb1;
};

__device__ __forceinline__ TileCoord decode_tile(const TcGemmParams& p, int64_t t) {
    TileCoord tc;
    tc.m_tile = static_cast<int>(t % p.tiles_m);
    int64_t r = t / p.tiles_m;
    tc.n_tile = static_cast<int>(r % p.tiles_n);
    r /= p.tiles_n;
    tc.split = static_cast<int>(r % p.splits);
    tc.batch = static_cast<int>(r / p.splits);
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

template <int BN, int A_MN, int B_MN, int DBIAS>
__global__ void __launch_bounds__(kThreads, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const TcGemmParams p, const int stages) {
    static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "tile width");
    static_assert(!DBIAS || BN <= 192, "dbias columns need room in TMEM");
    constexpr uint32_t kBTileBytes = BN * BK * 2;
    constexpr uint32_t kLoadBytes = kATileBytes + kBTileBytes;  // what TMA brings per stage
    constexpr uint32_t kStageBytes = kLoadBytes + (DBIAS ? kOnesBytes : 0);
    constexpr uint32_t kAccStride = BN + (DBIAS ? kDbiasCols : 0);  // TMEM columns per accumulator
    constexpr uint32_t kAccCols = 2 * kAccStride;
    constexpr uint32_t kTmemCols = kAccCols <= 128 ? 128 : (kAccCols <= 256 ? 256 : 512);
    constexpr uint32_t kIdesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
    constexpr uint32_t kIdescDbias = make_idesc_bf16(BM, BN + kDbiasCols, A_MN, B_MN);

    extern __shared__ uint8_t smem_raw[];
    // Swizzled tiles need 1024-byte alignment.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t staging_base = smem_base + static_cast<uint32_t>(stages) * kStageBytes;
    Control* ctl = reinterpret_cast<Control*>(smem_gen + static_cast<size_t>(stages) * kStageBytes +
                                              kStagingBytes);
    volatile int* abort_flag = &ctl->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&ctl->full[s]), 1);
            mbar_init(smem_u32(&ctl->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&ctl->tmem_full[a]), 1);
            mbar_init(smem_u32(&ctl->tmem_empty[a]), kEpilogueWarps);
        }
        ctl->abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        if (p.c_tma) prefetch_tensormap(&map_c);
    }
    if (DBIAS) {
        // bf16 1.0 everywhere: the block reads the same under any swizzle or major.
        for (int st = 0; st < stages; ++st) {
            uint32_t* ones = reinterpret_cast<uint32_t*>(smem_gen + static_cast<size_t>(st) * kStageBytes +
                                                         kLoadBytes);
            for (int i = threadIdx.x; i < static_cast<int>(kOnesBytes / 4); i += kThreads)
                ones[i] = 0x3F803F80u;
        }
        fence_proxy_async_smem();
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
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                const TileCoord tc = decode_tile(p, t);
                const int m0 = tc.m_tile * BM, n0 = tc.n_tile * BN;
                for (int kb = tc.kb0; kb < tc.kb1; ++kb) {
                    ok = bounded_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abort_flag,
                                      p.status, kDevWaitSmemEmpty, stage);
                    if (!ok) break;
                    const uint32_t full = smem_u32(&ctl->full[stage]);
                    const uint32_t a_dst = smem_base + static_cast<uint32_t>(stage) * kStageBytes;
                    const uint32_t b_dst = a_dst + kATileBytes;
                    mbar_arrive_expect_tx(full, kLoadBytes);
                    const int k0 = kb * BK;
                    if (A_MN) {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_3d(a_dst + j * kBlock64Bytes, &map_a, full, m0 + 64 * j, k0,
                                        tc.batch);
                    } else {
                        tma_load_3d(a_dst, &map_a, full, k0, m0, tc.batch);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_3d(b_dst + j * kBlock64Bytes, &map_b, full, n0 + 64 * j, k0,
                                        tc.batch);
                    } else {
                        tma_load_3d(b_dst, &map_b, full, k0, n0, tc.batch);
                    }
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // K-major: a k-step is 32 bytes along the swizzled row, LBO unused (16), SBO 1024.
            // MN-major: a k-step is 16 k-rows of 128 bytes, LBO = one 64-wide block, SBO 1024.
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            constexpr uint32_t kStepA = (A_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            constexpr uint32_t kStepB = (B_MN ? UMMA_K * 128 : UMMA_K * 2) >> 4;
            const uint32_t a_lo_base = (smem_base >> 4) | (((A_MN ? kBlock64Bytes : 16u) >> 4) << 16);
            const uint32_t b_lo_base = ((smem_base + kATileBytes) >> 4) | (((B_MN ? kBlock64Bytes : 16u) >> 4) << 16);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
                const TileCoord tc = decode_tile(p, t);
                ok = bounded_wait(smem_u32(&ctl->tmem_empty[acc]), acc_phase ^ 1u, abort_flag,
                                  p.status, kDevWaitTmemEmpty, acc);
                if (!ok) break;
                tc_fence_after_thread_sync();
                const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc) * kAccStride;
                // Tiles of the first tile column also multiply the ones block behind B.
                const uint32_t idesc = (DBIAS && tc.n_tile == 0) ? kIdescDbias : kIdesc;
                for (int kb = tc.kb0; kb < tc.kb1; ++kb) {
                    ok = bounded_wait(smem_u32(&ctl->full[stage]), phase, abort_flag, p.status,
                                      kDevWaitSmemFull, stage);
                    if (!ok) break;
                    tc_fence_after_thread_sync();
                    // Descriptors differ between k-steps and stages only in the 14-bit
                    // start-address field, so the issuing thread does one add per operand.
                    const uint32_t stage_off = static_cast<uint32_t>(stage) * (kStageBytes >> 4);
                    const uint32_t a_lo = a_lo_base + stage_off;
                    const uint32_t b_lo = b_lo_base + stage_off;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t da = (static_cast<uint64_t>(kDescHi) << 32) |
                                            static_cast<uint64_t>(a_lo + kk * kStepA);
                        const uint64_t db = (static_cast<uint64_t>(kDescHi) << 32) |
                                            static_cast<uint64_t>(b_lo + kk * kStepB);
                        umma_bf16(d_tmem, da, db, idesc, (kb > tc.kb0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&ctl->empty[stage]));  // frees the stage when the MMAs retire
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
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
        constexpr int kHalfCols = BN / 2;
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; ok && t < p.total_tiles; t += gridDim.x) {
            const TileCoord tc = decode_tile(p, t);
            ok = bounded_wait(smem_u32(&ctl->tmem_full[acc]), acc_phase, abort_flag, p.status,
                              kDevWaitTmemFull, acc);
            if (!ok) break;
            tc_fence_after_thread_sync();
            const int64_t row = static_cast<int64_t>(tc.m_tile) * BM + quarter * 32 + lane;
            const bool row_ok = row < p.m;
            const int64_t n0 = static_cast<int64_t>(tc.n_tile) * BN;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                   static_cast<uint32_t>(acc) * kAccStride;
            const bool partial = p.splits > 1;
            const bool via_tma = p.c_tma && !partial;
            const int tile_row = quarter * 32 + lane;  // row inside the 128-row tile
            const uint32_t slab = staging_base + static_cast<uint32_t>(half) * kSlabBytes;
            const bool store_leader = (warp == 2 + 4 * half) && lane == 0;
#pragma unroll 1
            for (int c0 = half * kHalfCols; c0 < (half + 1) * kHalfCols; c0 += 32) {
                if (n0 + c0 >= p.n) break;  // warp-uniform
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
                                     ((static_cast<int64_t>(tc.batch) * p.splits + tc.split) * p.m + row) * p.n +
                                     col;
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
                // through registers instead (warp-uniform and the same in all warps of a half).
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
                        tma_store_3d(&map_c, slab, static_cast<int32_t>(col), tc.m_tile * BM, tc.batch);
                        bulk_commit_group();
                    }
                } else if (row_ok) {
                    if (p.c_is_bf16)
                        store_chunk_bf16(static_cast<__nv_bfloat16*>(p.c) + c_off, v, valid);
                    else
                        store_chunk_f32(static_cast<float*>(p.c) + c_off, v, valid);
                }
            }
            if (DBIAS && tc.n_tile == 0 && half == 0) {
                // Accumulator column BN holds sum_k op(A)[row, k] (the ones block).
                uint32_t r[16];
                tmem_ld_32x16(t_row + static_cast<uint32_t>(BN), r);
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
        if ((warp == 2 || warp == 6) && lane == 0) bulk_wait_group0();
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
__global__ void splitk_reduce_kernel(const TcGemmParams p) {
    const int64_t total = static_cast<int64_t>(p.batch) * p.m * p.n;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < total) {
        const int64_t col = i % p.n;
        const int64_t row = (i / p.n) % p.m;
        const int64_t b = i / (p.n * p.m);
        const float* src = p.ws + (b * p.splits * p.m + row) * p.n + col;
        float acc = 0.0f;
        for (int s = 0; s < p.splits; ++s) acc += src[static_cast<int64_t>(s) * p.m * p.n];
        float v = p.alpha * acc;
        const int64_t c_off = b * p.stride_c + row * p.ldc + col;
        if (p.beta != 0.0f)
            v += p.beta * (p.c_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.c)[c_off])
                                       : static_cast<const float*>(p.c)[c_off]);
        if (p.epi_flags & kEpiBias)
            v += p.bias_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col])
                                : static_cast<const float*>(p.bias)[col];
        if (p.epi_flags & kEpiGelu) v = gelu_tanh_fast(v);
        if (p.c_is_bf16)
            static_cast<__nv_bfloat16*>(p.c)[c_off] = __float2bfloat16_rn(v);
        else
            static_cast<float*>(p.c)[c_off] = v;
    }
    if (p.dbias != nullptr && i < p.m) {
        float acc = 0.0f;
        for (int s = 0; s < p.splits; ++s) acc += p.ws_dbias[static_cast<int64_t>(s) * p.m + i];
        const float prev = p.dbias_beta != 0.0f ? p.dbias_beta * p.dbias[i] : 0.0f;
        p.dbias[i] = prev + acc;
    }
}

template <int BN, int A_MN, int B_MN, int DBIAS>
cudaError_t launch_one(const TcPlan& plan, const CUtensorMap& ma, const CUtensorMap& mb,
                       const CUtensorMap& mc, const TcGemmParams& p, cudaStream_t stream) {
    auto kern = tc_gemm_kernel<BN, A_MN, B_MN, DBIAS>;
    static bool configured = false;  // per instantiation; the attribute is sticky per device context
    static int configured_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured || configured_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
        configured_device = dev;
    }
    kern<<<plan.grid, kThreads, plan.smem_bytes, stream>>>(ma, mb, mc, p, plan.stages);
    count_launch(1);
    return cudaGetLastError();
}

template <int BN, int DBIAS>
cudaError_t launch_major(const TcPlan& plan, int a_mn, int b_mn, const CUtensorMap& ma,
                         const CUtensorMap& mb, const CUtensorMap& mc, const TcGemmParams& p,
                         cudaStream_t stream) {
    if (a_mn) {
        if (b_mn) return launch_one<BN, 1, 1, DBIAS>(plan, ma, mb, mc, p, stream);
        return launch_one<BN, 1, 0, DBIAS>(plan, ma, mb, mc, p, stream);
    }
    if (b_mn) return launch_one<BN, 0, 1, DBIAS>(plan, ma, mb, mc, p, stream);
    return launch_one<BN, 0, 0, DBIAS>(plan, ma, mb, mc, p, stream);
}

}  // namespace

size_t tc_smem_bytes(int bn, int stages, bool dbias) {
    const size_t stage = kATileBytes + static_cast<size_t>(bn) * BK * 2;
    return 1024 /* alignment slack */ + (stage + (dbias ? kOnesBytes : 0)) * stages + kStagingBytes +
           sizeof(Control);
}

cudaError_t launch_tc_gemm(const TcPlan& plan, int a_mn, int b_mn, const CUtensorMap& ma,
                           const CUtensorMap& mb, const CUtensorMap& mc, const TcGemmParams& p,
                           cudaStream_t stream) {
    const bool dbias = p.dbias != nullptr;
    if (dbias) {
        switch (plan.bn) {
            case 64: return launch_major<64, 1>(plan, a_mn, b_mn, ma, mb, mc, p, stream);
            case 128: return launch_major<128, 1>(plan, a_mn, b_mn, ma, mb, mc, p, stream);
            case 192: return launch_major<192, 1>(plan, a_mn, b_mn, ma, mb, mc, p, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    switch (plan.bn) {
        case 64: return launch_major<64, 0>(plan, a_mn, b_mn, ma, mb, mc, p, stream);
        case 128: return launch_major<128, 0>(plan, a_mn, b_mn, ma, mb, mc, p, stream);
        case 192: return launch_major<192, 0>(plan, a_mn, b_mn, ma, mb, mc, p, stream);
        case 256: return launch_major<256, 0>(plan, a_mn, b_mn, ma, mb, mc, p, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_splitk_reduce(const TcGemmParams& p, cudaStream_t stream) {
    const int64_t total = static_cast<int64_t>(p.batch) * p.m * p.n;
    const int64_t work = total > p.m ? total : p.m;
    const int block = 256;
    const int64_t grid = (work + block - 1) / block;
    splitk_reduce_kernel<<<static_cast<unsigned>(grid), block, 0, stream>>>(p);
    count_launch(1);
    return cudaGetLastError();
}

}  // namespace llmt_b200
