// extern "C" front end: argument validation, plan selection, TMA descriptor
// encoding and kernel launch.  Mirrors the checks llmt performs before it calls
// cuBLASLt (llmt: src/kernels/matmul.cpp:175-214) but reports them as status
// codes instead of aborting.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <initializer_list>

#include "../../include/llmt_b200.h"
#include "common.h"

namespace llmt_b200 {

namespace {

bool pairs_enabled();

thread_local char g_err[512] = "";
std::atomic<uint64_t> g_launches{0};

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return status;
}

__device__ DeviceStatus g_device_status;

// Split-K scratch for llmt_b200_gemm_static_scratch(): a fixed array inside the
// library image, so that entry point never has to ask anyone for memory.  Every
// GPU that loads the library carries these bytes until the process exits.
constexpr size_t kStaticScratchBytes = LLMT_B200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device.  In host code the
// array's name is only a handle for the runtime, not something a kernel can
// dereference; the real address comes from cudaGetSymbolAddress, asked once per
// device with that device current, and is cached here.
void* static_scratch_ptr(cudaError_t* err) {
    static void* ptrs[64] = {nullptr};
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        *err = cudaGetSymbolAddress(&p, g_static_scratch);
        if (*err != cudaSuccess) return nullptr;
        ptrs[dev] = p;
    }
    return ptrs[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// SMs the persistent kernels may occupy: 0 = all of them.  A data-parallel caller lowers it
// by the number of CTAs its collective library runs, so that a gradient all-reduce on a
// second stream finds free SMs while a GEMM launch is resident.
int g_sm_budget = 0;

int sm_count() {
    static int cached = 0;
    if (cached == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            cached = n;
        else
            return 148;  // B200; used only for planning queries made without a device
    }
    return g_sm_budget > 0 && g_sm_budget < cached ? g_sm_budget : cached;
}

// Cost of one 64-deep k-block of a tile in SM cycles.  Two bounds: the tensor pipe (2*bn
// cycles for the CTA's 128 rows, about 15 % more once the per-k-block commit is counted:
// 590 measured for bn = 256) and the rate at which one SM pulls operand bytes out of L2
// (about 76 bytes per cycle measured; a single CTA stages 128 + bn rows of 128 bytes).  A single
// CTA's 256-wide tile is load-bound (measured 610-665), a pair's is not; a pair's narrower
// tiles cost more per column than the model of either bound says (measured: 128-wide tiles
// take three quarters of the time of 256-wide ones), so they only pay against wave
// quantisation.
int kblock_cost(int bn, bool pairs) {
    if (pairs) {
        // measured: 590 for a 256-wide tile, the same per column at 192, and no less than 445
        const int c = 590 * bn / 256;
        return c > 445 ? c : 445;
    }
    const int mma = bn * 2 * 115 / 100;
    const int load = (128 + bn) * 128 / 76;
    return mma > load ? mma : load;
}

int ceil_div(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

// Debug hook, read once: LLMT_B200_DBIAS_TICKETS=1 keeps the ticket form of the fused dbias.
bool dbias_tickets_forced() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("LLMT_B200_DBIAS_TICKETS");
        v = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}

// dbias_mode: 0 none, 1 column sums of A stored [k, m] (two phases), 2 row sums of A stored [m, k].
void finish_plan(TcPlan* pl, int64_t m, int64_t n, int64_t k, int64_t batch, int dbias_mode, int bn, int splits,
                 bool pairs) {
    pl->bn = bn;
    pl->pairs = pairs ? 1 : 0;
    pl->tiles_m = ceil_div(m, pairs ? 256 : 128);
    pl->tiles_n = ceil_div(n, bn);
    pl->kblocks_total = ceil_div(k, 64);
    if (splits > pl->kblocks_total) splits = pl->kblocks_total;
    if (splits < 1) splits = 1;
    pl->kblocks_per_split = ceil_div(pl->kblocks_total, splits);
    pl->splits = pl->kblocks_total > 0 ? ceil_div(pl->kblocks_total, pl->kblocks_per_split) : 1;
    pl->num_tiles = static_cast<int64_t>(pl->tiles_m) * pl->tiles_n * pl->splits * batch;
    pl->workspace_bytes = 0;
    if (pl->splits > 1) {
        size_t ws = static_cast<size_t>(batch) * pl->splits * m * n * sizeof(float);
        pl->workspace_bytes = (ws + 255) / 256 * 256;
    }
    // The fused dbias runs as tickets of its own, independent of the product's tiling.
    const int cg = pairs ? 2 : 1;
    pl->dbias_mode = k > 0 ? dbias_mode : 0;
    // Column sums of a single (unbatched) product come from the A stages in shared memory (mode 3);
    // the ticket form (mode 1) remains for batches.
    if (pl->dbias_mode == 1 && batch <= 1 && !dbias_tickets_forced()) pl->dbias_mode = 3;
    pl->colsum_tiles = pl->dbias_rows = pl->fin_tiles = 0;
    pl->ws_dbias_off = 0;
    if (pl->dbias_mode == 3) {
        if (pl->splits > 1) {  // one row of sums per split; the split-K reduction adds them
            pl->ws_dbias_off = pl->workspace_bytes;
            pl->workspace_bytes += (static_cast<size_t>(pl->splits) * m * sizeof(float) + 255) / 256 * 256;
        }
    } else if (pl->dbias_mode == 1) {
        // chunks of at least 64 rows of A, at most 512 chunks
        const int64_t rows = ceil_div(k, 512) > 64 ? ceil_div(k, 512) : 64;
        pl->dbias_rows = static_cast<int>(rows);
        pl->colsum_tiles = ceil_div(k, rows);
        pl->fin_tiles = ceil_div(m, static_cast<int64_t>(tc_dbias_finish_per_cta()) * cg);
        pl->ws_dbias_off = pl->workspace_bytes;
        pl->workspace_bytes += (static_cast<size_t>(pl->colsum_tiles) * m * sizeof(float) + 255) / 256 * 256;
    } else if (pl->dbias_mode == 2) {
        pl->colsum_tiles = ceil_div(m, static_cast<int64_t>(tc_dbias_rows_per_cta()) * cg);
    }
}

// Split-K factor for a problem launched on its own: only when its tiles cannot fill
// the machine and the reduction is long enough to share.
int choose_splits(int64_t tiles, int kblocks_total, int sms) {
    int splits = 1;
    if (tiles * 2 <= sms && kblocks_total >= 8) {
        splits = static_cast<int>(sms / tiles);
        const int max_by_k = kblocks_total / 4;
        if (splits > max_by_k) splits = max_by_k;
        if (splits < 1) splits = 1;
    }
    return splits;
}

// Plan of a problem launched on its own: tile width and split count from a cycle model
// of waves of equal tiles.  A pure function of its arguments.
// `pairs`: the launch uses CTA pairs (256-row tiles, `units` = number of pairs); with
// MN-major B a pair needs a tile width that is a multiple of 128.
// `epi_step`: estimated cycles of one 32-column epilogue step of this problem, `c_bf16`: its result type.
// A tile is done when its main loop AND its epilogue are (they overlap across tiles): an epilogue
// warp takes every other 128-byte column unit, so a 192-wide bf16 tile (three units) costs it as many
// steps as a 256-wide one.
TcPlan make_plan(int64_t m, int64_t n, int64_t k, int64_t batch, int dbias_mode, int units,
                 int force_bn, int force_splits, bool pairs, bool b_mn, int epi_step = 1000, bool c_bf16 = true) {
    const int sms = units;
    const int cands[4] = {256, 192, 128, 64};
    const int tiles_m = ceil_div(m, pairs ? 256 : 128);
    const int kblocks_total = ceil_div(k, 64);
    int best_bn = 0, best_splits = 1;
    int64_t best_cost = 0;
    for (int bn : cands) {
        if (force_bn != 0 && bn != force_bn) continue;
        if (pairs && (bn == 64 || (b_mn && bn % 128 != 0))) continue;
        // Never pick a tile wider than needed when a narrower one covers n in one column.
        if (force_bn == 0 && bn > 64 && n <= bn - 64 && !(pairs && bn == 128)) continue;
        const int64_t tiles = static_cast<int64_t>(tiles_m) * ceil_div(n, bn) * batch;
        int splits = force_splits > 0 ? force_splits : choose_splits(tiles, kblocks_total, sms);
        if (splits > kblocks_total) splits = kblocks_total > 0 ? kblocks_total : 1;
        const int kps = ceil_div(kblocks_total, splits);
        const int64_t waves = (tiles * splits + sms - 1) / sms;
        // Estimated cycles: per wave the longer of main loop and epilogue, one pass over the partials when split.
        const int unit_cols = (c_bf16 && splits == 1) ? 64 : 32;
        const int steps = ((bn / unit_cols + 1) / 2) * (unit_cols / 32);
        const int64_t main_loop = static_cast<int64_t>(kblock_cost(bn, pairs)) * (kps > 0 ? kps : 1);
        const int64_t epilogue = static_cast<int64_t>(steps) * (splits == 1 ? epi_step : 1000);
        int64_t cost = waves * ((main_loop > epilogue ? main_loop : epilogue) + 4 * bn);
        if (splits > 1) cost += static_cast<int64_t>(splits) * 64 + 4000;
        if (best_bn == 0 || cost < best_cost) {
            best_bn = bn;
            best_cost = cost;
            best_splits = splits;
        }
    }
    TcPlan pl{};
    if (best_bn == 0) best_bn = pairs ? 128 : 64;
    finish_plan(&pl, m, n, k, batch, dbias_mode, best_bn, best_splits, pairs);
    return pl;
}

// Plan of a problem that shares its launch with others: the queue is dynamic, so wave
// quantisation of one problem does not matter; take the widest tile that wastes nothing
// and split only reductions that are longer than the average load of an SM.
TcPlan make_group_plan(int64_t m, int64_t n, int64_t k, int64_t batch, int dbias_mode, int sms,
                       int64_t group_kblock_tiles, int force_bn, int force_splits, bool pairs, bool b_mn) {
    int bn = 256;
    if (n <= 64) bn = pairs ? 128 : 64;
    else if (n <= 128) bn = 128;
    else if (n <= 192) bn = (pairs && b_mn) ? 256 : 192;
    if (force_bn != 0) bn = force_bn;
    const int kblocks_total = ceil_div(k, 64);
    int splits = 1;
    if (force_splits > 0) {
        splits = force_splits;
    } else {
        const int64_t avg = group_kblock_tiles / sms;  // k-blocks per SM if perfectly balanced
        const int64_t target = avg > 16 ? avg : 16;
        if (kblocks_total > target + target / 4) splits = ceil_div(kblocks_total, target);
        const int max_by_k = kblocks_total / 4 > 0 ? kblocks_total / 4 : 1;
        if (splits > max_by_k) splits = max_by_k;
    }
    TcPlan pl{};
    finish_plan(&pl, m, n, k, batch, dbias_mode, bn, splits, pairs);
    return pl;
}

// CTA pairs (cta_group::2, 256-row tiles) halve the B bytes each SM stages per flop: a single
// CTA's 128x256 tile is bound by the rate at which one SM pulls operands out of L2 (48 KB per
// k-block), a pair's is not (32 KB).  Measured +4..10 % on products without a fused dbias,
// with operands in L2 or streaming from HBM alike, so pairs are the default for those;
// LLMT_B200_PAIRS=0 keeps every launch on single CTAs (for comparisons), plan_cta_pairs
// chooses per call.
bool pairs_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("LLMT_B200_PAIRS");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}
// Whether a problem CAN run on CTA pairs, and whether the library chooses to.
bool pair_capable(const llmt_b200_gemm_desc* d) {
    if (d->m <= 128 || d->plan_tile_n == 64) return false;
    const bool b_mn = d->trans_b == 0;
    if (b_mn && d->plan_tile_n == 192) return false;
    return true;
}
bool pair_eligible(const llmt_b200_gemm_desc* d) {
    if (!pair_capable(d) || d->plan_cta_pairs == 1) return false;
    if (d->plan_cta_pairs == 2) return true;
    return pairs_enabled();
}
// Debug hook, read once: LLMT_B200_STATIC=1 replaces the dynamic tile queue by a static order.
bool static_schedule_forced() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("LLMT_B200_STATIC");
        v = (e != nullptr && e[0] == '1') ? 1 : 0;
    }
    return v == 1;
}
int pair_units() {
    static int forced = -1;  // debug hook, read once
    if (forced < 0) {
        const char* e = getenv("LLMT_B200_PAIR_UNITS");
        forced = (e != nullptr && atoi(e) > 0) ? atoi(e) : 0;
    }
    if (forced > 0) return forced;
    const int r = max_resident_pairs();
    const int by_sm = sm_count() / 2;
    return (r > 0 && r < by_sm) ? r : by_sm;
}
int dbias_mode_of(const llmt_b200_gemm_desc* d) { return d->dbias == nullptr ? 0 : (d->trans_a ? 1 : 2); }
// The row-wise epilogues see whole reductions: such a problem is never split along k.
int splits_wanted(const llmt_b200_gemm_desc* d) {
    return (d->epilogue & (LLMT_B200_EPI_GELU_BWD | LLMT_B200_EPI_SAVE_PRE)) ? 1 : d->plan_splits;
}
TcPlan plan_single(const llmt_b200_gemm_desc* d) {
    const bool pairs = pair_eligible(d);
    const int epi_step = 1000 + ((d->epilogue & LLMT_B200_EPI_BIAS) ? 100 : 0) + ((d->epilogue & LLMT_B200_EPI_GELU) ? 500 : 0) +
                         (d->beta != 0.0f ? 300 : 0);
    return make_plan(d->m, d->n, d->k, d->batch, dbias_mode_of(d), pairs ? pair_units() : sm_count(),
                     d->plan_tile_n, splits_wanted(d), pairs, d->trans_b == 0, epi_step, d->dtype_c == LLMT_B200_BF16);
}

bool overlaps(const void* p, size_t pb, const void* q, size_t qb) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p), b = reinterpret_cast<uintptr_t>(q);
    return a < b + qb && b < a + pb;
}

struct Checked {
    int64_t a_rows, a_cols, b_rows, b_cols;
    size_t a_bytes, b_bytes, c_bytes;  // extent of each operand in memory (0 for an empty problem)
    bool bf16;
};

// Shape/pointer contract; the order and wording follow llmt's check()
// (src/kernels/matmul.cpp:175-214) where a counterpart exists.
// c_optional: C may be null (the caller does not want the product itself stored).
int validate(const llmt_b200_gemm_desc* d, const void* c, const void* a, const void* b, Checked* out,
             bool c_optional = false) {
    if (d == nullptr) return fail(LLMT_B200_ERR_INVALID, "matmul: null descriptor");
    if ((c == nullptr && !c_optional) || a == nullptr || b == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "matmul: invalid tensor (null data)");
    if (d->m < 0 || d->n < 0 || d->k < 0 || d->batch < 0)
        return fail(LLMT_B200_ERR_INVALID, "matmul: negative dimension");
    // Tile counts and TMA coordinates are 32-bit, and a coordinate may point up to a tile past the end.
    constexpr int64_t kMaxDim = 0x7fffffff - 1024;
    if (d->m > kMaxDim || d->n > kMaxDim || d->k > kMaxDim || d->batch > kMaxDim)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: dimension above 2^31 - 1025");
    if (d->dtype_ab != LLMT_B200_FP32 && d->dtype_ab != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: dtype code %d not supported", d->dtype_ab);
    if (d->dtype_c != LLMT_B200_FP32 && d->dtype_c != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: dtype code %d not supported", d->dtype_c);
    if (d->dtype_ab == LLMT_B200_FP32 && d->dtype_c != LLMT_B200_FP32)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: mixed dtypes in one matmul (fp32 inputs need fp32 C)");
    out->bf16 = d->dtype_ab == LLMT_B200_BF16;
    out->a_rows = d->trans_a ? d->k : d->m;
    out->a_cols = d->trans_a ? d->m : d->k;
    out->b_rows = d->trans_b ? d->n : d->k;
    out->b_cols = d->trans_b ? d->k : d->n;
    if (d->lda < out->a_cols || d->ldb < out->b_cols || d->ldc < d->n)
        return fail(LLMT_B200_ERR_INVALID, "matmul: row pitch smaller than the row (lda=%lld ldb=%lld ldc=%lld)",
                    (long long)d->lda, (long long)d->ldb, (long long)d->ldc);
    const bool two_level = d->batch_inner > 0;
    if (two_level) {
        if (d->batch_inner > d->batch || d->batch % d->batch_inner != 0)
            return fail(LLMT_B200_ERR_INVALID, "matmul: batch_inner must divide batch");
        if (d->stride_a < 0 || d->stride_b < 0 || d->stride_c < 0 || d->stride_a_outer < 0 ||
            d->stride_b_outer < 0 || d->stride_c_outer < 0)
            return fail(LLMT_B200_ERR_INVALID, "matmul: negative batch stride");
        if (d->dbias != nullptr) return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: dbias with a batched product is not defined");
    } else if (d->batch > 1) {
        if (d->stride_a < (out->a_rows - 1) * d->lda + out->a_cols ||
            d->stride_b < (out->b_rows - 1) * d->ldb + out->b_cols ||
            d->stride_c < (d->m - 1) * d->ldc + d->n)
            return fail(LLMT_B200_ERR_INVALID, "matmul: batch stride smaller than one matrix");
    }
    if (d->plan_tile_n != 0 && d->plan_tile_n != 64 && d->plan_tile_n != 128 &&
        d->plan_tile_n != 192 && d->plan_tile_n != 256)
        return fail(LLMT_B200_ERR_INVALID, "matmul: plan_tile_n must be 0, 64, 128, 192 or 256");
    if (d->plan_cta_pairs < 0 || d->plan_cta_pairs > 2)
        return fail(LLMT_B200_ERR_INVALID, "matmul: plan_cta_pairs must be 0, 1 or 2");
    if (d->plan_cta_pairs == 2 && (d->m <= 128 || d->plan_tile_n == 64 || (d->trans_b == 0 && d->plan_tile_n == 192)))
        return fail(LLMT_B200_ERR_INVALID, "matmul: CTA pairs need m > 128 and a tile width of 128 or 256 "
                    "(192 only when B is stored [n, k])");
    if (d->plan_splits < 0) return fail(LLMT_B200_ERR_INVALID, "matmul: negative plan_splits");
    if (d->epilogue & LLMT_B200_EPI_SAVE_PRE) {
        if (!(d->epilogue & LLMT_B200_EPI_GELU) || (d->epilogue & LLMT_B200_EPI_GELU_BWD))
            return fail(LLMT_B200_ERR_INVALID, "matmul: EPI_SAVE_PRE goes with EPI_GELU (and EPI_BIAS) only");
        if (d->aux == nullptr) return fail(LLMT_B200_ERR_INVALID, "matmul: EPI_SAVE_PRE set but aux is null");
        if (d->dtype_ab != LLMT_B200_BF16)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: EPI_SAVE_PRE needs bf16 operands");
        if (d->dbias != nullptr) return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: EPI_SAVE_PRE with dbias is not defined");
    }
    if ((d->epilogue & ~(LLMT_B200_EPI_BIAS | LLMT_B200_EPI_GELU | LLMT_B200_EPI_GELU_BWD | LLMT_B200_EPI_SAVE_PRE)) != 0)
        return fail(LLMT_B200_ERR_INVALID, "matmul: unknown epilogue flags 0x%x", d->epilogue);
    if (d->epilogue & LLMT_B200_EPI_GELU_BWD) {
        if (d->epilogue != LLMT_B200_EPI_GELU_BWD)
            return fail(LLMT_B200_ERR_INVALID, "matmul: EPI_GELU_BWD stands alone among the epilogue flags");
        if (d->aux == nullptr) return fail(LLMT_B200_ERR_INVALID, "matmul: EPI_GELU_BWD set but aux is null");
        if (d->dtype_ab != LLMT_B200_BF16)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: EPI_GELU_BWD needs bf16 operands");
        if (d->beta != 0.0f) return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: EPI_GELU_BWD needs beta = 0");
        if (d->dbias != nullptr) return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: EPI_GELU_BWD with dbias is not defined");
    }
    if ((d->epilogue & LLMT_B200_EPI_BIAS) && d->bias == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "matmul: EPI_BIAS set but bias is null");
    if ((d->epilogue & LLMT_B200_EPI_BIAS) && d->bias_dtype != LLMT_B200_FP32 &&
        d->bias_dtype != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: bias dtype code %d not supported", d->bias_dtype);
    if (d->dbias != nullptr) {
        if (d->batch > 1)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: dbias with a batched product is not defined");
    }
    // Aliasing: C is updated in place; it must not overlap an input.
    const size_t es_ab = out->bf16 ? 2 : 4, es_c = d->dtype_c == LLMT_B200_BF16 ? 2 : 4;
    const int64_t nb = d->batch > 0 ? d->batch : 1;
    if (d->m > 0 && d->n > 0 && d->k > 0) {
        // extent of the batch: last item's offset (for a two-level layout: last of the last group)
        auto batch_span = [&](int64_t stride, int64_t stride_outer) -> int64_t {
            if (two_level) return (d->batch_inner - 1) * stride + (nb / d->batch_inner - 1) * stride_outer;
            return (nb - 1) * (nb > 1 ? stride : 0);
        };
        const size_t a_bytes = static_cast<size_t>(batch_span(d->stride_a, d->stride_a_outer) +
                                                   (out->a_rows - 1) * d->lda + out->a_cols) * es_ab;
        const size_t b_bytes = static_cast<size_t>(batch_span(d->stride_b, d->stride_b_outer) +
                                                   (out->b_rows - 1) * d->ldb + out->b_cols) * es_ab;
        const size_t c_bytes = c == nullptr ? 0 : static_cast<size_t>(batch_span(d->stride_c, d->stride_c_outer) +
                                                                      (d->m - 1) * d->ldc + d->n) * es_c;
        out->a_bytes = a_bytes; out->b_bytes = b_bytes; out->c_bytes = c_bytes;
        if (c_bytes != 0 && (overlaps(c, c_bytes, a, a_bytes) || overlaps(c, c_bytes, b, b_bytes)))
            return fail(LLMT_B200_ERR_INVALID, "matmul: C overlaps an input");
        // Nothing the call writes (C, dbias, workspace) may overlap anything else it touches.
        const size_t dbias_bytes = d->dbias != nullptr ? static_cast<size_t>(d->m) * 4 : 0;
        const size_t bias_bytes = (d->epilogue & LLMT_B200_EPI_BIAS)
                                      ? static_cast<size_t>(d->n) * (d->bias_dtype == LLMT_B200_BF16 ? 2 : 4) : 0;
        const size_t ws_bytes = d->workspace != nullptr ? static_cast<size_t>(d->workspace_bytes) : 0;
        struct Range { const void* p; size_t n; const char* what; };
        // aux has C's extent; it is read (EPI_GELU_BWD) or written (EPI_SAVE_PRE)
        const size_t aux_r = (d->epilogue & LLMT_B200_EPI_GELU_BWD) ? c_bytes : 0;
        const size_t aux_w = (d->epilogue & LLMT_B200_EPI_SAVE_PRE) ? c_bytes : 0;
        const Range reads[5] = {{a, a_bytes, "A"}, {b, b_bytes, "B"}, {d->bias, bias_bytes, "bias"}, {c, c_bytes, "C"},
                                {d->aux, aux_r, "aux"}};
        const Range writes[3] = {{d->dbias, dbias_bytes, "dbias"}, {d->workspace, ws_bytes, "workspace"}, {d->aux, aux_w, "aux"}};
        if (aux_r != 0 && overlaps(c, c_bytes, d->aux, aux_r)) return fail(LLMT_B200_ERR_INVALID, "matmul: C overlaps aux");
        for (const Range& w : writes) {
            if (w.n == 0) continue;
            for (const Range& r : reads)
                if (r.n != 0 && overlaps(w.p, w.n, r.p, r.n))
                    return fail(LLMT_B200_ERR_INVALID, "matmul: %s overlaps %s", w.what, r.what);
        }
        if (dbias_bytes != 0 && ws_bytes != 0 && overlaps(d->dbias, dbias_bytes, d->workspace, ws_bytes))
            return fail(LLMT_B200_ERR_INVALID, "matmul: dbias overlaps workspace");
    }
    return LLMT_B200_OK;
}

// Tensor map over row-major matrices [rows, cols] (pitch ld) in a batch laid out on two levels:
// `inner` items `stride` elements apart form a group, `outer` groups are `stride_outer` elements
// apart (a plain batch is one group).  Box of box_cols x box_rows elements of one matrix.
// elem_bytes 2 = bf16, 4 = fp32.
struct BatchLayout {
    int64_t inner = 1, stride = 0, outer = 1, stride_outer = 0;
};

BatchLayout batch_layout(int64_t batch, int64_t batch_inner, int64_t stride, int64_t stride_outer) {
    BatchLayout bl;
    if (batch_inner > 0) {
        bl.inner = batch_inner; bl.stride = stride; bl.outer = batch / batch_inner; bl.stride_outer = stride_outer;
    } else if (batch > 1) {
        bl.inner = batch; bl.stride = stride;
    }
    return bl;
}

int encode_map(CUtensorMap* map, const void* base, int elem_bytes, int64_t rows, int64_t cols,
               int64_t ld, const BatchLayout& bl, int box_cols, int box_rows, CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(LLMT_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    // a dimension of extent 1 still needs a stride that passes the encoder's checks
    const cuuint64_t one_matrix = static_cast<cuuint64_t>(rows) * ld;
    const cuuint64_t s1 = bl.inner > 1 ? static_cast<cuuint64_t>(bl.stride) : one_matrix;
    const cuuint64_t s2 = bl.outer > 1 ? static_cast<cuuint64_t>(bl.stride_outer) : s1 * static_cast<cuuint64_t>(bl.inner);
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                          static_cast<cuuint64_t>(bl.inner), static_cast<cuuint64_t>(bl.outer)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(ld) * elem_bytes, s1 * elem_bytes, s2 * elem_bytes};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                          4, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(LLMT_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d "
                    "(rows=%lld cols=%lld ld=%lld batch=%lld x %lld)", static_cast<int>(r),
                    (long long)rows, (long long)cols, (long long)ld, (long long)bl.inner, (long long)bl.outer);
    return LLMT_B200_OK;
}

// Encoded tensor maps are kept: a map is a pure function of (address, element size, shape,
// pitches, box, swizzle), a training step calls the same GEMMs on the same buffers over and
// over, and cuTensorMapEncodeTiled is the most expensive thing the host does per call.  This
// is the part of llmt's AlgoCache (include/llmt/kernels/algo_cache.h:18-42: resolve once per
// problem, replay) that has a cost worth caching here; the plan itself is recomputed, being a
// few integer operations.  Direct-mapped, per host thread, no device state.
struct MapKey {
    const void* base;
    int64_t rows, cols, ld, inner, stride, outer, stride_outer;
    int32_t elem_bytes, box_cols, box_rows, swizzle;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && inner == o.inner &&
               stride == o.stride && outer == o.outer && stride_outer == o.stride_outer &&
               elem_bytes == o.elem_bytes && box_cols == o.box_cols && box_rows == o.box_rows &&
               swizzle == o.swizzle;
    }
};
struct MapCacheEntry {
    MapKey key;
    bool used;
    CUtensorMap map;
};
constexpr int kMapCacheSlots = 1024;
std::atomic<uint64_t> g_map_cache_hits{0}, g_map_cache_misses{0};

int cached_map(CUtensorMap* map, const void* base, int elem_bytes, int64_t rows, int64_t cols, int64_t ld,
               const BatchLayout& bl, int box_cols, int box_rows, CUtensorMapSwizzle swizzle) {
    thread_local MapCacheEntry* table = nullptr;
    if (table == nullptr) table = new MapCacheEntry[kMapCacheSlots]();
    const MapKey key{base, rows, cols, ld, bl.inner, bl.inner > 1 ? bl.stride : 0, bl.outer,
                     bl.outer > 1 ? bl.stride_outer : 0, elem_bytes, box_cols, box_rows, static_cast<int32_t>(swizzle)};
    uint64_t h = 1469598103934665603ull;  // FNV-1a over the key's words, as llmt's AlgoKeyHash does
    const uint64_t words[10] = {reinterpret_cast<uintptr_t>(base), static_cast<uint64_t>(rows),
                                static_cast<uint64_t>(cols), static_cast<uint64_t>(ld),
                                static_cast<uint64_t>(key.inner), static_cast<uint64_t>(key.stride),
                                static_cast<uint64_t>(key.outer), static_cast<uint64_t>(key.stride_outer),
                                (static_cast<uint64_t>(elem_bytes) << 32) | static_cast<uint32_t>(box_cols),
                                (static_cast<uint64_t>(box_rows) << 32) | static_cast<uint32_t>(swizzle)};
    for (uint64_t w : words) { h ^= w; h *= 1099511628211ull; }
    MapCacheEntry& e = table[(h ^ (h >> 29)) % kMapCacheSlots];
    if (e.used && e.key == key) {
        *map = e.map;
        g_map_cache_hits.fetch_add(1, std::memory_order_relaxed);
        return LLMT_B200_OK;
    }
    const int st = encode_map(map, base, elem_bytes, rows, cols, ld, bl, box_cols, box_rows, swizzle);
    if (st != LLMT_B200_OK) return st;
    e.key = key; e.used = true; e.map = *map;
    g_map_cache_misses.fetch_add(1, std::memory_order_relaxed);
    return LLMT_B200_OK;
}

// bf16 operand map boxed for 128-byte-swizzled tiles (64 elements wide).
int encode_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld,
                       const BatchLayout& bl, int box_rows) {
    return cached_map(map, base, 2, rows, cols, ld, bl, 64, box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
}

// Tile-queue counters: zero between launches (the kernel re-arms its counter); launches
// take them round-robin so that kernels in flight at the same time do not share one.
constexpr int kSchedSlots = 64;
static __device__ int32_t g_sched_counters[kSchedSlots];
// Arrival counters of the two-phase dbias reduction, one pair per launch slot; the kernel
// re-arms them too.
static __device__ int32_t g_dbias_sync[kSchedSlots][2];
// Chunk counters of the exchanges that ride along, one per launch slot; re-armed by the kernel.
static __device__ int32_t g_ride_counters[kSchedSlots];

// Per-device host state.  Several devices per process are supported as long as each device's
// calls come from one host thread at a time (llmt's rule: one thread issues the launches,
// src/kernels/matmul.cpp:23-27).
struct DeviceGlobals {
    bool ready = false;
    int32_t* counters = nullptr;
    int32_t* dbias_sync = nullptr;
    int32_t* ride_counters = nullptr;
    unsigned next = 0;
};

DeviceGlobals* device_globals_slot() {
    static DeviceGlobals globals[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return &globals[dev];
}

// First use on a device: resolves and zeroes the tile-queue counters.  This is a synchronous
// memset, so the first GEMM on a device must not be issued inside a stream capture.
int device_globals(DeviceGlobals** out) {
    DeviceGlobals* g = device_globals_slot();
    if (g == nullptr) return fail(LLMT_B200_ERR_CUDA, "no current CUDA device");
    if (!g->ready) {
        void* ctr = nullptr;
        void* sync = nullptr;
        void* ride = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ctr, g_sched_counters);
        if (e == cudaSuccess) e = cudaMemset(ctr, 0, sizeof(int32_t) * kSchedSlots);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&sync, g_dbias_sync);
        if (e == cudaSuccess) e = cudaMemset(sync, 0, sizeof(int32_t) * kSchedSlots * 2);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&ride, g_ride_counters);
        if (e == cudaSuccess) e = cudaMemset(ride, 0, sizeof(int32_t) * kSchedSlots);
        if (e != cudaSuccess)
            return fail(LLMT_B200_ERR_CUDA, "device set-up failed: %s", cudaGetErrorString(e));
        g->counters = static_cast<int32_t*>(ctr);
        g->dbias_sync = static_cast<int32_t*>(sync);
        g->ride_counters = static_cast<int32_t*>(ride);
        g->ready = true;
    }
    *out = g;
    return LLMT_B200_OK;
}

// Bound of every wait inside the kernels (nanoseconds of %globaltimer).
uint64_t g_wait_limit_ns = 2000000000ull;
uint64_t g_comm_wait_limit_ns = 4000000000ull;

// TMA needs 16-byte aligned bases, pitches and batch strides.  An operand that breaks one of
// the rules - a contiguous [tokens, 50257] dLogits, a slice x[:, 1:] - is first copied into
// the workspace with an aligned base and its pitch rounded up ("repacked").
bool needs_repack(const void* base, int64_t ld, int64_t batch, int64_t stride, int64_t batch_inner = 0,
                  int64_t stride_outer = 0) {
    return (reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (ld % 8) != 0 || (batch > 1 && (stride % 8) != 0) ||
           (batch_inner > 0 && (stride_outer % 8) != 0);
}

struct Repack {
    bool a = false, b = false;
    int64_t lda = 0, ldb = 0, stride_a = 0, stride_b = 0;  // layout of the repacked copies
    size_t bytes_a = 0, bytes_b = 0;                       // 256-byte rounded
    size_t total() const { return bytes_a + bytes_b; }
};

// a, b: the operands' addresses, or null when only the size is wanted for operands that are
// known to be 16-byte aligned.
Repack repack_plan(const llmt_b200_gemm_desc* d, const Checked& ck, const void* a, const void* b) {
    Repack r;
    const int64_t nb = d->batch > 1 ? d->batch : 1;
    auto round8 = [](int64_t v) { return (v + 7) / 8 * 8; };
    if (d->k > 0 && needs_repack(a, d->lda, d->batch, d->stride_a, d->batch_inner, d->stride_a_outer)) {
        r.a = true;
        r.lda = round8(ck.a_cols);
        r.stride_a = ck.a_rows * r.lda;
        r.bytes_a = (static_cast<size_t>(nb) * r.stride_a * 2 + 255) / 256 * 256;
    }
    if (d->k > 0 && needs_repack(b, d->ldb, d->batch, d->stride_b, d->batch_inner, d->stride_b_outer)) {
        r.b = true;
        r.ldb = round8(ck.b_cols);
        r.stride_b = ck.b_rows * r.ldb;
        r.bytes_b = (static_cast<size_t>(nb) * r.stride_b * 2 + 255) / 256 * 256;
    }
    return r;
}

// Copies the operands that need it behind the split-K region of the workspace and rewrites
// the (local) descriptor and pointers to use the copies.
// Copies made for earlier problems of the same grouped launch: an operand that several problems
// share (dy is the A operand of a layer's dX and of its dW) is copied once.
struct RepackDone {
    const void* src;
    int64_t rows, cols, ld, nb, stride;
    const void* dst;
};
struct RepackCache {
    RepackDone done[2 * kMaxGroupProblems];
    int n = 0;
    const void* find(const void* src, int64_t rows, int64_t cols, int64_t ld, int64_t nb, int64_t stride) const {
        for (int i = 0; i < n; ++i) {
            const RepackDone& r = done[i];
            if (r.src == src && r.rows == rows && r.cols == cols && r.ld == ld && r.nb == nb && r.stride == stride) return r.dst;
        }
        return nullptr;
    }
    void add(const void* src, int64_t rows, int64_t cols, int64_t ld, int64_t nb, int64_t stride, const void* dst) {
        if (n < 2 * kMaxGroupProblems) done[n++] = RepackDone{src, rows, cols, ld, nb, stride, dst};
    }
};

int apply_repack(llmt_b200_gemm_desc* d, const Checked& ck, const Repack& rp, size_t ws_offset,
                 const void** a, const void** b, cudaStream_t stream, RepackCache* cache = nullptr) {
    char* base = static_cast<char*>(d->workspace) + ws_offset;
    const int64_t nb = d->batch > 1 ? d->batch : 1;
    auto one = [&](const void** src, int64_t rows, int64_t cols, int64_t ld, int64_t stride, int64_t new_ld,
                   int64_t new_stride, char* dst) -> int {
        const void* have = cache != nullptr ? cache->find(*src, rows, cols, ld, nb, stride) : nullptr;
        if (have == nullptr) {
            cudaError_t e = launch_repack_bf16(dst, *src, rows, cols, ld, new_ld, nb, stride, new_stride, stream);
            if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
            if (cache != nullptr) cache->add(*src, rows, cols, ld, nb, stride, dst);
            have = dst;
        }
        *src = have;
        return LLMT_B200_OK;
    };
    if (rp.a) {
        const int st = one(a, ck.a_rows, ck.a_cols, d->lda, d->batch > 1 ? d->stride_a : 0, rp.lda, rp.stride_a, base);
        if (st != LLMT_B200_OK) return st;
        d->lda = rp.lda;
        d->stride_a = rp.stride_a;
        base += rp.bytes_a;
    }
    if (rp.b) {
        const int st = one(b, ck.b_rows, ck.b_cols, d->ldb, d->batch > 1 ? d->stride_b : 0, rp.ldb, rp.stride_b, base);
        if (st != LLMT_B200_OK) return st;
        d->ldb = rp.ldb;
        d->stride_b = rp.stride_b;
    }
    return LLMT_B200_OK;
}

int check_workspace(const llmt_b200_gemm_desc* d, const TcPlan& pl, size_t repack_bytes = 0) {
    const size_t need = pl.workspace_bytes + repack_bytes;
    if (need == 0) return LLMT_B200_OK;
    if (d->workspace == nullptr || d->workspace_bytes < need)
        return fail(LLMT_B200_ERR_WORKSPACE,
                    "matmul: needs %llu workspace bytes (split-K partial sums %llu, repacked operands %llu), got %llu",
                    (unsigned long long)need, (unsigned long long)pl.workspace_bytes,
                    (unsigned long long)repack_bytes, (unsigned long long)d->workspace_bytes);
    if (reinterpret_cast<uintptr_t>(d->workspace) & 255u)
        return fail(LLMT_B200_ERR_INVALID, "matmul: workspace must be 256-byte aligned");
    return LLMT_B200_OK;
}

// Fills the kernel-side description of one problem (tensor maps included).
int fill_problem(GroupProblem* p, const llmt_b200_gemm_desc* d, const Checked& ck, const TcPlan& pl,
                 void* c, const void* a, const void* b) {
    memset(static_cast<void*>(p), 0, sizeof *p);
    p->m = d->m; p->n = d->n; p->k = d->k;
    p->batch = static_cast<int32_t>(d->batch);
    p->tiles_m = pl.tiles_m; p->tiles_n = pl.tiles_n; p->splits = pl.splits;
    p->inv_tiles_m = 1.0f / static_cast<float>(pl.tiles_m);
    p->inv_tiles_n = 1.0f / static_cast<float>(pl.tiles_n);
    p->inv_splits = 1.0f / static_cast<float>(pl.splits);
    p->kblocks_total = pl.kblocks_total;
    p->kblocks_per_split = pl.kblocks_per_split;
    p->bn = pl.bn;
    p->a_mn = d->trans_a ? 1 : 0;  // A stored [k, m]: m contiguous
    p->b_mn = d->trans_b ? 0 : 1;  // B stored [k, n]: n contiguous
    p->num_tiles = static_cast<int32_t>(pl.num_tiles);
    p->batch_inner = static_cast<int32_t>(d->batch_inner);
    p->inv_batch_inner = d->batch_inner > 0 ? 1.0f / static_cast<float>(d->batch_inner) : 0.0f;
    p->c = c; p->ldc = d->ldc; p->stride_c = d->batch > 1 ? d->stride_c : 0;
    p->stride_c_outer = d->batch_inner > 0 ? d->stride_c_outer : 0;
    p->c_is_bf16 = d->dtype_c == LLMT_B200_BF16;
    p->alpha = d->alpha; p->beta = d->beta;
    p->bias = d->bias; p->bias_is_bf16 = d->bias_dtype == LLMT_B200_BF16;
    p->epi_flags = d->epilogue & (LLMT_B200_EPI_BIAS | LLMT_B200_EPI_GELU);
    if (d->epilogue & LLMT_B200_EPI_GELU_BWD) {
        p->epi_flags |= kEpiGeluBwd;
        p->ext_ptr = d->aux;
    }
    if (d->epilogue & LLMT_B200_EPI_SAVE_PRE) {
        p->epi_flags |= kEpiSavePre;
        p->ext_ptr = d->aux;
    }
    p->dbias = d->dbias; p->dbias_beta = d->dbias_beta;
    p->a_raw = a; p->lda = d->lda;
    p->dbias_mode = pl.dbias_mode;
    p->colsum_tiles = pl.colsum_tiles;
    p->dbias_rows = pl.dbias_rows;
    p->fin_tiles = pl.fin_tiles;
    if (pl.splits > 1) p->ws = static_cast<float*>(d->workspace);
    if (pl.dbias_mode == 1 || (pl.dbias_mode == 3 && pl.splits > 1))
        p->ws_dbias = reinterpret_cast<float*>(static_cast<char*>(d->workspace) + pl.ws_dbias_off);
    if (d->k == 0) return LLMT_B200_OK;  // no operand is read
    int st = encode_operand_map(&p->map_a, a, ck.a_rows, ck.a_cols, d->lda,
                                batch_layout(d->batch, d->batch_inner, d->stride_a, d->stride_a_outer), p->a_mn ? 64 : 128);
    if (st != LLMT_B200_OK) return st;
    st = encode_operand_map(&p->map_b, b, ck.b_rows, ck.b_cols, d->ldb,
                            batch_layout(d->batch, d->batch_inner, d->stride_b, d->stride_b_outer),
                            p->b_mn ? 64 : (pl.pairs ? pl.bn / 2 : pl.bn));
    if (st != LLMT_B200_OK) return st;
    // Results leave through shared memory and TMA stores (boxes of 32 rows x 128 bytes) when
    // their layout allows a tensor map (16-byte aligned base, pitch and batch stride);
    // otherwise straight from registers.
    if (pl.splits > 1) {
        if (d->n % 4 == 0) {
            st = cached_map(&p->map_ws, d->workspace, 4, d->m, d->n, d->n,
                            batch_layout(d->batch * pl.splits, 0, d->m * d->n, 0), 32, 32, CU_TENSOR_MAP_SWIZZLE_128B);
            if (st != LLMT_B200_OK) return st;
            p->ws_tma = 1;
        }
        return LLMT_B200_OK;
    }
    const int ces = p->c_is_bf16 ? 2 : 4;
    if (c != nullptr && (reinterpret_cast<uintptr_t>(c) & 15u) == 0 && (d->ldc * ces) % 16 == 0 &&
        (d->batch <= 1 || (d->stride_c * ces) % 16 == 0) &&
        (d->batch_inner <= 0 || (d->stride_c_outer * ces) % 16 == 0)) {
        st = cached_map(&p->map_c, c, ces, d->m, d->n, d->ldc,
                        batch_layout(d->batch, d->batch_inner, d->stride_c, d->stride_c_outer), p->c_is_bf16 ? 64 : 32, 32,
                        CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != LLMT_B200_OK) return st;
        p->c_tma = 1;
    }
    return LLMT_B200_OK;
}

// Launches the tensor-core kernel over `count` filled problems (longest tiles first),
// then the fixed-order reduction of every problem that was split.
int launch_group(GroupProblem* probs, int count, bool pairs, cudaStream_t stream, const RideExchange* ride = nullptr,
                 bool lse = false) {
    DeviceGlobals* g = nullptr;
    int st = device_globals(&g);
    if (st != LLMT_B200_OK) return st;
    thread_local GroupParams gp;
    // A problem with a row-wise epilogue takes the whole launch to the kernels that carry those.
    for (int i = 0; i < count; ++i)
        if (probs[i].epi_flags & (kEpiLse | kEpiCausal | kEpiExpSub | kEpiMulAux | kEpiCeGrad | kEpiGeluBwd | kEpiSavePre)) lse = true;
    // Longest reductions first: with a dynamic queue this is longest-processing-time-first.
    int order[kMaxGroupProblems];
    for (int i = 0; i < count; ++i) order[i] = i;
    for (int i = 1; i < count; ++i)
        for (int j = i; j > 0 && probs[order[j]].kblocks_per_split > probs[order[j - 1]].kblocks_per_split; --j) {
            const int t = order[j]; order[j] = order[j - 1]; order[j - 1] = t;
        }
    // Ticket layout: the dbias reductions of all problems first (they keep only the epilogue
    // warps busy, so the CTAs that draw them go straight on to an MMA tile), then the MMA tiles,
    // then the tickets that finish the two-phase dbias reductions.
    int64_t colsum_total = 0, fin_total = 0;
    int n = 0;
    for (int i = 0; i < count; ++i) {
        GroupProblem& p = probs[order[i]];
        if (p.k == 0 || p.num_tiles == 0) continue;
        p.colsum_begin = static_cast<int32_t>(colsum_total);
        colsum_total += p.colsum_tiles;
        p.fin_begin = static_cast<int32_t>(fin_total);
        fin_total += p.fin_tiles;
        gp.prob[n++] = p;
    }
    if (ride != nullptr && n == 0)
        return fail(LLMT_B200_ERR_INVALID, "gemm_grouped_exchange: the launch has no tile to ride along with");
    int64_t total = colsum_total;
    for (int i = 0; i < n; ++i) {
        if (total + gp.prob[i].num_tiles + fin_total > 0x7fffff00)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: too many tiles in one launch");
        gp.prob[i].tile_begin = static_cast<int32_t>(total);
        total += gp.prob[i].num_tiles;
    }
    if (n > 0) {
        const unsigned slot = g->next++ % kSchedSlots;
        gp.num_problems = n;
        gp.colsum_total = static_cast<int32_t>(colsum_total);
        gp.fin_begin = static_cast<int32_t>(total);
        total += fin_total;
        // An exchange that rides along is the side warps' work: its chunks are not tickets.
        if (ride != nullptr) gp.ride = *ride;
        else gp.ride.tiles = 0;
        gp.ride_counter = g->ride_counters + slot;
        gp.total_tiles = static_cast<int32_t>(total);
        gp.sched_counter = g->counters + slot;
        gp.dbias_sync = g->dbias_sync + 2 * slot;
        gp.static_schedule = static_schedule_forced() ? 1 : 0;
        gp.wait_limit_ns = g_wait_limit_ns;
        gp.status = device_status_ptr();
        if (gp.status == nullptr) return fail(LLMT_B200_ERR_CUDA, "cannot resolve the device status word");
        const int units = pairs ? pair_units() : sm_count();
        // (with an exchange riding along every unit is launched: its side warps share the chunks)
        const int grid = static_cast<int>(total < units && ride == nullptr ? total : units) * (pairs ? 2 : 1);
        cudaError_t e = launch_tc_grouped(gp, grid, pairs, stream, lse);
        if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    }
    for (int i = 0; i < count; ++i) {
        GroupProblem p = probs[i];
        if (p.k == 0) p.splits = 0;  // empty reduction: C = epilogue(beta * C)
        if (p.splits == 1) continue;
        cudaError_t e = launch_splitk_reduce(p, stream);
        if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    }
    return LLMT_B200_OK;
}

int run_bf16(const llmt_b200_gemm_desc* d, const Checked& ck, void* c, const void* a, const void* b,
             cudaStream_t stream) {
    const TcPlan pl = plan_single(d);
    const Repack rp = repack_plan(d, ck, a, b);
    if (rp.total() > 0 && d->batch_inner > 0)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: operands of a two-level batch layout must start on 16-byte "
                    "boundaries with pitches and strides that are multiples of 8 elements");
    int st = check_workspace(d, pl, rp.total());
    if (st != LLMT_B200_OK) return st;
    llmt_b200_gemm_desc local = *d;
    if (rp.total() > 0) {
        st = apply_repack(&local, ck, rp, pl.workspace_bytes, &a, &b, stream);
        if (st != LLMT_B200_OK) return st;
    }
    GroupProblem p;
    st = fill_problem(&p, &local, ck, pl, c, a, b);
    if (st != LLMT_B200_OK) return st;
    return launch_group(&p, 1, pl.pairs != 0, stream);
}

// Group plans: every problem is planned knowing the total work of the launch.
bool plan_group(const llmt_b200_gemm_desc* descs, int count, TcPlan* plans) {
    bool pairs = true;  // a launch is either all pairs or all single CTAs
    for (int i = 0; i < count; ++i) pairs = pairs && pair_eligible(&descs[i]);
    const int sms = pairs ? pair_units() : sm_count();
    int64_t work = 0;
    for (int i = 0; i < count; ++i) {
        const llmt_b200_gemm_desc& d = descs[i];
        work += static_cast<int64_t>(ceil_div(d.m, pairs ? 256 : 128)) * ceil_div(d.n, 256) *
                (d.batch > 0 ? d.batch : 1) * ceil_div(d.k, 64);
    }
    for (int i = 0; i < count; ++i) {
        const llmt_b200_gemm_desc& d = descs[i];
        plans[i] = count == 1 ? plan_single(&d)
                              : make_group_plan(d.m, d.n, d.k, d.batch, dbias_mode_of(&d), sms, work,
                                                d.plan_tile_n, splits_wanted(&d), pairs, d.trans_b == 0);
    }
    return count == 1 ? plans[0].pairs != 0 : pairs;
}

int run_fp32(const llmt_b200_gemm_desc* d, void* c, const void* a, const void* b, cudaStream_t stream) {
    Fp32GemmParams p{};
    p.m = d->m; p.n = d->n; p.k = d->k; p.batch = d->batch;
    p.a = static_cast<const float*>(a);
    p.b = static_cast<const float*>(b);
    p.c = static_cast<float*>(c);
    p.lda = d->lda; p.ldb = d->ldb; p.ldc = d->ldc;
    p.stride_a = d->batch > 1 ? d->stride_a : 0;
    p.stride_b = d->batch > 1 ? d->stride_b : 0;
    p.stride_c = d->batch > 1 ? d->stride_c : 0;
    p.batch_inner = d->batch_inner > 0 ? d->batch_inner : 0;
    p.stride_a_outer = d->stride_a_outer; p.stride_b_outer = d->stride_b_outer; p.stride_c_outer = d->stride_c_outer;
    p.trans_a = d->trans_a; p.trans_b = d->trans_b;
    p.alpha = d->alpha; p.beta = d->beta;
    p.bias = d->bias; p.bias_is_bf16 = d->bias_dtype == LLMT_B200_BF16;
    p.epi_flags = d->epilogue;
    if (d->batch > 65535) return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: fp32 path supports batch <= 65535");
    cudaError_t e = launch_fp32_gemm(p, stream);
    // The strict-fp32 path has nothing to fuse the bias gradient into: a second small kernel.
    if (e == cudaSuccess && d->dbias != nullptr) e = launch_fp32_rowsum(p, d->dbias, d->dbias_beta, stream);
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

}  // namespace

void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

DeviceStatus* device_status_ptr() {
    // One address per device; resolved with that device current.
    static DeviceStatus* ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<DeviceStatus*>(p);
    }
    return ptrs[dev];
}

}  // namespace llmt_b200

using namespace llmt_b200;

extern "C" {

int llmt_b200_gemm(const llmt_b200_gemm_desc* d, void* c, const void* a, const void* b, void* stream) {
    Checked ck{};
    const int st = validate(d, c, a, b, &ck);
    if (st != LLMT_B200_OK) return st;
    if (d->m == 0 || d->n == 0 || d->batch == 0) return LLMT_B200_OK;  // nothing to write
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return ck.bf16 ? run_bf16(d, ck, c, a, b, s) : run_fp32(d, c, a, b, s);
}

int llmt_b200_gemm_static_scratch(const llmt_b200_gemm_desc* d, void* c, const void* a, const void* b,
                                  void* stream) {
    Checked ck{};
    const int st = validate(d, c, a, b, &ck);
    if (st != LLMT_B200_OK) return st;
    if (d->m == 0 || d->n == 0 || d->batch == 0) return LLMT_B200_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!ck.bf16) return run_fp32(d, c, a, b, s);  // the fp32 path uses no scratch at all
    // Size check first: a problem that does not fit is turned away before the scratch is
    // resolved and before anything is enqueued.
    const size_t need = plan_single(d).workspace_bytes + repack_plan(d, ck, a, b).total();
    if (need > kStaticScratchBytes)
        return fail(LLMT_B200_ERR_WORKSPACE,
                    "gemm_static_scratch: this problem's split-K plan needs %llu scratch bytes but the "
                    "built-in scratch holds %llu; use llmt_b200_gemm with a caller workspace, or force "
                    "fewer splits with plan_splits",
                    (unsigned long long)need, (unsigned long long)kStaticScratchBytes);
    llmt_b200_gemm_desc local = *d;  // the caller's workspace fields are ignored
    local.workspace = nullptr;
    local.workspace_bytes = 0;
    if (need > 0) {
        cudaError_t e = cudaSuccess;
        void* scratch = static_scratch_ptr(&e);
        if (scratch == nullptr)
            return fail(LLMT_B200_ERR_CUDA, "gemm_static_scratch: cannot resolve the built-in scratch: %s",
                        cudaGetErrorString(e));
        local.workspace = scratch;
        local.workspace_bytes = kStaticScratchBytes;
    }
    return run_bf16(&local, ck, c, a, b, s);
}

namespace {
int gemm_grouped_impl(const llmt_b200_gemm_desc* descs, void* const* c, const void* const* a,
                      const void* const* b, int32_t count, void* stream, const llmt_b200_comm_desc* comm,
                      int64_t xoffset, int64_t xcount, int32_t xindex) {
    if (descs == nullptr || c == nullptr || a == nullptr || b == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "gemm_grouped: null argument");
    if (count < 1 || count > kMaxGroupProblems)
        return fail(LLMT_B200_ERR_INVALID, "gemm_grouped: count must be 1..%d", kMaxGroupProblems);
    Checked ck[kMaxGroupProblems] = {};
    for (int i = 0; i < count; ++i) {
        const int st = validate(&descs[i], c[i], a[i], b[i], &ck[i]);
        if (st != LLMT_B200_OK) return st;
        if (!ck[i].bf16)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "gemm_grouped: problem %d is not a bf16 problem", i);
        // A problem must not write (C, dbias, workspace) what another problem of the same launch
        // reads or writes: the tiles of all problems run concurrently.
        for (int j = 0; j < i; ++j) {
            struct Range { const void* p; size_t n; };
            auto writes_of = [&](int q, Range* out) {
                out[0] = {c[q], ck[q].c_bytes};
                out[1] = {descs[q].dbias, descs[q].dbias != nullptr ? static_cast<size_t>(descs[q].m) * 4 : 0};
                out[2] = {descs[q].workspace, descs[q].workspace != nullptr ? static_cast<size_t>(descs[q].workspace_bytes) : 0};
            };
            auto touches_of = [&](int q, Range* out) {
                writes_of(q, out);
                out[3] = {a[q], ck[q].a_bytes};
                out[4] = {b[q], ck[q].b_bytes};
                out[5] = {descs[q].bias, (descs[q].epilogue & LLMT_B200_EPI_BIAS)
                                             ? static_cast<size_t>(descs[q].n) * (descs[q].bias_dtype == LLMT_B200_BF16 ? 2 : 4) : 0};
            };
            Range wi[3], wj[3], ti[6], tj[6];
            writes_of(i, wi); writes_of(j, wj); touches_of(i, ti); touches_of(j, tj);
            bool clash = false;
            for (const Range& w : wi)
                for (const Range& t : tj) clash = clash || (w.n != 0 && t.n != 0 && overlaps(w.p, w.n, t.p, t.n));
            for (const Range& w : wj)
                for (const Range& t : ti) clash = clash || (w.n != 0 && t.n != 0 && overlaps(w.p, w.n, t.p, t.n));
            if (clash)
                return fail(LLMT_B200_ERR_INVALID, "gemm_grouped: problems %d and %d are not independent", j, i);
        }
    }
    if (comm != nullptr) {
        // The exchange that rides along: its arguments are checked before anything is planned.
        if (comm->world < 2 || comm->world > kMaxCommRanks || comm->rank < 0 || comm->rank >= comm->world)
            return fail(LLMT_B200_ERR_INVALID, "gemm_grouped_exchange: bad rank/world");
        if (comm->grad_mc == nullptr)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "gemm_grouped_exchange: needs the span's NVSwitch multicast mapping "
                        "(comm.grad_mc); use llmt_b200_grad_allreduce after the launch instead");
        if (xoffset < 0 || xcount <= 0 || xoffset % 4 != 0 || xcount % 4 != 0)
            return fail(LLMT_B200_ERR_INVALID, "gemm_grouped_exchange: offset and count must be positive multiples of 4 floats");
        if (xindex < 0 || xindex >= kMaxRidesPerStep)
            return fail(LLMT_B200_ERR_INVALID, "gemm_grouped_exchange: index must be 0..%d", kMaxRidesPerStep - 1);
        for (int r = 0; r < comm->world; ++r)
            if (comm->grad[r] == nullptr || comm->flags[r] == nullptr)
                return fail(LLMT_B200_ERR_INVALID, "gemm_grouped_exchange: null buffer for rank %d", r);
        // The range must be complete before this launch starts: nothing in the launch may write it.
        const char* x_lo = static_cast<const char*>(comm->grad[comm->rank]) + xoffset * 4;
        for (int i = 0; i < count; ++i) {
            const bool hits = overlaps(x_lo, static_cast<size_t>(xcount) * 4, c[i], ck[i].c_bytes) ||
                              (descs[i].dbias != nullptr &&
                               overlaps(x_lo, static_cast<size_t>(xcount) * 4, descs[i].dbias, static_cast<size_t>(descs[i].m) * 4));
            if (hits)
                return fail(LLMT_B200_ERR_INVALID, "gemm_grouped_exchange: problem %d writes into the exchanged range; "
                            "only ranges that earlier launches completed may ride along", i);
        }
    }
    TcPlan plans[kMaxGroupProblems];
    const bool pairs = plan_group(descs, count, plans);
    for (int i = 0; i < count; ++i)
        if (descs[i].plan_cta_pairs == 2 && !pairs)
            return fail(LLMT_B200_ERR_INVALID,
                        "gemm_grouped: problem %d asks for CTA pairs, but another problem of the launch cannot run "
                        "on pairs (a launch is all pairs or all single CTAs)", i);
    GroupProblem probs[kMaxGroupProblems];
    RepackCache repacked;
    int n = 0;
    for (int i = 0; i < count; ++i) {
        if (descs[i].m == 0 || descs[i].n == 0 || descs[i].batch == 0) continue;
        const Repack rp = repack_plan(&descs[i], ck[i], a[i], b[i]);
        if (rp.total() > 0 && descs[i].batch_inner > 0)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "gemm_grouped: operands of a two-level batch layout must be "
                        "addressable by TMA as they are");
        int st = check_workspace(&descs[i], plans[i], rp.total());
        if (st != LLMT_B200_OK) return st;
        llmt_b200_gemm_desc local = descs[i];
        const void* ai = a[i];
        const void* bi = b[i];
        if (rp.total() > 0) {
            st = apply_repack(&local, ck[i], rp, plans[i].workspace_bytes, &ai, &bi,
                              static_cast<cudaStream_t>(stream), &repacked);
            if (st != LLMT_B200_OK) return st;
        }
        st = fill_problem(&probs[n], &local, ck[i], plans[i], c[i], ai, bi);
        if (st != LLMT_B200_OK) return st;
        ++n;
    }
    if (comm == nullptr) {
        if (n == 0) return LLMT_B200_OK;
        return launch_group(probs, n, pairs, static_cast<cudaStream_t>(stream));
    }
    RideExchange ride{};
    ride.mc = static_cast<float*>(comm->grad_mc) + xoffset;
    ride.n4 = xcount / 4;
    ride.local = static_cast<uint32_t*>(comm->flags[comm->rank]);
    for (int r = 0; r < comm->world; ++r)
        ride.peer_ready[r] = static_cast<uint32_t*>(comm->flags[r]) + kRideReady + comm->rank;
    ride.world = comm->world;
    ride.rank = comm->rank;
    ride.index = xindex;
    // About 32 KB of this rank's share per chunk: four passes of a side warp with 8 KB in flight.
    const int64_t share_bytes = (ride.n4 + comm->world - 1) / comm->world * 16;
    int64_t tiles = (share_bytes + 32767) / 32768;
    if (tiles < 1) tiles = 1;
    if (tiles > 0x3fffffff) tiles = 0x3fffffff;
    ride.tiles = static_cast<int32_t>(tiles);
    return launch_group(probs, n, pairs, static_cast<cudaStream_t>(stream), &ride);
}
}  // namespace

int llmt_b200_gemm_grouped(const llmt_b200_gemm_desc* descs, void* const* c, const void* const* a,
                           const void* const* b, int32_t count, void* stream) {
    return gemm_grouped_impl(descs, c, a, b, count, stream, nullptr, 0, 0, 0);
}

int llmt_b200_gemm_grouped_exchange(const llmt_b200_gemm_desc* descs, void* const* c, const void* const* a,
                                    const void* const* b, int32_t count, const llmt_b200_comm_desc* comm,
                                    int64_t offset, int64_t count_floats, int32_t index, void* stream) {
    if (comm == nullptr) return fail(LLMT_B200_ERR_INVALID, "gemm_grouped_exchange: null exchange descriptor");
    return gemm_grouped_impl(descs, c, a, b, count, stream, comm, offset, count_floats, index);
}

namespace {
void shape_only(const llmt_b200_gemm_desc& d, Checked* ck) {
    ck->a_rows = d.trans_a ? d.k : d.m; ck->a_cols = d.trans_a ? d.m : d.k;
    ck->b_rows = d.trans_b ? d.n : d.k; ck->b_cols = d.trans_b ? d.k : d.n;
}
bool is_tc_problem(const llmt_b200_gemm_desc& d) {
    return d.dtype_ab == LLMT_B200_BF16 && d.m > 0 && d.n > 0 && d.k > 0 && d.batch > 0;
}
}  // namespace

namespace {
// Layout of the workspace of llmt_b200_lm_head_ce_fwd: the GEMM's own scratch (repacked operands),
// then the per-part (maximum, sum of exponentials) pairs, then the target logits.
struct LmHeadCePlan {
    TcPlan pl;
    size_t gemm_bytes, stats_off, tgt_off, grad_off, sum_off, total;
    int parts;
};
// One plan for the forward and the backward call on the same product, whatever type each of them
// stores: the backward pass may reuse the statistics the forward pass left in the workspace.
LmHeadCePlan lm_head_ce_plan(const llmt_b200_gemm_desc* d, const Checked& ck, const void* a, const void* b) {
    LmHeadCePlan r;
    llmt_b200_gemm_desc local = *d;
    local.plan_splits = 1;  // the epilogue sees whole reductions
    local.dtype_c = LLMT_B200_FP32;
    r.pl = plan_single(&local);
    r.gemm_bytes = r.pl.workspace_bytes + repack_plan(&local, ck, a, b).total();
    r.parts = 2 * r.pl.tiles_n;
    r.stats_off = (r.gemm_bytes + 255) / 256 * 256;
    r.tgt_off = r.stats_off + (static_cast<size_t>(r.parts) * d->m * 8 + 255) / 256 * 256;
    r.grad_off = r.tgt_off + (static_cast<size_t>(d->m) * 4 + 255) / 256 * 256;    // (lse, weight) per row
    r.sum_off = r.grad_off + (static_cast<size_t>(d->m) * 8 + 255) / 256 * 256;    // the mask's sum
    r.total = r.sum_off + 256;
    return r;
}
int lm_head_ce_check(const llmt_b200_gemm_desc* d) {
    if (d->dtype_ab != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "lm_head_ce_fwd: bf16 operands only");
    if (d->batch > 1) return fail(LLMT_B200_ERR_UNSUPPORTED, "lm_head_ce_fwd: one product, no batch");
    if (d->dbias != nullptr || (d->epilogue & LLMT_B200_EPI_GELU))
        return fail(LLMT_B200_ERR_UNSUPPORTED, "lm_head_ce_fwd: no dbias, no GELU");
    if (d->m < 1 || d->n < 1 || d->k < 1 || d->batch < 1) return fail(LLMT_B200_ERR_INVALID, "lm_head_ce_fwd: empty problem");
    return LLMT_B200_OK;
}
}  // namespace

uint64_t llmt_b200_lm_head_ce_workspace_bytes(const llmt_b200_gemm_desc* d, const void* a, const void* b) {
    if (d == nullptr || !is_tc_problem(*d) || d->batch > 1) return 0;
    Checked ck{};
    shape_only(*d, &ck);
    return lm_head_ce_plan(d, ck, a, b).total;
}

int llmt_b200_lm_head_ce_fwd(const llmt_b200_gemm_desc* d, void* logits, const void* a, const void* b,
                             const int32_t* targets, const float* mask, float* row_nll, float* loss,
                             void* stream) {
    Checked ck{};
    int st = validate(d, logits, a, b, &ck, /*c_optional=*/true);
    if (st != LLMT_B200_OK) return st;
    st = lm_head_ce_check(d);
    if (st != LLMT_B200_OK) return st;
    if (targets == nullptr || mask == nullptr || row_nll == nullptr || loss == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "lm_head_ce_fwd: null targets, mask, row_nll or loss");
    if (logits == nullptr && d->beta != 0.0f)
        return fail(LLMT_B200_ERR_INVALID, "lm_head_ce_fwd: beta needs the logits tensor");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    llmt_b200_gemm_desc local = *d;
    local.plan_splits = 1;
    const LmHeadCePlan lp = lm_head_ce_plan(d, ck, a, b);
    if (d->workspace == nullptr || d->workspace_bytes < lp.total)
        return fail(LLMT_B200_ERR_WORKSPACE, "lm_head_ce_fwd: needs %llu workspace bytes (llmt_b200_lm_head_ce_workspace_bytes), got %llu",
                    (unsigned long long)lp.total, (unsigned long long)d->workspace_bytes);
    if (reinterpret_cast<uintptr_t>(d->workspace) & 255u)
        return fail(LLMT_B200_ERR_INVALID, "matmul: workspace must be 256-byte aligned");
    const Repack rp = repack_plan(&local, ck, a, b);
    if (rp.total() > 0) {
        st = apply_repack(&local, ck, rp, lp.pl.workspace_bytes, &a, &b, s);
        if (st != LLMT_B200_OK) return st;
    }
    GroupProblem p;
    st = fill_problem(&p, &local, ck, lp.pl, logits, a, b);
    if (st != LLMT_B200_OK) return st;
    char* ws = static_cast<char*>(d->workspace);
    p.ext_stats = reinterpret_cast<float2*>(ws + lp.stats_off);
    p.ext_rowvec = reinterpret_cast<float*>(ws + lp.tgt_off);
    p.ext_ptr = targets;
    p.epi_flags |= kEpiLse;
    st = launch_group(&p, 1, lp.pl.pairs != 0, s, nullptr, /*lse=*/true);
    if (st != LLMT_B200_OK) return st;
    cudaError_t e = launch_cross_entropy_from_stats(loss, row_nll, p.ext_stats, p.ext_rowvec, mask, d->m, lp.parts, s);
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_lm_head_ce_bwd(const llmt_b200_gemm_desc* d, void* dlogits, const void* a, const void* b,
                             const int32_t* targets, const float* mask, float dloss, int32_t stats_valid,
                             void* stream) {
    Checked ck{};
    int st = validate(d, dlogits, a, b, &ck);
    if (st != LLMT_B200_OK) return st;
    st = lm_head_ce_check(d);
    if (st != LLMT_B200_OK) return st;
    if (targets == nullptr || mask == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "lm_head_ce_bwd: null targets or mask");
    if (d->beta != 0.0f) return fail(LLMT_B200_ERR_UNSUPPORTED, "lm_head_ce_bwd: beta must be 0");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    llmt_b200_gemm_desc local = *d;
    local.plan_splits = 1;
    const LmHeadCePlan lp = lm_head_ce_plan(d, ck, a, b);
    if (d->workspace == nullptr || d->workspace_bytes < lp.total)
        return fail(LLMT_B200_ERR_WORKSPACE, "lm_head_ce_bwd: needs %llu workspace bytes (llmt_b200_lm_head_ce_workspace_bytes), got %llu",
                    (unsigned long long)lp.total, (unsigned long long)d->workspace_bytes);
    if (reinterpret_cast<uintptr_t>(d->workspace) & 255u)
        return fail(LLMT_B200_ERR_INVALID, "matmul: workspace must be 256-byte aligned");
    const Repack rp = repack_plan(&local, ck, a, b);
    if (rp.total() > 0) {
        st = apply_repack(&local, ck, rp, lp.pl.workspace_bytes, &a, &b, s);
        if (st != LLMT_B200_OK) return st;
    }
    char* ws = static_cast<char*>(d->workspace);
    float2* stats = reinterpret_cast<float2*>(ws + lp.stats_off);
    GroupProblem p;
    if (!stats_valid) {
        // the statistics pass of the forward call, storing nothing
        st = fill_problem(&p, &local, ck, lp.pl, nullptr, a, b);
        if (st != LLMT_B200_OK) return st;
        p.ext_stats = stats;
        p.ext_rowvec = nullptr;
        p.ext_ptr = nullptr;
        p.epi_flags |= kEpiLse;
        st = launch_group(&p, 1, lp.pl.pairs != 0, s, nullptr, /*lse=*/true);
        if (st != LLMT_B200_OK) return st;
    }
    float2* rows = reinterpret_cast<float2*>(ws + lp.grad_off);
    cudaError_t e = launch_ce_grad_rows(rows, stats, nullptr, mask, reinterpret_cast<float*>(ws + lp.sum_off), dloss,
                                        d->m, lp.parts, s);
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    st = fill_problem(&p, &local, ck, lp.pl, dlogits, a, b);
    if (st != LLMT_B200_OK) return st;
    p.ext_stats = rows;
    p.ext_rowvec = nullptr;
    p.ext_ptr = targets;
    p.epi_flags |= kEpiCeGrad;
    return launch_group(&p, 1, lp.pl.pairs != 0, s, nullptr, /*lse=*/true);
}

int llmt_b200_cross_entropy_bwd(float* dlogits, const float* logits, const int32_t* targets, const float* mask,
                                float dloss, int64_t rows, int64_t vocab, int64_t ld_in, int64_t ld_out, void* stream) {
    if (dlogits == nullptr || logits == nullptr || targets == nullptr || mask == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "cross_entropy_bwd: invalid tensor (null data)");
    if (rows < 1 || vocab < 1 || ld_in < vocab || ld_out < vocab)
        return fail(LLMT_B200_ERR_INVALID, "cross_entropy_bwd: bad shape (rows %lld, vocab %lld, pitches %lld %lld)",
                    (long long)rows, (long long)vocab, (long long)ld_in, (long long)ld_out);
    if (dlogits != logits && overlaps(dlogits, static_cast<size_t>(rows) * ld_out * 4, logits, static_cast<size_t>(rows) * ld_in * 4))
        return fail(LLMT_B200_ERR_INVALID, "cross_entropy_bwd: dlogits must be the logits tensor itself or not overlap it");
    if (dlogits == logits && ld_in != ld_out)
        return fail(LLMT_B200_ERR_INVALID, "cross_entropy_bwd: in place needs one pitch");
    cudaError_t e = launch_cross_entropy_bwd(dlogits, logits, targets, mask, dloss, rows, vocab, ld_in, ld_out,
                                             static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

namespace {
// Workspace of the softmax fused around a GEMM: the GEMM's own scratch (repacked operands), the
// per-part (maximum, sum of exponentials) pairs of every row, the rows' log-sum-exp.
struct GemmSoftmaxPlan {
    TcPlan pl;
    size_t gemm_bytes, stats_off, lse_off, total;
    int parts;
    int64_t rows;  // batch * m
};
GemmSoftmaxPlan gemm_softmax_plan(const llmt_b200_gemm_desc* d, const Checked& ck, const void* a, const void* b) {
    GemmSoftmaxPlan r;
    llmt_b200_gemm_desc local = *d;
    local.plan_splits = 1;  // the epilogue sees whole reductions
    r.pl = plan_single(&local);
    r.gemm_bytes = r.pl.workspace_bytes + repack_plan(&local, ck, a, b).total();
    r.parts = 2 * r.pl.tiles_n;
    r.rows = d->m * (d->batch > 1 ? d->batch : 1);
    r.stats_off = (r.gemm_bytes + 255) / 256 * 256;
    r.lse_off = r.stats_off + (static_cast<size_t>(r.parts) * r.rows * 8 + 255) / 256 * 256;
    r.total = r.lse_off + (static_cast<size_t>(r.rows) * 4 + 255) / 256 * 256;
    return r;
}
int gemm_softmax_check(const llmt_b200_gemm_desc* d, int32_t causal, const char* who) {
    if (d->dtype_ab != LLMT_B200_BF16) return fail(LLMT_B200_ERR_UNSUPPORTED, "%s: bf16 operands only", who);
    if (d->dbias != nullptr || d->epilogue != 0)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "%s: no bias, no GELU, no dbias", who);
    if (d->beta != 0.0f) return fail(LLMT_B200_ERR_UNSUPPORTED, "%s: beta must be 0", who);
    if (d->m < 1 || d->n < 1 || d->k < 1 || d->batch < 1) return fail(LLMT_B200_ERR_INVALID, "%s: empty problem", who);
    if (causal && d->m != d->n)
        return fail(LLMT_B200_ERR_INVALID, "%s: causal mask requires square scores (Tq=%lld Tk=%lld)", who,
                    (long long)d->m, (long long)d->n);
    return LLMT_B200_OK;
}
}  // namespace

uint64_t llmt_b200_gemm_softmax_workspace_bytes(const llmt_b200_gemm_desc* d, const void* a, const void* b) {
    if (d == nullptr || !is_tc_problem(*d)) return 0;
    Checked ck{};
    shape_only(*d, &ck);
    return gemm_softmax_plan(d, ck, a, b).total;
}

int llmt_b200_gemm_softmax_fwd(const llmt_b200_gemm_desc* d, void* probs, const void* a, const void* b,
                               int32_t causal, float* lse, void* stream) {
    Checked ck{};
    int st = validate(d, probs, a, b, &ck);
    if (st != LLMT_B200_OK) return st;
    st = gemm_softmax_check(d, causal, "gemm_softmax_fwd");
    if (st != LLMT_B200_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    llmt_b200_gemm_desc local = *d;
    local.plan_splits = 1;
    const GemmSoftmaxPlan sp = gemm_softmax_plan(d, ck, a, b);
    if (d->workspace == nullptr || d->workspace_bytes < sp.total)
        return fail(LLMT_B200_ERR_WORKSPACE, "gemm_softmax_fwd: needs %llu workspace bytes (llmt_b200_gemm_softmax_workspace_bytes), got %llu",
                    (unsigned long long)sp.total, (unsigned long long)d->workspace_bytes);
    if (reinterpret_cast<uintptr_t>(d->workspace) & 255u)
        return fail(LLMT_B200_ERR_INVALID, "matmul: workspace must be 256-byte aligned");
    const Repack rp = repack_plan(&local, ck, a, b);
    if (rp.total() > 0) {
        st = apply_repack(&local, ck, rp, sp.pl.workspace_bytes, &a, &b, s);
        if (st != LLMT_B200_OK) return st;
    }
    char* ws = static_cast<char*>(d->workspace);
    float* row_lse = lse != nullptr ? lse : reinterpret_cast<float*>(ws + sp.lse_off);
    const int mask_flag = causal ? kEpiCausal : 0;
    // Pass 1: the product's tiles are made and looked at, not stored.
    GroupProblem p;
    st = fill_problem(&p, &local, ck, sp.pl, nullptr, a, b);
    if (st != LLMT_B200_OK) return st;
    p.ext_stats = reinterpret_cast<float2*>(ws + sp.stats_off);
    p.ext_rowvec = nullptr;
    p.ext_ptr = nullptr;
    p.epi_flags |= kEpiLse | mask_flag;
    st = launch_group(&p, 1, sp.pl.pairs != 0, s, nullptr, /*lse=*/true);
    if (st != LLMT_B200_OK) return st;
    cudaError_t e = launch_lse_from_stats(row_lse, p.ext_stats, sp.rows, sp.parts, s);
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    // Pass 2: the same tiles again (the same bits: one plan, one order of additions), leaving as
    // exp(v - lse[row]).
    st = fill_problem(&p, &local, ck, sp.pl, probs, a, b);
    if (st != LLMT_B200_OK) return st;
    p.ext_stats = nullptr;
    p.ext_rowvec = row_lse;
    p.ext_ptr = nullptr;
    p.epi_flags |= kEpiExpSub | mask_flag;
    return launch_group(&p, 1, sp.pl.pairs != 0, s, nullptr, /*lse=*/true);
}

int llmt_b200_gemm_softmax_bwd(const llmt_b200_gemm_desc* d, void* ds, const void* a, const void* b,
                               const void* probs, const float* row_dot, int32_t causal, void* stream) {
    Checked ck{};
    int st = validate(d, ds, a, b, &ck);
    if (st != LLMT_B200_OK) return st;
    st = gemm_softmax_check(d, causal, "gemm_softmax_bwd");
    if (st != LLMT_B200_OK) return st;
    if (probs == nullptr || row_dot == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "gemm_softmax_bwd: null probabilities or row sums");
    if (probs == ds || overlaps(probs, ck.c_bytes, ds, ck.c_bytes))
        return fail(LLMT_B200_ERR_INVALID, "gemm_softmax_bwd: the probabilities and dS must not overlap");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    llmt_b200_gemm_desc local = *d;
    local.plan_splits = 1;
    const TcPlan pl = plan_single(&local);
    const Repack rp = repack_plan(&local, ck, a, b);
    const size_t need = pl.workspace_bytes + rp.total();
    if (need > 0) {
        if (d->workspace == nullptr || d->workspace_bytes < need)
            return fail(LLMT_B200_ERR_WORKSPACE, "gemm_softmax_bwd: needs %llu workspace bytes (llmt_b200_gemm_workspace_bytes), got %llu",
                        (unsigned long long)need, (unsigned long long)d->workspace_bytes);
        if (reinterpret_cast<uintptr_t>(d->workspace) & 255u)
            return fail(LLMT_B200_ERR_INVALID, "matmul: workspace must be 256-byte aligned");
    }
    if (rp.total() > 0) {
        st = apply_repack(&local, ck, rp, pl.workspace_bytes, &a, &b, s);
        if (st != LLMT_B200_OK) return st;
    }
    GroupProblem p;
    st = fill_problem(&p, &local, ck, pl, ds, a, b);
    if (st != LLMT_B200_OK) return st;
    p.ext_stats = nullptr;
    p.ext_rowvec = const_cast<float*>(row_dot);
    p.ext_ptr = probs;
    p.epi_flags |= kEpiMulAux | (causal ? kEpiCausal : 0);
    return launch_group(&p, 1, pl.pairs != 0, s, nullptr, /*lse=*/true);
}

int llmt_b200_rowdot(float* out, const void* x, const void* y, int64_t rows, int64_t cols, int64_t ldx,
                     int64_t ldy, int32_t dtype, void* stream) {
    if (out == nullptr || x == nullptr || y == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "rowdot: invalid tensor (null data)");
    if (rows < 0 || cols < 1 || ldx < cols || ldy < cols)
        return fail(LLMT_B200_ERR_INVALID, "rowdot: bad shape (rows %lld, cols %lld, pitches %lld %lld)",
                    (long long)rows, (long long)cols, (long long)ldx, (long long)ldy);
    if (dtype != LLMT_B200_BF16 && dtype != LLMT_B200_FP32)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "rowdot: no kernel for dtype code %d", dtype);
    if (rows == 0) return LLMT_B200_OK;
    cudaError_t e = launch_rowdot(out, x, y, rows, cols, ldx, ldy, dtype == LLMT_B200_BF16, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_cross_entropy_fwd(float* loss, float* row_nll, const float* logits, const int32_t* targets,
                                const float* mask, int64_t rows, int64_t vocab, int64_t ld, void* stream) {
    if (loss == nullptr || row_nll == nullptr || logits == nullptr || targets == nullptr || mask == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "cross_entropy_fwd: invalid tensor (null data)");
    if (rows < 1 || vocab < 1 || ld < vocab)
        return fail(LLMT_B200_ERR_INVALID, "cross_entropy_fwd: bad shape (rows %lld, vocab %lld, pitch %lld)",
                    (long long)rows, (long long)vocab, (long long)ld);
    cudaError_t e = launch_cross_entropy_fwd(loss, row_nll, logits, targets, mask, rows, vocab, ld,
                                             static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_exchange_begin_step(const llmt_b200_comm_desc* comm, void* stream) {
    if (comm == nullptr || comm->rank < 0 || comm->rank >= kMaxCommRanks || comm->flags[comm->rank] == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "exchange_begin_step: bad exchange descriptor");
    cudaError_t e = launch_exchange_begin_step(static_cast<uint32_t*>(comm->flags[comm->rank]) + kRideStep,
                                               static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}


int llmt_b200_gemm_grouped_workspace_bytes(const llmt_b200_gemm_desc* descs, int32_t count,
                                           uint64_t* bytes_per_problem) {
    if (descs == nullptr || bytes_per_problem == nullptr || count < 1 || count > kMaxGroupProblems)
        return fail(LLMT_B200_ERR_INVALID, "gemm_grouped_workspace_bytes: bad argument");
    TcPlan plans[kMaxGroupProblems];
    plan_group(descs, count, plans);
    for (int i = 0; i < count; ++i) {
        Checked ck{};
        shape_only(descs[i], &ck);
        bytes_per_problem[i] = is_tc_problem(descs[i])
                                   ? plans[i].workspace_bytes + repack_plan(&descs[i], ck, nullptr, nullptr).total() : 0;
    }
    return LLMT_B200_OK;
}

uint64_t llmt_b200_gemm_workspace_bytes(const llmt_b200_gemm_desc* d) {
    return llmt_b200_gemm_workspace_bytes_for(d, nullptr, nullptr);
}

uint64_t llmt_b200_gemm_workspace_bytes_for(const llmt_b200_gemm_desc* d, const void* a, const void* b) {
    if (d == nullptr || !is_tc_problem(*d)) return 0;
    Checked ck{};
    shape_only(*d, &ck);
    return plan_single(d).workspace_bytes + repack_plan(d, ck, a, b).total();
}

int llmt_b200_gemm_plan(const llmt_b200_gemm_desc* d, char* buf, size_t n) {
    if (d == nullptr || buf == nullptr || n == 0) return fail(LLMT_B200_ERR_INVALID, "plan: null argument");
    if (d->dtype_ab != LLMT_B200_BF16) {
        snprintf(buf, n, "fp32-simt tile=64x64x16 grid=%lldx%lldx%lld",
                 (long long)((d->n + 63) / 64), (long long)((d->m + 63) / 64), (long long)d->batch);
        return LLMT_B200_OK;
    }
    const TcPlan pl = plan_single(d);
    const int units = pl.pairs ? pair_units() : sm_count();
    const int64_t tickets = pl.num_tiles + pl.colsum_tiles + pl.fin_tiles;
    snprintf(buf, n, "tcgen05 %s tile=%dx%dx64 stages=%d splits=%d tiles=%dx%d kblocks=%d dbias_tickets=%d grid=%d smem=%zu ws=%zu resident_pairs=%d",
             pl.pairs ? "cta-pair" : "1-cta", pl.pairs ? 256 : 128, pl.bn, pl.pairs ? tc_pair_stages() : 4, pl.splits, pl.tiles_m,
             pl.tiles_n, pl.kblocks_total, pl.colsum_tiles + pl.fin_tiles,
             static_cast<int>(tickets < units ? tickets : units) * (pl.pairs ? 2 : 1),
             tc_grouped_smem_bytes(), pl.workspace_bytes, pl.pairs ? max_resident_pairs() : 0);
    return LLMT_B200_OK;
}

int llmt_b200_softmax_fwd(void* y, const void* x, int64_t rows, int64_t tq, int64_t tk, int32_t dtype,
                          int32_t causal, void* stream) {
    if (y == nullptr || x == nullptr) return fail(LLMT_B200_ERR_INVALID, "softmax_fwd: invalid tensor (null data)");
    if (rows < 0 || tq <= 0 || tk <= 0) return fail(LLMT_B200_ERR_INVALID, "softmax_fwd: bad shape");
    if (causal && tq != tk)
        return fail(LLMT_B200_ERR_INVALID, "softmax_fwd: causal mask requires square scores (Tq=%lld Tk=%lld)",
                    (long long)tq, (long long)tk);
    if (dtype != LLMT_B200_FP32 && dtype != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "softmax_fwd: no kernel for dtype code %d", dtype);
    if (rows == 0) return LLMT_B200_OK;
    cudaError_t e = launch_softmax_fwd(y, x, rows, tq, tk, dtype == LLMT_B200_BF16, causal,
                                       static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_softmax_bwd(void* ds, const void* p, const void* dp, int64_t rows, int64_t tk,
                          int32_t dtype, void* stream) {
    if (ds == nullptr || p == nullptr || dp == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "softmax_bwd: invalid tensor (null data)");
    if (rows < 0 || tk <= 0) return fail(LLMT_B200_ERR_INVALID, "softmax_bwd: bad shape");
    if (dtype != LLMT_B200_FP32 && dtype != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "softmax_bwd: no kernel for dtype code %d", dtype);
    if (rows == 0) return LLMT_B200_OK;
    cudaError_t e = launch_softmax_bwd(ds, p, dp, rows, tk, dtype == LLMT_B200_BF16,
                                       static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_head_merge(void* y, const void* x, int64_t b, int64_t h, int64_t t, int64_t hd, int32_t dtype,
                         void* stream) {
    if (y == nullptr || x == nullptr) return fail(LLMT_B200_ERR_INVALID, "permute_merge: invalid tensor (null data)");
    if (b < 0 || h <= 0 || t < 0 || hd <= 0) return fail(LLMT_B200_ERR_INVALID, "permute_merge: bad shape");
    if (dtype != LLMT_B200_FP32 && dtype != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "permute_merge: no kernel for dtype code %d", dtype);
    const int es = dtype == LLMT_B200_BF16 ? 2 : 4;
    const size_t bytes = static_cast<size_t>(b) * h * t * hd * es;
    if (bytes == 0) return LLMT_B200_OK;
    if (overlaps(y, bytes, x, bytes)) return fail(LLMT_B200_ERR_INVALID, "permute_merge: y must not alias x");
    cudaError_t e = launch_head_merge(y, x, b, h, t, hd, es, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_head_split(void* q, void* k, void* v, const void* qkv, int64_t b, int64_t h, int64_t t, int64_t hd,
                         int32_t dtype, void* stream) {
    if (q == nullptr || k == nullptr || v == nullptr || qkv == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "permute_split: invalid tensor (null data)");
    if (b < 0 || h <= 0 || t < 0 || hd <= 0) return fail(LLMT_B200_ERR_INVALID, "permute_split: bad shape");
    if (dtype != LLMT_B200_FP32 && dtype != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "permute_split: no kernel for dtype code %d", dtype);
    const int es = dtype == LLMT_B200_BF16 ? 2 : 4;
    const size_t part = static_cast<size_t>(b) * h * t * hd * es;
    if (part == 0) return LLMT_B200_OK;
    for (const void* out : {q, k, v})
        if (overlaps(out, part, qkv, 3 * part)) return fail(LLMT_B200_ERR_INVALID, "permute_split: outputs must not alias qkv");
    cudaError_t e = launch_head_split(q, k, v, qkv, b, h, t, hd, es, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_device_status(int32_t* code, int32_t* detail) {
    DeviceStatus* dp = device_status_ptr();
    if (dp == nullptr) return fail(LLMT_B200_ERR_CUDA, "cannot resolve the device status word");
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "device synchronize failed: %s", cudaGetErrorString(e));
    DeviceStatus h{};
    e = cudaMemcpy(&h, dp, sizeof h, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "status read failed: %s", cudaGetErrorString(e));
    if (code) *code = h.code;
    if (detail) *detail = h.detail;
    if (h.code != 0) {
        DeviceStatus z{};
        cudaMemcpy(dp, &z, sizeof z, cudaMemcpyHostToDevice);
        // A kernel that gave up may have left its tile-queue counter part-way; results of
        // launches that were in flight are void, later launches start from clean counters.
        DeviceGlobals* g = device_globals_slot();
        if (g != nullptr && g->ready) {
            cudaMemset(g->counters, 0, sizeof(int32_t) * kSchedSlots);
            cudaMemset(g->dbias_sync, 0, sizeof(int32_t) * kSchedSlots * 2);
            cudaMemset(g->ride_counters, 0, sizeof(int32_t) * kSchedSlots);
        }
        return fail(LLMT_B200_ERR_DEVICE, "a kernel gave up on a bounded wait: code %d detail %d block %d",
                    h.code, h.detail, h.block);
    }
    return LLMT_B200_OK;
}

namespace {
int fill_comm(llmt_b200::CommRank* c, const llmt_b200_comm_desc* d, int64_t offset, int64_t count) {
    using namespace llmt_b200;
    if (d == nullptr) return fail(LLMT_B200_ERR_INVALID, "allreduce: null communicator");
    if (d->world < 1 || d->world > kMaxCommRanks || d->rank < 0 || d->rank >= d->world)
        return fail(LLMT_B200_ERR_INVALID, "allreduce: rank %d / world %d out of range (1..%d ranks)", d->rank,
                    d->world, kMaxCommRanks);
    if (offset < 0 || count < 0 || offset % 4 != 0 || count % 4 != 0)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "allreduce: offset and count must be non-negative multiples of 4 floats");
    const int64_t shard = (count / 4 + d->world - 1) / d->world * 4;
    if (d->slot_elems % 4 != 0 || shard > d->slot_elems)
        return fail(LLMT_B200_ERR_WORKSPACE, "allreduce: staging slot of %lld floats too small (need %lld)",
                    static_cast<long long>(d->slot_elems), static_cast<long long>(shard));
    if (d->epoch == nullptr) return fail(LLMT_B200_ERR_INVALID, "allreduce: null epoch buffer");
    for (int r = 0; r < d->world; ++r) {
        if (d->grad[r] == nullptr || d->stage[r] == nullptr || d->flags[r] == nullptr)
            return fail(LLMT_B200_ERR_INVALID, "allreduce: null buffer for rank %d", r);
        if ((reinterpret_cast<uintptr_t>(d->grad[r]) | reinterpret_cast<uintptr_t>(d->stage[r])) % 16 != 0)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "allreduce: buffers of rank %d not 16-byte aligned", r);
        c->grad[r] = static_cast<float*>(d->grad[r]);
        c->stage[r] = static_cast<float*>(d->stage[r]);
        c->flags[r] = static_cast<uint32_t*>(d->flags[r]);
    }
    if (reinterpret_cast<uintptr_t>(d->grad_mc) % 16 != 0)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "allreduce: multicast address not 16-byte aligned");
    c->grad_mc = static_cast<float*>(d->grad_mc);
    c->epoch = static_cast<uint32_t*>(d->epoch);
    c->status = device_status_ptr();
    if (c->status == nullptr) return fail(LLMT_B200_ERR_CUDA, "cannot resolve the device status word");
    c->slot_elems = d->slot_elems;
    c->rank = d->rank;
    c->world = d->world;
    return LLMT_B200_OK;
}
}  // namespace

int llmt_b200_grad_allreduce(const llmt_b200_comm_desc* comm, int64_t offset, int64_t count, int32_t ctas,
                             void* stream) {
    using namespace llmt_b200;
    if (ctas < 1 || ctas > kMaxCommCtas)
        return fail(LLMT_B200_ERR_INVALID, "allreduce: ctas must be 1..%d", kMaxCommCtas);
    thread_local AllreduceParams p;
    int st = fill_comm(&p.ctx[0], comm, offset, count);
    if (st != LLMT_B200_OK) return st;
    if (comm->world == 1 || count == 0) return LLMT_B200_OK;
    p.offset = offset;
    p.count = count;
    p.wait_limit_ns = g_comm_wait_limit_ns;
    cudaError_t e = comm->grad_mc != nullptr ? launch_grad_allreduce_mc(p, ctas, static_cast<cudaStream_t>(stream))
                                             : launch_grad_allreduce(p, ctas, 0, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_grad_allreduce_emulated(const llmt_b200_comm_desc* comms, int32_t world, int64_t offset,
                                      int64_t count, int32_t ctas, void* stream) {
    using namespace llmt_b200;
    if (comms == nullptr || world < 1 || world > kMaxCommRanks)
        return fail(LLMT_B200_ERR_INVALID, "allreduce: world must be 1..%d", kMaxCommRanks);
    if (ctas < 1 || ctas > kMaxCommCtas)
        return fail(LLMT_B200_ERR_INVALID, "allreduce: ctas must be 1..%d", kMaxCommCtas);
    thread_local AllreduceParams p;
    for (int r = 0; r < world; ++r) {
        if (comms[r].world != world || comms[r].rank != r)
            return fail(LLMT_B200_ERR_INVALID, "allreduce: descriptor %d is not rank %d of %d", r, r, world);
        int st = fill_comm(&p.ctx[r], &comms[r], offset, count);
        if (st != LLMT_B200_OK) return st;
    }
    if (world == 1 || count == 0) return LLMT_B200_OK;
    p.offset = offset;
    p.count = count;
    p.wait_limit_ns = g_comm_wait_limit_ns;
    cudaError_t e = launch_grad_allreduce(p, ctas, world, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_zero_grads(float* span, int64_t count, void* stream) {
    using namespace llmt_b200;
    if (count < 0) return fail(LLMT_B200_ERR_INVALID, "zero_grads: negative count");
    if (count == 0) return LLMT_B200_OK;
    if (span == nullptr) return fail(LLMT_B200_ERR_INVALID, "zero_grads: invalid tensor (null data)");
    if (reinterpret_cast<uintptr_t>(span) % sizeof(float) != 0)
        return fail(LLMT_B200_ERR_INVALID, "zero_grads: span is not aligned to its element type");
    cudaError_t e = launch_zero_f32(span, count, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    return LLMT_B200_OK;
}

int llmt_b200_set_sm_budget(int32_t sms) {
    if (sms < 0) {
        fail(LLMT_B200_ERR_INVALID, "sm budget: must be >= 0 (0 = every SM)");
        return -1;
    }
    const int prev = g_sm_budget;
    g_sm_budget = sms;
    return prev;
}

int llmt_b200_set_wait_limit_ns(uint64_t gemm_ns, uint64_t exchange_ns) {
    if (gemm_ns != 0) g_wait_limit_ns = gemm_ns;
    if (exchange_ns != 0) g_comm_wait_limit_ns = exchange_ns;
    return LLMT_B200_OK;
}

void llmt_b200_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses) {
    if (hits != nullptr) *hits = g_map_cache_hits.load(std::memory_order_relaxed);
    if (misses != nullptr) *misses = g_map_cache_misses.load(std::memory_order_relaxed);
}

uint64_t llmt_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* llmt_b200_last_error(void) { return g_err; }

int llmt_b200_abi_version(void) { return LLMT_B200_ABI_VERSION; }

}  // extern "C"
