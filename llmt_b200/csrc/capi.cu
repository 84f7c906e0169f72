// extern "C" front end: argument validation, plan selection, TMA descriptor
// encoding and kernel launch.  Mirrors the checks llmt performs before it calls
// cuBLASLt (llmt: src/kernels/matmul.cpp:175-214) but reports them as status
// codes instead of aborting.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/llmt_b200.h"
#include "common.h"

namespace llmt_b200 {

namespace {

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
    return cached;
}

// Cost of one 64-deep k-block of a 128 x bn tile in SM cycles: the larger of the
// tensor-core time (128*bn*64*2 flop at 8192 flop/clk) and the shared-memory
// operand read time ((128+bn) rows x 128 B at 128 B/clk).
int kblock_cost(int bn) { return bn * 2 > 128 + bn ? bn * 2 : 128 + bn; }

// Split-K factor for a problem that has `tiles` output tiles: only when the
// tiles cannot fill the machine and the reduction is long enough to share.
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

TcPlan make_plan(int64_t m, int64_t n, int64_t k, int64_t batch, bool dbias, int sms,
                 int force_bn = 0, int force_splits = 0) {
    TcPlan pl{};
    const int cands[4] = {256, 192, 128, 64};
    const int tiles_m = static_cast<int>((m + 127) / 128);
    const int kblocks_total = static_cast<int>((k + 63) / 64);
    int best_bn = 0, best_splits = 1;
    int64_t best_cost = 0;
    for (int bn : cands) {
        if (dbias && bn > 192) continue;
        if (force_bn != 0 && bn != force_bn) continue;
        // Never pick a tile wider than needed when a narrower one covers n in one column.
        if (force_bn == 0 && bn > 64 && n <= bn - 64) continue;
        const int64_t tiles = static_cast<int64_t>(tiles_m) * ((n + bn - 1) / bn) * batch;
        int splits = force_splits > 0 ? force_splits : choose_splits(tiles, kblocks_total, sms);
        if (splits > kblocks_total) splits = kblocks_total > 0 ? kblocks_total : 1;
        const int kps = (kblocks_total + splits - 1) / splits;
        const int64_t waves = (tiles * splits + sms - 1) / sms;
        // Estimated cycles: main loops, plus one pass over the partial sums when split.
        int64_t cost = waves * kblock_cost(bn) * (kps > 0 ? kps : 1);
        if (splits > 1) cost += static_cast<int64_t>(splits) * 64;
        if (best_bn == 0 || cost < best_cost) {
            best_bn = bn;
            best_cost = cost;
            best_splits = splits;
        }
    }
    pl.bn = best_bn;
    pl.tiles_m = tiles_m;
    pl.tiles_n = static_cast<int>((n + pl.bn - 1) / pl.bn);
    pl.kblocks_total = kblocks_total;
    const int64_t tiles = static_cast<int64_t>(pl.tiles_m) * pl.tiles_n * batch;
    const int splits = best_splits;
    pl.kblocks_per_split = (pl.kblocks_total + splits - 1) / splits;
    if (pl.kblocks_per_split < 1) pl.kblocks_per_split = 1;
    pl.splits = pl.kblocks_total > 0 ? (pl.kblocks_total + pl.kblocks_per_split - 1) / pl.kblocks_per_split : 1;
    const int64_t total = tiles * pl.splits;
    pl.grid = static_cast<int>(total < sms ? total : sms);
    int stages = 8;
    while (stages > 2 && tc_smem_bytes(pl.bn, stages, dbias) > 227u * 1024u) --stages;
    pl.stages = stages;
    pl.smem_bytes = tc_smem_bytes(pl.bn, stages, dbias);
    pl.workspace_bytes = 0;
    if (pl.splits > 1) {
        size_t ws = static_cast<size_t>(batch) * pl.splits * m * n * sizeof(float);
        ws = (ws + 255) / 256 * 256;
        if (dbias) ws += (static_cast<size_t>(pl.splits) * m * sizeof(float) + 255) / 256 * 256;
        pl.workspace_bytes = ws;
    }
    return pl;
}

bool overlaps(const void* p, size_t pb, const void* q, size_t qb) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p), b = reinterpret_cast<uintptr_t>(q);
    return a < b + qb && b < a + pb;
}

struct Checked {
    int64_t a_rows, a_cols, b_rows, b_cols;
    bool bf16;
};

// Shape/pointer contract; the order and wording follow llmt's check()
// (src/kernels/matmul.cpp:175-214) where a counterpart exists.
int validate(const llmt_b200_gemm_desc* d, const void* c, const void* a, const void* b, Checked* out) {
    if (d == nullptr) return fail(LLMT_B200_ERR_INVALID, "matmul: null descriptor");
    if (c == nullptr || a == nullptr || b == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "matmul: invalid tensor (null data)");
    if (d->m < 0 || d->n < 0 || d->k < 0 || d->batch < 0)
        return fail(LLMT_B200_ERR_INVALID, "matmul: negative dimension");
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
    if (d->batch > 1) {
        if (d->stride_a < (out->a_rows - 1) * d->lda + out->a_cols ||
            d->stride_b < (out->b_rows - 1) * d->ldb + out->b_cols ||
            d->stride_c < (d->m - 1) * d->ldc + d->n)
            return fail(LLMT_B200_ERR_INVALID, "matmul: batch stride smaller than one matrix");
    }
    if (d->plan_tile_n != 0 && d->plan_tile_n != 64 && d->plan_tile_n != 128 &&
        d->plan_tile_n != 192 && d->plan_tile_n != 256)
        return fail(LLMT_B200_ERR_INVALID, "matmul: plan_tile_n must be 0, 64, 128, 192 or 256");
    if (d->plan_tile_n == 256 && d->dbias != nullptr)
        return fail(LLMT_B200_ERR_INVALID, "matmul: the fused dbias needs plan_tile_n <= 192");
    if (d->plan_splits < 0) return fail(LLMT_B200_ERR_INVALID, "matmul: negative plan_splits");
    if ((d->epilogue & ~(LLMT_B200_EPI_BIAS | LLMT_B200_EPI_GELU)) != 0)
        return fail(LLMT_B200_ERR_INVALID, "matmul: unknown epilogue flags 0x%x", d->epilogue);
    if ((d->epilogue & LLMT_B200_EPI_BIAS) && d->bias == nullptr)
        return fail(LLMT_B200_ERR_INVALID, "matmul: EPI_BIAS set but bias is null");
    if ((d->epilogue & LLMT_B200_EPI_BIAS) && d->bias_dtype != LLMT_B200_FP32 &&
        d->bias_dtype != LLMT_B200_BF16)
        return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: bias dtype code %d not supported", d->bias_dtype);
    if (d->dbias != nullptr) {
        if (!out->bf16)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: dbias is fused only into the bf16 path");
        if (d->batch > 1)
            return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: dbias with a batched product is not defined");
    }
    // Aliasing: C is updated in place; it must not overlap an input.
    const size_t es_ab = out->bf16 ? 2 : 4, es_c = d->dtype_c == LLMT_B200_BF16 ? 2 : 4;
    const int64_t nb = d->batch > 0 ? d->batch : 1;
    if (d->m > 0 && d->n > 0 && d->k > 0) {
        const size_t a_bytes = static_cast<size_t>((nb - 1) * (nb > 1 ? d->stride_a : 0) +
                                                   (out->a_rows - 1) * d->lda + out->a_cols) * es_ab;
        const size_t b_bytes = static_cast<size_t>((nb - 1) * (nb > 1 ? d->stride_b : 0) +
                                                   (out->b_rows - 1) * d->ldb + out->b_cols) * es_ab;
        const size_t c_bytes = static_cast<size_t>((nb - 1) * (nb > 1 ? d->stride_c : 0) +
                                                   (d->m - 1) * d->ldc + d->n) * es_c;
        if (overlaps(c, c_bytes, a, a_bytes) || overlaps(c, c_bytes, b, b_bytes))
            return fail(LLMT_B200_ERR_INVALID, "matmul: C overlaps an input");
    }
    return LLMT_B200_OK;
}

// Tensor map over one row-major matrix [rows, cols] (pitch ld, `batch` items `stride`
// elements apart) with a box of box_cols x box_rows elements.  elem_bytes 2 = bf16, 4 = fp32.
int encode_map(CUtensorMap* map, const void* base, int elem_bytes, int64_t rows, int64_t cols,
               int64_t ld, int64_t batch, int64_t stride, int box_cols, int box_rows,
               CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return fail(LLMT_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    const cuuint64_t stride_elems = batch > 1 ? static_cast<cuuint64_t>(stride)
                                              : static_cast<cuuint64_t>(rows) * ld;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                          static_cast<cuuint64_t>(batch > 1 ? batch : 1)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * elem_bytes, stride_elems * elem_bytes};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                          3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(LLMT_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d "
                    "(rows=%lld cols=%lld ld=%lld batch=%lld)", static_cast<int>(r),
                    (long long)rows, (long long)cols, (long long)ld, (long long)batch);
    return LLMT_B200_OK;
}

// bf16 operand map boxed for 128-byte-swizzled tiles (64 elements wide).
int encode_operand_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t ld,
                       int64_t batch, int64_t stride, int box_rows) {
    return encode_map(map, base, 2, rows, cols, ld, batch, stride, 64, box_rows,
                      CU_TENSOR_MAP_SWIZZLE_128B);
}

int run_bf16(const llmt_b200_gemm_desc* d, const Checked& ck, void* c, const void* a, const void* b,
             cudaStream_t stream) {
    // TMA needs 16-byte aligned bases and pitches.
    if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(b) & 15u))
        return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: bf16 operands must start on a 16-byte boundary");
    if ((d->lda % 8) != 0 || (d->ldb % 8) != 0 ||
        (d->batch > 1 && ((d->stride_a % 8) != 0 || (d->stride_b % 8) != 0)))
        return fail(LLMT_B200_ERR_UNSUPPORTED,
                    "matmul: bf16 row pitch / batch stride must be a multiple of 8 elements "
                    "(lda=%lld ldb=%lld)", (long long)d->lda, (long long)d->ldb);
    const bool dbias = d->dbias != nullptr;
    const TcPlan pl = make_plan(d->m, d->n, d->k, d->batch, dbias, sm_count(), d->plan_tile_n, d->plan_splits);
    if (pl.workspace_bytes > 0) {
        if (d->workspace == nullptr || d->workspace_bytes < pl.workspace_bytes)
            return fail(LLMT_B200_ERR_WORKSPACE, "matmul: split-K needs %llu workspace bytes, got %llu",
                        (unsigned long long)pl.workspace_bytes, (unsigned long long)d->workspace_bytes);
        if (reinterpret_cast<uintptr_t>(d->workspace) & 255u)
            return fail(LLMT_B200_ERR_INVALID, "matmul: workspace must be 256-byte aligned");
    }
    TcGemmParams p{};
    p.m = d->m; p.n = d->n; p.k = d->k;
    p.batch = static_cast<int32_t>(d->batch);
    p.tiles_m = pl.tiles_m; p.tiles_n = pl.tiles_n; p.splits = pl.splits;
    p.kblocks_total = pl.kblocks_total;
    p.kblocks_per_split = pl.kblocks_per_split;
    p.total_tiles = static_cast<int64_t>(pl.tiles_m) * pl.tiles_n * pl.splits * d->batch;
    p.c = c; p.ldc = d->ldc; p.stride_c = d->batch > 1 ? d->stride_c : 0;
    p.c_is_bf16 = d->dtype_c == LLMT_B200_BF16;
    p.alpha = d->alpha; p.beta = d->beta;
    p.bias = d->bias; p.bias_is_bf16 = d->bias_dtype == LLMT_B200_BF16;
    p.epi_flags = d->epilogue;
    p.dbias = d->dbias; p.dbias_beta = d->dbias_beta;
    p.status = device_status_ptr();
    if (p.status == nullptr) return fail(LLMT_B200_ERR_CUDA, "cannot resolve the device status word");
    if (pl.splits > 1) {
        p.ws = static_cast<float*>(d->workspace);
        size_t ws = static_cast<size_t>(d->batch) * pl.splits * d->m * d->n * sizeof(float);
        ws = (ws + 255) / 256 * 256;
        p.ws_dbias = dbias ? reinterpret_cast<float*>(static_cast<char*>(d->workspace) + ws) : nullptr;
    }
    if (d->k == 0) {
        // Empty reduction: C = epilogue(beta * C).  The reduce kernel with zero
        // partial sums computes exactly that.
        p.splits = 0;
        cudaError_t e = launch_splitk_reduce(p, stream);
        if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
        return LLMT_B200_OK;
    }
    const int a_mn = d->trans_a ? 1 : 0;  // A stored [k, m]: m contiguous
    const int b_mn = d->trans_b ? 0 : 1;  // B stored [k, n]: n contiguous
    CUtensorMap ma, mb;
    int st = encode_operand_map(&ma, a, ck.a_rows, ck.a_cols, d->lda, d->batch, d->stride_a,
                                a_mn ? 64 : 128);
    if (st != LLMT_B200_OK) return st;
    st = encode_operand_map(&mb, b, ck.b_rows, ck.b_cols, d->ldb, d->batch, d->stride_b,
                            b_mn ? 64 : pl.bn);
    if (st != LLMT_B200_OK) return st;
    // C leaves through shared memory and TMA stores when its layout allows a tensor map
    // (16-byte aligned base, pitch and batch stride); otherwise straight from registers.
    CUtensorMap mc;
    memset(&mc, 0, sizeof mc);
    const int ces = p.c_is_bf16 ? 2 : 4;
    if ((reinterpret_cast<uintptr_t>(c) & 15u) == 0 && (d->ldc * ces) % 16 == 0 &&
        (d->batch <= 1 || (d->stride_c * ces) % 16 == 0) && pl.splits == 1) {
        st = encode_map(&mc, c, ces, d->m, d->n, d->ldc, d->batch, d->stride_c, 32, 128,
                        p.c_is_bf16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
        if (st != LLMT_B200_OK) return st;
        p.c_tma = 1;
    }
    cudaError_t e = launch_tc_gemm(pl, a_mn, b_mn, ma, mb, mc, p, stream);
    if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    if (pl.splits > 1) {
        e = launch_splitk_reduce(p, stream);
        if (e != cudaSuccess) return fail(LLMT_B200_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
    }
    return LLMT_B200_OK;
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
    p.trans_a = d->trans_a; p.trans_b = d->trans_b;
    p.alpha = d->alpha; p.beta = d->beta;
    p.bias = d->bias; p.bias_is_bf16 = d->bias_dtype == LLMT_B200_BF16;
    p.epi_flags = d->epilogue;
    if (d->batch > 65535) return fail(LLMT_B200_ERR_UNSUPPORTED, "matmul: fp32 path supports batch <= 65535");
    cudaError_t e = launch_fp32_gemm(p, stream);
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
    const size_t need = make_plan(d->m, d->n, d->k, d->batch, d->dbias != nullptr, sm_count(),
                                  d->plan_tile_n, d->plan_splits).workspace_bytes;
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

uint64_t llmt_b200_gemm_workspace_bytes(const llmt_b200_gemm_desc* d) {
    if (d == nullptr || d->dtype_ab != LLMT_B200_BF16 || d->m <= 0 || d->n <= 0 || d->k <= 0 ||
        d->batch <= 0)
        return 0;
    return make_plan(d->m, d->n, d->k, d->batch, d->dbias != nullptr, sm_count(), d->plan_tile_n,
                     d->plan_splits).workspace_bytes;
}

int llmt_b200_gemm_plan(const llmt_b200_gemm_desc* d, char* buf, size_t n) {
    if (d == nullptr || buf == nullptr || n == 0) return fail(LLMT_B200_ERR_INVALID, "plan: null argument");
    if (d->dtype_ab != LLMT_B200_BF16) {
        snprintf(buf, n, "fp32-simt tile=64x64x16 grid=%lldx%lldx%lld",
                 (long long)((d->n + 63) / 64), (long long)((d->m + 63) / 64), (long long)d->batch);
        return LLMT_B200_OK;
    }
    const TcPlan pl = make_plan(d->m, d->n, d->k, d->batch, d->dbias != nullptr, sm_count(), d->plan_tile_n,
                     d->plan_splits);
    snprintf(buf, n, "tcgen05 tile=128x%dx64 stages=%d splits=%d tiles=%dx%d kblocks=%d grid=%d smem=%zu ws=%zu",
             pl.bn, pl.stages, pl.splits, pl.tiles_m, pl.tiles_n, pl.kblocks_total, pl.grid,
             pl.smem_bytes, pl.workspace_bytes);
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
        return fail(LLMT_B200_ERR_DEVICE, "a kernel gave up on a bounded wait: code %d detail %d block %d",
                    h.code, h.detail, h.block);
    }
    return LLMT_B200_OK;
}

uint64_t llmt_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char* llmt_b200_last_error(void) { return g_err; }

int llmt_b200_abi_version(void) { return LLMT_B200_ABI_VERSION; }

}  // extern "C"
