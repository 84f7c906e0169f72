// Internal declarations shared by the kernels and the C-ABI front end.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace llmt_b200 {

// Device-side health word (see llmt_b200_device_status in the public header).
// code: 0 healthy; otherwise the first failure recorded wins.
struct DeviceStatus {
    int32_t code;
    int32_t detail;
    int32_t block;
    int32_t reserved;
};

enum DeviceErr : int32_t {
    kDevOk = 0,
    kDevWaitSmemEmpty = 1,   // TMA producer gave up waiting for a free pipeline slot
    kDevWaitSmemFull = 2,    // MMA issuer gave up waiting for operand bytes to land
    kDevWaitTmemEmpty = 3,   // MMA issuer gave up waiting for the epilogue to drain an accumulator
    kDevWaitTmemFull = 4,    // epilogue gave up waiting for an accumulator to complete
    kDevWaitSched = 5,       // a role gave up waiting on the tile scheduler ring
    kDevWaitPeer = 6         // the gradient all-reduce gave up waiting for a peer rank's flag
};

constexpr int kEpiBias = 1;
constexpr int kEpiGelu = 2;
// Row-wise epilogues that only the kernels built with the extended epilogue carry out:
constexpr int kEpiLse = 0x100;     // per row and per half tile: maximum and sum of exponentials -> ext_stats
constexpr int kEpiCausal = 0x200;  // columns beyond the row's own index do not exist (value exactly 0 when stored)
constexpr int kEpiExpSub = 0x400;  // v = exp(v - ext_rowvec[row])
constexpr int kEpiMulAux = 0x800;  // v = aux[row, col] * (v - ext_rowvec[row]), aux laid out like C
constexpr int kEpiSavePre = 0x4000; // the value before the GELU is stored too, at aux[row, col] (aux laid out like C)
constexpr int kEpiGeluBwd = 0x2000; // v = v * gelu'(aux[row, col]), aux (the pre-activation) laid out like C
constexpr int kEpiCeGrad = 0x1000; // v = (exp(v - lse[row]) - [col == target[row]]) * g[row]: the cross-entropy's dLogits

constexpr int kMaxGroupProblems = 8;

// One GEMM of a group as the tensor-core kernel sees it: the scalars, which the kernel copies
// into shared memory once (a problem is picked per tile at run time, and reading kernel
// parameters through a run-time index is slow), and the tensor maps, which TMA reads in place.
struct ProblemScalars {
    int64_t m, n, k;
    int32_t batch;
    int32_t batch_inner;        // > 0: batch item b is item b % batch_inner of group b / batch_inner (two-level layout)
    float inv_batch_inner;
    int32_t tiles_m, tiles_n, splits;
    float inv_tiles_m, inv_tiles_n, inv_splits;  // reciprocals, for the kernel's ticket decoding
    int32_t kblocks_total;      // ceil(k / 64)
    int32_t kblocks_per_split;  // k-blocks handled by each split (the last one may be shorter)
    int32_t bn;                 // tile width along N: 64, 128, 192 or 256 (tile height is 128 per CTA)
    int32_t a_mn, b_mn;         // operand stored with M / N contiguous (transposed use)
    int32_t tile_begin;         // first MMA tile of this problem in the group's queue
    int32_t num_tiles;          // tiles_m * tiles_n * splits * batch
    int32_t dbias_mode;         // 0 none; 1 column sums of A stored [k, m] by tickets (two phases); 2 row sums of A stored
                                // [m, k] by tickets; 3 column sums of A stored [k, m] from the stages in shared memory
    int32_t colsum_begin;       // first dbias ticket of this problem in the group's queue
    int32_t colsum_tiles;       // mode 1: chunks of rows of A; mode 2: blocks of rows of op(A)
    int32_t dbias_rows;         // mode 1: rows of A per ticket
    int32_t fin_begin;          // first finishing ticket of this problem (mode 1), relative to the group's first
    int32_t fin_tiles;          // finishing tickets: blocks of 256 values of i per CTA
    void* c;
    int64_t ldc, stride_c;
    int64_t stride_c_outer;     // two-level layout: elements between groups of batch items of C
    int32_t c_is_bf16;
    int32_t c_tma;              // map_c is valid: tiles leave through shared memory + TMA store
    int32_t ws_tma;             // map_ws is valid
    float alpha, beta;
    const void* bias;
    int32_t bias_is_bf16;
    int32_t epi_flags;
    const void* a_raw;          // A as the dbias reduction reads it (plain loads): base and row pitch
    int64_t lda;
    float* ws;                  // split-K partial sums [batch][splits][m][n] fp32 (splits > 1)
    float* dbias;               // fp32 [m] or null
    float dbias_beta;
    float* ws_dbias;            // mode 1: [colsum_tiles][m] fp32 partial sums; mode 3 with splits: [splits][m]
    // Extended epilogue (the kernels built with it only; which parts run: epi_flags).
    //   kEpiLse: per row and per half tile the maximum and the sum of exponentials of the columns
    //            produced go to ext_stats; if ext_ptr is set it is the rows' target columns
    //            (int32 [m], one product only) and the target's value goes to ext_rowvec.
    //   kEpiExpSub / kEpiMulAux: ext_rowvec is READ, one value per row of every batch item;
    //            kEpiMulAux reads ext_ptr as the aux tensor (C's element type, pitch and strides).
    //   kEpiSavePre: ext_ptr is WRITTEN: the pre-activation, C's element type, pitch and strides.
    //   kEpiGeluBwd: ext_ptr is the aux tensor (the pre-activation; C's element type, pitch and strides).
    //   kEpiCeGrad: ext_stats is READ as one (lse, g) pair per row, ext_ptr is the rows' target
    //            columns (int32 [m], one product only).
    float2* ext_stats;          // [2 * tiles_n][batch][m]
    float* ext_rowvec;          // [batch][m]
    const void* ext_ptr;
};
static_assert(sizeof(ProblemScalars) % 8 == 0 && sizeof(ProblemScalars) <= 264, "ProblemScalars is copied to shared memory");

struct alignas(64) GroupProblem : ProblemScalars {
    CUtensorMap map_a, map_b;   // operand loads (128B swizzle)
    CUtensorMap map_c;          // C store: boxes of 32 rows x 128 bytes (64 bf16 or 32 fp32 columns)
    CUtensorMap map_ws;         // split-K partial sums [batch*splits][m][n] fp32, same boxes
};

// ---- gradient all-reduce over peer memory -------------------------------------------------
constexpr int kMaxCommRanks = 8;
constexpr int kMaxCommCtas = 128;
constexpr int kCommThreads = 256;
// Words behind the per-CTA flag words of an exchange (offsets in 32-bit words from `flags`):
// kRideReady + w = "rank w's partial sums of ride-along exchange e are complete" (written by rank w
// into every other rank's copy), kRideStep = this rank's step counter (local).
constexpr int kRideWords = 2 * kMaxCommRanks * kMaxCommCtas;
constexpr int kRideReady = kRideWords;
constexpr int kRideStep = kRideWords + kMaxCommRanks;
constexpr int kMaxRidesPerStep = 16;

// A range of the gradient span that a GEMM launch sums over the ranks on the side ("rides along"):
// tickets that only the epilogue warps work on, through the NVSwitch multicast mapping of the
// span, while the tensor pipe runs the launch's tiles.  tiles == 0: none.
struct RideExchange {
    float* mc;                             // multicast address of the first float of the range
    int64_t n4;                            // length of the range in 16-byte units
    uint32_t* local;                       // this rank's flag words
    uint32_t* peer_ready[kMaxCommRanks];   // [r]: where this rank announces itself to rank r
    int32_t world, rank;
    int32_t index;                         // which ride-along exchange of the step (0 .. kMaxRidesPerStep-1)
    int32_t tiles;                         // chunks this rank's share of the range is cut into
};

struct GroupParams {
    GroupProblem prob[kMaxGroupProblems];
    RideExchange ride;
    int32_t* ride_counter;      // the side warps draw the exchange's chunks from it; zero between launches
    int32_t num_problems;
    int32_t total_tiles;        // tickets of the launch: dbias reductions, MMA tiles, dbias finishing tickets
    int32_t colsum_total;       // tickets [0, colsum_total) are dbias reductions
    int32_t fin_begin;          // tickets [fin_begin, total_tiles) finish the two-phase dbias reductions
    int32_t* dbias_sync;        // [2] arrival counters of the two phases; zero between launches
    int32_t static_schedule;    // 1 = ticket i goes to CTA i % grid instead of the dynamic queue
    int32_t* sched_counter;     // zero between launches; the kernel re-arms it
    DeviceStatus* status;
    uint64_t wait_limit_ns;     // every wait inside the kernel gives up after this long
};

// One rank's view of the exchange: the same three buffers on every rank, as pointers this
// rank can dereference ([rank] = its own copy), plus its private call counters.
struct CommRank {
    float* grad[kMaxCommRanks];      // flat fp32 gradient span
    float* grad_mc;                  // the span through an NVSwitch multicast mapping, or null
    float* stage[kMaxCommRanks];     // staging area: `world` slots of slot_elems floats
    uint32_t* flags[kMaxCommRanks];  // [2 phases][kMaxCommRanks writers][kMaxCommCtas] call counters
    uint32_t* epoch;                 // [kMaxCommCtas] calls completed by each CTA of this rank
    DeviceStatus* status;
    int64_t slot_elems;
    int32_t rank, world;
};

struct AllreduceParams {
    CommRank ctx[kMaxCommRanks];     // [0] on a real rank; one per rank when emulated on one device
    int64_t offset, count;           // range of the span, in floats (multiples of 4)
    uint64_t wait_limit_ns;          // every cross-rank wait gives up after this long
};

cudaError_t launch_grad_allreduce(const AllreduceParams& p, int ctas, int emulated_ranks, cudaStream_t stream);
cudaError_t launch_grad_allreduce_mc(const AllreduceParams& p, int ctas, cudaStream_t stream);
cudaError_t launch_exchange_begin_step(uint32_t* step_word, cudaStream_t stream);

// Plan of one problem: the pure function of the problem (and of the work it shares a
// launch with) that fixes tile width and split count.
struct TcPlan {
    int bn;
    int pairs;       // 1 = CTA pairs (256-row tiles, cta_group::2)
    int splits;
    int tiles_m, tiles_n;
    int kblocks_total, kblocks_per_split;
    int64_t num_tiles;
    int dbias_mode;     // 0 none, 1 column sums in two phases, 2 row sums, 3 column sums from shared memory
    int colsum_tiles;   // dbias reduction tickets
    int dbias_rows;     // mode 1: rows of A per ticket
    int fin_tiles;      // mode 1: finishing tickets
    size_t ws_dbias_off;  // mode 1: offset of the partial sums inside the workspace
    size_t workspace_bytes;
};

struct Fp32GemmParams {
    int64_t m, n, k, batch;
    const float* a;
    const float* b;
    float* c;
    int64_t lda, ldb, ldc;
    int64_t stride_a, stride_b, stride_c;
    int64_t batch_inner, stride_a_outer, stride_b_outer, stride_c_outer;  // two-level batch layout (batch_inner 0 = plain)
    int32_t trans_a, trans_b;
    float alpha, beta;
    const void* bias;
    int32_t bias_is_bf16;
    int32_t epi_flags;
};

// tanh-GELU in fp32, the expression of llmt's gelu kernel (src/kernels/gelu.cu:23-26).
__device__ __forceinline__ float gelu_tanh_precise(float v) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * v * (1.0f + tanhf(k0 * (v + k1 * v * v * v)));
}

// Same function in the form  gelu(v) = v * sigmoid(2u) = v / (1 + exp(-2u)),
// u = k0*(v + k1*v^3): algebraically identical to 0.5*v*(1+tanh(u)), no cancellation
// for negative v, and five FP32 operations plus one exp2 and one reciprocal on the
// special-function unit per element (relative error of the result ~1e-6).  The epilogue
// warps are bound by the number of instructions they issue, not by the special-function
// unit: forms that trade the reciprocal for Newton steps on the FMA pipe, or use the hardware
// tanh with a guarded tail, measured 20-25 % slower on the GELU launch.
__device__ __forceinline__ float gelu_tanh_fast(float v) {
    const float a0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;  // -2*k0*log2(e)
    const float a1 = a0 * 0.044715f;
    const float w = v * fmaf(a1, v * v, a0);  // -2u * log2(e)
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(w));         // exp(-2u); +inf for very negative v
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));  // sigmoid(2u); 0 when e = +inf
    return v * r;
}

// The same function with the hardware tanh: five FP32 operations and ONE special-function
// operation per element.  tanh.approx is good to 2^-11 relative, so the result carries an
// absolute error of up to 0.5 |v| 2^-11 (2.4e-4 |v|): below the rounding of a bf16 result
// (2^-9 relative) wherever |gelu(v)| > |v| / 8, and at most one bf16 unit of the largest
// negative values (-0.17) on the tail v < -1, where gelu(v) itself tends to zero.  For bf16
// results only.
__device__ __forceinline__ float gelu_tanh_hw(float v) {
    const float k0 = 0.7978845608028654f;  // sqrt(2/pi)
    const float k1 = k0 * 0.044715f;
    const float u = v * fmaf(k1, v * v, k0);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    const float h = 0.5f * v;
    return fmaf(h, t, h);
}

// Derivative of the tanh-GELU, gelu'(x) = 0.5 (1 + t) + 0.5 x (1 - t^2) u'(x) with
// t = tanh(u), u = k0 (x + k1 x^3), u' = k0 (1 + 3 k1 x^2); hardware tanh (2^-11): for results
// that are rounded to bf16.
__device__ __forceinline__ float dgelu_tanh_hw(float x) {
    const float k0 = 0.7978845608028654f;
    const float k1 = k0 * 0.044715f;
    const float x2 = x * x;
    const float u = x * fmaf(k1, x2, k0);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    const float du = fmaf(3.0f * k1, x2, k0);
    const float hx = 0.5f * x;
    return fmaf(hx * du, fmaf(-t, t, 1.0f), fmaf(0.5f, t, 0.5f));
}
// The same with tanhf: for fp32 results.
__device__ __forceinline__ float dgelu_tanh_precise(float x) {
    const float k0 = 0.7978845608028654f;
    const float k1 = k0 * 0.044715f;
    const float x2 = x * x;
    const float t = tanhf(x * fmaf(k1, x2, k0));
    const float du = fmaf(3.0f * k1, x2, k0);
    return fmaf(0.5f * x * du, fmaf(-t, t, 1.0f), fmaf(0.5f, t, 0.5f));
}

// Launchers implemented in the .cu files.  All return a cudaError_t from the launch.
cudaError_t launch_tc_grouped(const GroupParams& gp, int grid, bool pairs, cudaStream_t stream, bool lse = false);
cudaError_t launch_cross_entropy_fwd(float* loss, float* row_nll, const float* logits, const int32_t* targets,
                                     const float* mask, int64_t rows, int64_t v, int64_t ld, cudaStream_t stream);
cudaError_t launch_cross_entropy_from_stats(float* loss, float* row_nll, const void* stats, const float* tgt,
                                            const float* mask, int64_t rows, int parts, cudaStream_t stream);
int max_resident_pairs(void);
cudaError_t launch_splitk_reduce(const GroupProblem& p, cudaStream_t stream);
size_t tc_grouped_smem_bytes(void);
int tc_pair_stages(void);
int tc_dbias_rows_per_cta(void);
int tc_dbias_finish_per_cta(void);
cudaError_t launch_fp32_gemm(const Fp32GemmParams& p, cudaStream_t stream);
cudaError_t launch_fp32_rowsum(const Fp32GemmParams& p, float* dbias, float dbias_beta, cudaStream_t stream);
cudaError_t launch_zero_f32(float* dst, int64_t n, cudaStream_t stream);
cudaError_t launch_repack_bf16(void* dst, const void* src, int64_t rows, int64_t cols, int64_t ld_src,
                               int64_t ld_dst, int64_t batch, int64_t stride_src, int64_t stride_dst,
                               cudaStream_t stream);
cudaError_t launch_softmax_fwd(void* y, const void* x, int64_t rows, int64_t tq, int64_t tk,
                               int is_bf16, int causal, cudaStream_t stream);
cudaError_t launch_softmax_bwd(void* ds, const void* p, const void* dp, int64_t rows, int64_t tk,
                               int is_bf16, cudaStream_t stream);
cudaError_t launch_head_merge(void* y, const void* x, int64_t B, int64_t H, int64_t T, int64_t hd, int elem_bytes,
                              cudaStream_t stream);
cudaError_t launch_head_split(void* q, void* k, void* v, const void* qkv, int64_t B, int64_t H, int64_t T, int64_t hd,
                              int elem_bytes, cudaStream_t stream);
cudaError_t launch_cross_entropy_bwd(float* dlogits, const float* logits, const int32_t* targets, const float* mask,
                                     float dloss, int64_t rows, int64_t v, int64_t ld_in, int64_t ld_out,
                                     cudaStream_t stream);
cudaError_t launch_ce_grad_rows(void* out, const void* stats, const float* lse_in, const float* mask, float* mask_sum,
                                float dloss, int64_t rows, int parts, cudaStream_t stream);
cudaError_t launch_lse_from_stats(float* lse, const void* stats, int64_t rows, int parts, cudaStream_t stream);
cudaError_t launch_rowdot(float* out, const void* x, const void* y, int64_t rows, int64_t cols, int64_t ldx,
                          int64_t ldy, int is_bf16, cudaStream_t stream);
DeviceStatus* device_status_ptr(void);

void count_launch(int n);

}  // namespace llmt_b200
