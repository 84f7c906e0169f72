/*
 * llmt_b200 — C ABI of the B200-native matrix-multiply path for llmt.
 *
 * This is the boundary a host program binds: plain pointers and sizes, no
 * C++ types, no framework types.  Every entry point enqueues work on the CUDA
 * stream it is given and returns without synchronising; nothing here
 * allocates device memory; nothing aborts or throws — errors come back as a
 * non-zero status and llmt_b200_last_error() explains the most recent one on
 * the calling thread.
 *
 * Threading: as in llmt (src/kernels/matmul.cpp:23-27) one host thread at a time issues the
 * calls for a device.  Several devices per process are supported (one thread each, or one
 * thread switching devices): all per-device host state is kept per device, and the first GEMM
 * call on a device does a small synchronous set-up, so make it outside any stream capture.
 *
 * The library replaces the one call llmt makes into cuBLASLt
 * (llmt: src/kernels/matmul.cpp:116-170, reached from kernels::matmul,
 * include/llmt/kernels/matmul.h:23-24).  Tensors are row-major; weights are
 * [out, in]; C is read and written in place when beta != 0.
 *
 * Element type codes are llmt's DType codes (include/llmt/core/dtype.h:15):
 * 0 = fp32, 1 = bf16.
 */
#ifndef LLMT_B200_H
#define LLMT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLMT_B200_ABI_VERSION 5

#if defined(__GNUC__)
#define LLMT_B200_API __attribute__((visibility("default")))
#else
#define LLMT_B200_API
#endif

enum llmt_b200_dtype { LLMT_B200_FP32 = 0, LLMT_B200_BF16 = 1 };

/* Epilogue flags (bit set).  Order of application on the fp32 accumulator:
 *   v = alpha * (op(A) op(B)) + beta * C_in ;  v += bias[j] ;  v = gelu_tanh(v) ;
 *   C = cast(v).
 * gelu_tanh is llmt's formula (src/kernels/gelu.cu:23-26) evaluated in fp32.
 * llmt itself has no bias and runs GELU as a separate kernel
 * (src/layers/mlp.cpp:14-18); with flags == 0 the result is llmt's matmul. */
enum llmt_b200_epilogue {
    LLMT_B200_EPI_NONE = 0,
    LLMT_B200_EPI_BIAS = 1,
    LLMT_B200_EPI_GELU = 2,
    /* C = (alpha * op(A) * op(B)) * gelu'(aux): the dX product of the layer that follows a tanh-GELU,
     * leaving directly as the gradient with respect to the GELU's input.  desc.aux = the saved
     * pre-activation, in C's type, pitch and batch strides.  bf16 operands, beta = 0, alone among
     * the epilogue flags.  (llmt docs/TODO.md:223: gelu_bwd, planned as a kernel of its own.) */
    LLMT_B200_EPI_GELU_BWD = 4,
    /* With EPI_GELU: the value the GELU sees (after alpha, beta and bias) is stored as a second
     * result at desc.aux, in C's type, pitch and batch strides: the pre-activation that
     * EPI_GELU_BWD reads in the backward pass.  One launch gives h = gelu(pre) and pre, where llmt's
     * MLP (src/layers/mlp.cpp:14-18) keeps only the tensor its gelu kernel overwrote.  bf16
     * operands; aux must not overlap anything else the call touches. */
    LLMT_B200_EPI_SAVE_PRE = 8
};

enum llmt_b200_status {
    LLMT_B200_OK = 0,
    LLMT_B200_ERR_INVALID = 1,     /* contract violation (shape, pointer, alignment, aliasing) */
    LLMT_B200_ERR_UNSUPPORTED = 2, /* valid request this build has no kernel for */
    LLMT_B200_ERR_WORKSPACE = 3,   /* workspace missing or smaller than required */
    LLMT_B200_ERR_CUDA = 4,        /* a CUDA runtime / driver call failed */
    LLMT_B200_ERR_DEVICE = 5       /* a kernel gave up on a bounded wait (see device_status) */
};

/*
 * One GEMM problem:  C[b] = epilogue(alpha * op(A[b]) * op(B[b]) + beta * C[b]).
 * Mirrors the Problem llmt derives in src/kernels/matmul.cpp:79-86,175-214,
 * with explicit row pitches added so padded buffers can be used.
 *
 *   op(A) is [m,k]: A is stored [m,k] (trans_a = 0) or [k,m] (trans_a = 1).
 *   op(B) is [k,n]: B is stored [k,n] (trans_b = 0) or [n,k] (trans_b = 1).
 *   lda/ldb/ldc  row pitch in elements of each row-major buffer (>= its column count).
 *                Any pitch and any element-aligned base work.  bf16 operands whose base is
 *                16-byte aligned and whose pitch and batch stride are multiples of 8 elements
 *                are read in place; others (a contiguous [tokens, 50257] matrix, a slice
 *                x[:, 1:]) are first copied to such a layout inside the workspace (one extra
 *                pass over that operand; llmt_b200_gemm_workspace_bytes_for counts it).
 *                m, n, k and batch must be below 2^31 - 1024.
 *   stride_*     elements between consecutive batch items; ignored when batch == 1.
 *   dtype_ab     element type of A and B; dtype_c of C.  Supported pairs:
 *                (fp32, fp32) strict fp32 FMA path; (bf16, bf16) and (bf16, fp32)
 *                tensor-core path with fp32 accumulation.
 *   bias         [n] values added to every row when EPI_BIAS is set (bias_dtype: fp32 or bf16).
 *   dbias        optional fp32 [m]:  dbias[i] = dbias_beta * dbias[i] + sum_p op(A)[i,p].
 *                For llmt's dW call (src/layers/linear.cpp:27-29: A = dy, trans_a = 1)
 *                this is the bias gradient, summed over tokens, in a fixed order, by the same
 *                launch that computes dW (on the strict-fp32 path: by a second small kernel).
 *   Aliasing     C is read and written in place.  C, dbias and the workspace must not overlap
 *                one another, A, B or bias (checked by address range).
 *   plan_*       tuning overrides of the tile width, split-K factor and CTA pairing; 0 leaves the
 *                choice to the library (the default plan is a pure function of the
 *                problem, so results stay reproducible either way).
 *   workspace    device scratch for split-K partial sums and repacked operands;
 *                llmt_b200_gemm_workspace_bytes() gives the size this problem needs (0 for
 *                most problems).  Plays the role of RunCtx::blas_workspace
 *                (include/llmt/core/run_ctx.h:35-36).
 */
typedef struct llmt_b200_gemm_desc {
    int64_t m, n, k, batch;
    int64_t lda, ldb, ldc;
    int64_t stride_a, stride_b, stride_c;
    int32_t trans_a, trans_b;
    int32_t dtype_ab, dtype_c;
    float alpha, beta;
    int32_t epilogue;
    int32_t bias_dtype;
    const void* bias;
    float* dbias;
    float dbias_beta;
    int32_t plan_tile_n;   /* 0 = choose; else force the tile width: 64, 128, 192 or 256 */
    int32_t plan_splits;   /* 0 = choose; else force the split-K factor (>= 1) */
    int32_t plan_cta_pairs; /* 0 = choose; 1 = single CTAs (128-row tiles); 2 = CTA pairs (256-row tiles) */
    void* workspace;
    uint64_t workspace_bytes;
    /* Two-level batch layout (0 = plain: item b sits b * stride_x past the base).  With
     * batch_inner = I > 0 (I divides batch) item b sits (b % I) * stride_x + (b / I) * stride_x_outer
     * past the base, and stride_x may be smaller than one matrix.  This is how the per-head
     * products of an attention layer read Q, K, V straight out of the [B, T, 3*H*hd] output of
     * the QKV projection (ld = 3*H*hd, stride = hd, stride_outer = T*3*H*hd, batch = B*H,
     * batch_inner = H) and write their result straight into [B, T, H*hd]: the head split and
     * merge that llmt runs as copy kernels (src/kernels/permute.cu:18-46) become strides.  bf16
     * operands in such a layout must be addressable by TMA as they are (16-byte aligned base,
     * pitches and strides multiples of 8 elements). */
    int64_t batch_inner;
    int64_t stride_a_outer, stride_b_outer, stride_c_outer;
    const void* aux;       /* EPI_GELU_BWD: read; EPI_SAVE_PRE: written (the library casts the const away); else ignored */
} llmt_b200_gemm_desc;

/* Replaces llmt's kernels::matmul body (src/kernels/matmul.cpp:218-222 ->
 * run(), :116-170).  `stream` is a cudaStream_t.  Deterministic: the same
 * descriptor and inputs give bitwise-identical output on every call. */
LLMT_B200_API int llmt_b200_gemm(const llmt_b200_gemm_desc* desc, void* c, const void* a, const void* b,
                   void* stream);

/* Several independent bf16 problems in ONE launch: a single persistent kernel draws the
 * tiles of all of them from one queue, longest reductions first, so the tail of one
 * product overlaps the head of the next and short products fill the SMs a long one
 * leaves idle.  The natural use is llmt's Linear::backward (src/layers/linear.cpp:22-30),
 * whose two kernels::matmul calls (dx = dy W and dW += dy^T x) depend on nothing but dy:
 * pass both descriptors here.  count <= 8; every problem must be a bf16 problem and no
 * problem may write memory (C, dbias, workspace) that another problem of the call reads or
 * writes (checked by address range).  A launch runs on CTA pairs or on single CTAs as a
 * whole: plan_cta_pairs = 2 on one problem is refused when another cannot pair.  Each problem's
 * desc carries its own workspace; llmt_b200_gemm_grouped_workspace_bytes gives the sizes
 * (the split-K choice depends on the work the problems share the launch with).
 * Results are bitwise those of the same plan run alone: which SM computes a tile changes
 * nothing in the tile's arithmetic. */
LLMT_B200_API int llmt_b200_gemm_grouped(const llmt_b200_gemm_desc* descs, void* const* c,
                                         const void* const* a, const void* const* b, int32_t count,
                                         void* stream);
LLMT_B200_API int llmt_b200_gemm_grouped_workspace_bytes(const llmt_b200_gemm_desc* descs, int32_t count,
                                                         uint64_t* bytes_per_problem);

/* Size of the scratch array compiled into the library for llmt_b200_gemm_static_scratch. */
#define LLMT_B200_STATIC_SCRATCH_BYTES (32u << 20)

/* Same computation and same results as llmt_b200_gemm, for hosts that are not able to
 * hand the library a workspace.  (No counterpart in llmt: llmt's Device always owns a
 * cudaMalloc'ed cuBLASLt workspace.)  Some callers cannot call cudaMalloc at the point
 * where they need a GEMM: a serving or training loop whose memory plan is frozen and in
 * which an allocation would stall every stream of the device, a plugin that is given
 * tensors but no allocator, a foreign-language host that binds only this one function.
 * Here the split-K scratch is a fixed LLMT_B200_STATIC_SCRATCH_BYTES array inside the
 * library image (every GPU that loads the library holds it until the process exits);
 * desc->workspace and desc->workspace_bytes are ignored.  The call allocates nothing —
 * no cudaMalloc, no cudaFree, no allocating library routine.
 *   - A problem whose split-K plan needs more than LLMT_B200_STATIC_SCRATCH_BYTES is
 *     refused with LLMT_B200_ERR_WORKSPACE before anything is launched (lower
 *     plan_splits, or use llmt_b200_gemm with your own workspace).
 *   - The first call on each device that needs scratch looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current) and remembers it.  Make that first
 *     call outside any stream capture.
 *   - All calls share the one array and it keeps whatever the previous call left there.
 *     Nothing in it has to start at zero: every partial sum that is read back has been
 *     written earlier in the same call.  Two calls that need scratch and may run on the GPU
 *     at the same time (different streams, or different host threads) race on it: keep
 *     such calls on one stream, or order them with events. */
LLMT_B200_API int llmt_b200_gemm_static_scratch(const llmt_b200_gemm_desc* desc, void* c, const void* a,
                                                const void* b, void* stream);

/* Bytes of workspace llmt_b200_gemm needs for this problem (may be 0).  Pure
 * function of the descriptor and of the device's SM count.  Assumes A and B start on
 * 16-byte boundaries; llmt_b200_gemm_workspace_bytes_for also takes their addresses and
 * counts the aligned copy an operand with an odd base address needs. */
LLMT_B200_API uint64_t llmt_b200_gemm_workspace_bytes(const llmt_b200_gemm_desc* desc);
LLMT_B200_API uint64_t llmt_b200_gemm_workspace_bytes_for(const llmt_b200_gemm_desc* desc, const void* a,
                                                          const void* b);

/* Writes a one-line description of the kernel plan chosen for `desc` (tile shape,
 * pipeline depth, split count, grid) into buf.  The plan is a pure function of
 * the problem, which is what makes results reproducible — the role llmt's
 * AlgoCache plays (include/llmt/kernels/algo_cache.h:18-42).  Returns a status. */
LLMT_B200_API int llmt_b200_gemm_plan(const llmt_b200_gemm_desc* desc, char* buf, size_t buf_bytes);

/* Row softmax helper with llmt's masking rule (src/kernels/softmax.cu:25-51):
 * x, y are [rows, tk] with row r belonging to query r % tq; under causal != 0
 * only columns <= r % tq take part and the others are written as exact zeros.
 * In place (y == x) allowed.  fp32 arithmetic; dtype is the storage type. */
LLMT_B200_API int llmt_b200_softmax_fwd(void* y, const void* x, int64_t rows, int64_t tq, int64_t tk,
                          int32_t dtype, int32_t causal, void* stream);

/* dS = P * (dP - rowsum(dP * P)) per row (llmt docs/TODO.md:227). */
LLMT_B200_API int llmt_b200_softmax_bwd(void* ds, const void* p, const void* dp, int64_t rows, int64_t tk,
                          int32_t dtype, void* stream);

/* Head split and merge as copies (llmt include/llmt/kernels/permute.h:21-46, kernels in
 * src/kernels/permute.cu:18-46):
 *   merge: y[b, t, h*hd + d] = x[b, h, t, d]                       x [B,H,T,hd] -> y [B,T,H*hd]
 *   split: q|k|v[b, h, t, d] = qkv[b, t, part*H*hd + h*hd + d]     qkv [B,T,3*H*hd] -> 3 x [B,H,T,hd]
 * Outputs must not alias inputs.  The GEMM entry points can read and write the per-head layout
 * in place through batch_inner / stride_*_outer, which makes these copies unnecessary on the
 * attention path; they exist for callers that want the re-shelved tensors themselves. */
LLMT_B200_API int llmt_b200_head_merge(void* y, const void* x, int64_t b, int64_t h, int64_t t, int64_t hd,
                                       int32_t dtype, void* stream);
LLMT_B200_API int llmt_b200_head_split(void* q, void* k, void* v, const void* qkv, int64_t b, int64_t h, int64_t t,
                                       int64_t hd, int32_t dtype, void* stream);

/* Device-side health word.  Kernels never spin without bound: a wait that runs
 * out records (code, detail) here and the kernel drains and returns.  This call
 * synchronises the device, copies the word back and clears it.  code == 0 means
 * healthy.  Returns LLMT_B200_ERR_DEVICE when a code was pending; the results of the
 * launches that were in flight are then void, and the library's tile queues are reset so
 * that later launches are unaffected. */
LLMT_B200_API int llmt_b200_device_status(int32_t* code, int32_t* detail);

/* How long a wait inside a kernel may last before it gives up, in nanoseconds: gemm_ns for
 * the GEMM kernels' barrier waits (default 2 s), exchange_ns for the gradient exchange's
 * waits on its peers (default 4 s); 0 leaves a value as it is.  Applies to launches made
 * after the call.  Meant for tests and for hosts with their own watchdog period. */
LLMT_B200_API int llmt_b200_set_wait_limit_ns(uint64_t gemm_ns, uint64_t exchange_ns);

/* Host-side cache of encoded TMA descriptors (the counterpart of llmt's AlgoCache,
 * include/llmt/kernels/algo_cache.h:18-42: what is expensive to resolve is resolved once per
 * problem and replayed): number of look-ups answered from the cache and number that had to
 * encode, on all threads, since the library was loaded. */
LLMT_B200_API void llmt_b200_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses);

/* Zeroes `count` floats of the flat gradient span: the zero_grad that llmt leaves to the optimizer
 * between steps (include/llmt/model/param_store.h:142-148; llmt would use its fill_value kernel,
 * src/kernels/fill.cu:13-31).  Same effect as a memset; launched with programmatic stream
 * serialization so that the next GEMM's set-up overlaps it. */
LLMT_B200_API int llmt_b200_zero_grads(float* span, int64_t count, void* stream);

/* SMs the persistent GEMM kernels may occupy from now on: 0 (the default) = every SM.
 * Planning and grid size follow it.  A data-parallel caller lowers it by the number of
 * CTAs its collective library runs (e.g. 148 - 8), so that the all-reduce of one layer's
 * gradients, enqueued on a second stream, finds free SMs while the next layer's GEMM
 * launch is resident.  Returns the previous value, or a negative value for sms < 0.
 * llmt has no counterpart (single GPU: docs/TODO.md:12-16). */
LLMT_B200_API int llmt_b200_set_sm_budget(int32_t sms);

/* ---- gradient exchange of the data-parallel path ------------------------------------------
 * Sum of a range of the flat fp32 gradient span over `world` ranks (one process per GPU),
 * in place, over NVLink peer memory: one kernel of `ctas` CTAs that pushes every foreign
 * shard to its owner, sums each shard once in rank order and copies the sum back to every
 * rank.  All ranks end with the same bits; reruns reproduce them.  llmt is single-GPU; the
 * span is the seam its ParamStore documents for this (include/llmt/model/param_store.h:131-135).
 *
 * The caller allocates three buffers on every rank and exchanges their addresses with
 * whatever peer-mapping mechanism it has (CUDA IPC, VMM handles, a symmetric-memory
 * allocator); [i] is rank i's buffer as THIS rank can address it, [rank] the local one:
 *   grad  : the fp32 span itself
 *   stage : world * slot_elems floats of scratch
 *   flags : LLMT_B200_COMM_FLAG_BYTES, zeroed once before the first call
 * and, private to the rank, `epoch`: LLMT_B200_COMM_EPOCH_BYTES, zeroed once.
 * offset and count are in floats, multiples of 4; ceil(count / 4 / world) * 4 <= slot_elems.
 * Every rank must make the same sequence of calls with the same ctas; one call at a time
 * per communicator (enqueue them on one stream).  A peer that never arrives ends the wait
 * after a few seconds with LLMT_B200_DEV_WAIT_PEER in the device status word, not a hang.
 * Run it beside the GEMM kernels by lowering their SM budget by `ctas`. */
#define LLMT_B200_COMM_MAX_RANKS 8
#define LLMT_B200_COMM_MAX_CTAS 128
#define LLMT_B200_COMM_FLAG_BYTES (2 * LLMT_B200_COMM_MAX_RANKS * LLMT_B200_COMM_MAX_CTAS * 4 + 256)
#define LLMT_B200_COMM_EPOCH_BYTES (LLMT_B200_COMM_MAX_CTAS * 4)
#define LLMT_B200_DEV_WAIT_PEER 6

typedef struct llmt_b200_comm_desc {
    int32_t rank, world;
    void* grad[LLMT_B200_COMM_MAX_RANKS];
    void* stage[LLMT_B200_COMM_MAX_RANKS];
    void* flags[LLMT_B200_COMM_MAX_RANKS];
    void* epoch;
    int64_t slot_elems;
    void* grad_mc;   /* the span through an NVSwitch multicast mapping that covers every rank's
                        copy, or NULL.  When set, the sum is formed inside the switch
                        (multimem.ld_reduce) and broadcast by it (multimem.st): each rank moves
                        1/world of the range instead of world-1 shards, `stage` is not touched,
                        and the order of the additions is the switch's, not rank order. */
} llmt_b200_comm_desc;

LLMT_B200_API int llmt_b200_grad_allreduce(const llmt_b200_comm_desc* comm, int64_t offset, int64_t count,
                             int32_t ctas, void* stream);

/* A grouped launch that also sums a range of the gradient span over the ranks ("rides along"):
 * llmt_b200_gemm_grouped plus, inside the same kernel, the all-reduce of floats
 * [offset, offset + count) of the span, done by the launch's epilogue warps through the NVSwitch
 * multicast mapping (comm->grad_mc, required: LLMT_B200_ERR_UNSUPPORTED without it) while the
 * tensor pipe runs the launch's tiles, so the transfer costs no launch, no SM and no exposed time.
 * No counterpart in llmt (it has no collective).
 *   - The range must have been completed by EARLIER work on this stream (e.g. the previous
 *     layer's backward launch); a launch that writes into it is refused.
 *   - Every rank makes the same call with the same offset, count and index.  `index`
 *     (0..15) numbers the ride-along exchanges of one step; llmt_b200_exchange_begin_step starts
 *     a step (it advances a counter on the device, so a captured step can be replayed).
 *   - The sums are in every rank's span once a later llmt_b200_grad_allreduce call on the same
 *     stream has returned on the device (any range: typically the last layer's slice, which no
 *     later launch can carry); until then other ranks may still be writing them.
 *   - Every cross-rank wait is bounded (llmt_b200_set_wait_limit_ns); a rank that never arrives
 *     ends the launch with LLMT_B200_DEV_WAIT_PEER in the status word. */
LLMT_B200_API int llmt_b200_gemm_grouped_exchange(const llmt_b200_gemm_desc* descs, void* const* c,
                                    const void* const* a, const void* const* b, int32_t count,
                                    const llmt_b200_comm_desc* comm, int64_t offset, int64_t count_floats,
                                    int32_t index, void* stream);
LLMT_B200_API int llmt_b200_exchange_begin_step(const llmt_b200_comm_desc* comm, void* stream);

/* ---- the consumer of the LM-head logits (llmt include/llmt/kernels/cross_entropy.h:36-37) ----
 *
 * llmt_b200_cross_entropy_fwd: llmt's cross_entropy_fwd on fp32 logits [rows, vocab] (row pitch
 * ld), int32 targets [rows], fp32 mask [rows]:
 *   row_nll[r] = mask[r] * (log sum_v exp(logits[r, v]) - logits[r, targets[r]]),
 *   loss[0]    = sum_r row_nll[r] / sum_r mask[r]     (fixed-order sums: same bits every run).
 *
 * llmt_b200_lm_head_ce_fwd: the same result straight from the LM-head product
 * logits = alpha * op(A) * op(B) (+ bias), without the [rows, vocab] tensor having to exist: the GEMM's
 * epilogue keeps, per row and per half tile, the maximum and the sum of exponentials of the columns it
 * produced and the target's logit, and a small kernel combines them.  `logits` may be NULL (nothing is
 * stored) or the tensor to store as llmt_b200_gemm would.  bf16 operands, one product (no batch), no
 * GELU, no dbias; desc.workspace must hold llmt_b200_lm_head_ce_workspace_bytes(desc, a, b) bytes.
 * No counterpart in llmt (its cross_entropy_fwd reads logits from memory). */
LLMT_B200_API int llmt_b200_cross_entropy_fwd(float* loss, float* row_nll, const float* logits, const int32_t* targets,
                                const float* mask, int64_t rows, int64_t vocab, int64_t ld, void* stream);
LLMT_B200_API uint64_t llmt_b200_lm_head_ce_workspace_bytes(const llmt_b200_gemm_desc* desc, const void* a, const void* b);
LLMT_B200_API int llmt_b200_lm_head_ce_fwd(const llmt_b200_gemm_desc* desc, void* logits, const void* a, const void* b,
                             const int32_t* targets, const float* mask, float* row_nll, float* loss, void* stream);

/* The backward pass of the same loss (llmt docs/TODO.md:216-217, planned there as cross_entropy_bwd:
 * dlogits = (softmax - onehot) * mask / sum(mask), written in place of the logits).
 *
 * llmt_b200_cross_entropy_bwd: that kernel on fp32 logits in memory; dlogits may be the logits tensor
 * itself (in place, one pitch) or a tensor that does not overlap it.  `dloss` scales the result
 * (the upstream gradient of the mean loss, 1 for a plain backward pass).
 *
 * llmt_b200_lm_head_ce_bwd: the same gradient without logits in memory: the LM-head product is made
 * again and leaves as (exp(logit - lse[row]) - [col == target[row]]) * dloss * mask[row] / sum(mask)
 * in desc.dtype_c (bf16: directly the operand of the LM head's dX and dW products), pitch desc.ldc.
 * Same desc (apart from dtype_c / ldc), operands and workspace size as llmt_b200_lm_head_ce_fwd.
 * stats_valid != 0: desc.workspace still holds what llmt_b200_lm_head_ce_fwd left there for this
 * product (nothing else has used it since), so the statistics pass is skipped; 0: it is run first.
 * No counterparts in llmt (planned, not written). */
LLMT_B200_API int llmt_b200_cross_entropy_bwd(float* dlogits, const float* logits, const int32_t* targets, const float* mask,
                                float dloss, int64_t rows, int64_t vocab, int64_t ld_in, int64_t ld_out, void* stream);
LLMT_B200_API int llmt_b200_lm_head_ce_bwd(const llmt_b200_gemm_desc* desc, void* dlogits, const void* a, const void* b,
                             const int32_t* targets, const float* mask, float dloss, int32_t stats_valid, void* stream);

/* ---- the softmax of an attention layer fused around its GEMMs --------------------------------
 * (llmt src/kernels/attention.cpp:60-62: scores = alpha q k^T, softmax in place, y = probs v;
 *  src/kernels/softmax.cu:25-51: the masking rule; docs/TODO.md:226-228: the backward products.)
 *
 * llmt_b200_gemm_softmax_fwd: probs = softmax over each row of S = alpha * op(A) * op(B) (every item of
 * a batch by itself), under llmt's causal rule when `causal` != 0 (row q sees columns 0..q; the others
 * are stored as exact zeros), WITHOUT S ever being stored: the GEMM kernel runs twice over the same
 * tiles.  The first launch stores nothing; its epilogue leaves, per row and per half tile, the maximum
 * and the sum of exponentials; a small kernel turns them into the rows' log-sum-exp; the second launch
 * makes the same tiles again (same plan, same bits) and stores exp(S - lse[row]) in C's type.  What
 * llmt writes and reads three times (scores out, scores in, probs out) is written once.  The
 * arithmetic is fp32 on the fp32 accumulators (llmt rounds the scores to the tensor's type first).
 *   lse: fp32 [batch * m], optional; receives the rows' log-sum-exp.
 * bf16 operands; beta 0; no bias, GELU, dbias; desc.workspace must hold
 * llmt_b200_gemm_softmax_workspace_bytes(desc, a, b) bytes.
 *
 * llmt_b200_gemm_softmax_bwd: dS = probs ⊙ (alpha * op(A) * op(B) - row_dot[row]) as the epilogue of
 * the product that makes dP = dO v^T: dP itself is never stored.  `probs` has C's type, pitch and
 * batch strides and must not overlap dS; row_dot is fp32 [batch * m] and holds
 * sum_j dP[r, j] * probs[r, j], which equals sum_d dO[r, d] * O[r, d] for O = probs v
 * (llmt_b200_rowdot on dO and O computes it).  Workspace as llmt_b200_gemm.
 *
 * llmt_b200_rowdot: out[r] = sum_j x[r, j] * y[r, j] in fp32 over [rows, cols] tensors with row
 * pitches ldx, ldy (elements).
 * No counterparts in llmt (its softmax is a kernel of its own between the GEMMs; it has no attention
 * backward). */
LLMT_B200_API uint64_t llmt_b200_gemm_softmax_workspace_bytes(const llmt_b200_gemm_desc* desc, const void* a, const void* b);
LLMT_B200_API int llmt_b200_gemm_softmax_fwd(const llmt_b200_gemm_desc* desc, void* probs, const void* a, const void* b,
                               int32_t causal, float* lse, void* stream);
LLMT_B200_API int llmt_b200_gemm_softmax_bwd(const llmt_b200_gemm_desc* desc, void* ds, const void* a, const void* b,
                               const void* probs, const float* row_dot, int32_t causal, void* stream);
LLMT_B200_API int llmt_b200_rowdot(float* out, const void* x, const void* y, int64_t rows, int64_t cols, int64_t ldx,
                     int64_t ldy, int32_t dtype, void* stream);

/* The same exchange with all `world` ranks living on ONE device (comms[r] is rank r's
 * descriptor, every pointer local): a single cooperative launch of world * ctas CTAs.
 * For tests of the algorithm where fewer GPUs than ranks are at hand. */
LLMT_B200_API int llmt_b200_grad_allreduce_emulated(const llmt_b200_comm_desc* comms, int32_t world, int64_t offset,
                                      int64_t count, int32_t ctas, void* stream);

/* Number of kernels this library has launched from this process so far. */
LLMT_B200_API uint64_t llmt_b200_launch_count(void);

/* Message for the most recent non-zero status on this thread ("" if none). */
LLMT_B200_API const char* llmt_b200_last_error(void);

LLMT_B200_API int llmt_b200_abi_version(void);

#ifdef __cplusplus
}
#endif

#endif /* LLMT_B200_H */
