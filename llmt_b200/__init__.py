"""llmt_b200 — Python binding of the C ABI in include/llmt_b200.h.

The product is the shared library llmt_b200/lib/libllmt_b200.so (hand-written
sm_100a kernels behind `extern "C"` entry points). This module only loads it
with ctypes and passes device pointers of torch tensors through; torch is used
for device memory and streams, never for arithmetic. There is no fallback: if
the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# LLMT_B200_LIB selects another build of the same library (e.g. an instrumented one).
LIB_PATH = os.environ.get("LLMT_B200_LIB") or os.path.join(_HERE, "lib", "libllmt_b200.so")

FP32, BF16 = 0, 1
EPI_NONE, EPI_BIAS, EPI_GELU, EPI_GELU_BWD, EPI_SAVE_PRE = 0, 1, 2, 4, 8
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE = 0, 1, 2, 3, 4, 5

EXPORTS = [
    "llmt_b200_gemm", "llmt_b200_gemm_grouped", "llmt_b200_gemm_grouped_workspace_bytes",
    "llmt_b200_gemm_static_scratch", "llmt_b200_gemm_workspace_bytes", "llmt_b200_gemm_plan",
    "llmt_b200_softmax_fwd", "llmt_b200_softmax_bwd", "llmt_b200_device_status",
    "llmt_b200_launch_count", "llmt_b200_last_error", "llmt_b200_abi_version",
    "llmt_b200_set_sm_budget", "llmt_b200_grad_allreduce", "llmt_b200_grad_allreduce_emulated",
    "llmt_b200_zero_grads", "llmt_b200_gemm_workspace_bytes_for", "llmt_b200_set_wait_limit_ns",
    "llmt_b200_tensor_map_cache_stats", "llmt_b200_head_merge", "llmt_b200_head_split",
    "llmt_b200_gemm_grouped_exchange", "llmt_b200_exchange_begin_step",
    "llmt_b200_cross_entropy_fwd", "llmt_b200_lm_head_ce_workspace_bytes", "llmt_b200_lm_head_ce_fwd",
    "llmt_b200_gemm_softmax_workspace_bytes", "llmt_b200_gemm_softmax_fwd", "llmt_b200_gemm_softmax_bwd",
    "llmt_b200_rowdot", "llmt_b200_cross_entropy_bwd", "llmt_b200_lm_head_ce_bwd",
]

COMM_MAX_RANKS, COMM_MAX_CTAS = 8, 128
COMM_FLAG_BYTES = 2 * COMM_MAX_RANKS * COMM_MAX_CTAS * 4 + 256
MAX_RIDES_PER_STEP = 16
COMM_EPOCH_BYTES = COMM_MAX_CTAS * 4
DEV_WAIT_PEER = 6


class CommDesc(ctypes.Structure):
    """llmt_b200_comm_desc of include/llmt_b200.h."""
    _fields_ = [("rank", ctypes.c_int32), ("world", ctypes.c_int32),
                ("grad", ctypes.c_void_p * COMM_MAX_RANKS), ("stage", ctypes.c_void_p * COMM_MAX_RANKS),
                ("flags", ctypes.c_void_p * COMM_MAX_RANKS), ("epoch", ctypes.c_void_p),
                ("slot_elems", ctypes.c_int64), ("grad_mc", ctypes.c_void_p)]


class GemmDesc(ctypes.Structure):
    """struct llmt_b200_gemm_desc (include/llmt_b200.h)."""
    _fields_ = [
        ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64), ("batch", ctypes.c_int64),
        ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
        ("stride_a", ctypes.c_int64), ("stride_b", ctypes.c_int64), ("stride_c", ctypes.c_int64),
        ("trans_a", ctypes.c_int32), ("trans_b", ctypes.c_int32),
        ("dtype_ab", ctypes.c_int32), ("dtype_c", ctypes.c_int32),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
        ("epilogue", ctypes.c_int32), ("bias_dtype", ctypes.c_int32),
        ("bias", ctypes.c_void_p), ("dbias", ctypes.c_void_p),
        ("dbias_beta", ctypes.c_float), ("plan_tile_n", ctypes.c_int32),
        ("plan_splits", ctypes.c_int32), ("plan_cta_pairs", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_uint64),
        ("batch_inner", ctypes.c_int64), ("stride_a_outer", ctypes.c_int64),
        ("stride_b_outer", ctypes.c_int64), ("stride_c_outer", ctypes.c_int64),
        ("aux", ctypes.c_void_p),
    ]


class LlmtB200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"llmt_b200 status {status}: {message}")
        self.status = status


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the C-ABI library. Raises if it has not been built — there is no
    other implementation to fall back to."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LlmtB200Error(-1, f"{LIB_PATH} is missing; run `python -m llmt_b200.build`")
        L = ctypes.CDLL(LIB_PATH)
        L.llmt_b200_gemm.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_void_p]
        L.llmt_b200_gemm.restype = ctypes.c_int
        L.llmt_b200_gemm_grouped.argtypes = [ctypes.POINTER(GemmDesc), ctypes.POINTER(ctypes.c_void_p),
                                             ctypes.POINTER(ctypes.c_void_p),
                                             ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32,
                                             ctypes.c_void_p]
        L.llmt_b200_gemm_grouped.restype = ctypes.c_int
        L.llmt_b200_gemm_grouped_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_int32,
                                                             ctypes.POINTER(ctypes.c_uint64)]
        L.llmt_b200_gemm_grouped_workspace_bytes.restype = ctypes.c_int
        L.llmt_b200_gemm_static_scratch.argtypes = L.llmt_b200_gemm.argtypes
        L.llmt_b200_gemm_static_scratch.restype = ctypes.c_int
        L.llmt_b200_gemm_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc)]
        L.llmt_b200_gemm_workspace_bytes.restype = ctypes.c_uint64
        L.llmt_b200_gemm_workspace_bytes_for.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_void_p, ctypes.c_void_p]
        L.llmt_b200_gemm_workspace_bytes_for.restype = ctypes.c_uint64
        L.llmt_b200_set_wait_limit_ns.argtypes = [ctypes.c_uint64, ctypes.c_uint64]
        L.llmt_b200_set_wait_limit_ns.restype = ctypes.c_int
        L.llmt_b200_tensor_map_cache_stats.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]
        L.llmt_b200_tensor_map_cache_stats.restype = None
        L.llmt_b200_head_merge.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                           ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_head_merge.restype = ctypes.c_int
        L.llmt_b200_head_split.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                           ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                           ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_head_split.restype = ctypes.c_int
        L.llmt_b200_gemm_plan.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_char_p, ctypes.c_size_t]
        L.llmt_b200_gemm_plan.restype = ctypes.c_int
        L.llmt_b200_softmax_fwd.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                            ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_softmax_fwd.restype = ctypes.c_int
        L.llmt_b200_softmax_bwd.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                            ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                            ctypes.c_void_p]
        L.llmt_b200_softmax_bwd.restype = ctypes.c_int
        L.llmt_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_int32),
                                              ctypes.POINTER(ctypes.c_int32)]
        L.llmt_b200_device_status.restype = ctypes.c_int
        L.llmt_b200_launch_count.restype = ctypes.c_uint64
        L.llmt_b200_grad_allreduce.argtypes = [ctypes.POINTER(CommDesc), ctypes.c_int64, ctypes.c_int64,
                                               ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_grad_allreduce.restype = ctypes.c_int
        L.llmt_b200_grad_allreduce_emulated.argtypes = [ctypes.POINTER(CommDesc), ctypes.c_int32, ctypes.c_int64,
                                                        ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_grad_allreduce_emulated.restype = ctypes.c_int
        L.llmt_b200_gemm_grouped_exchange.argtypes = [ctypes.POINTER(GemmDesc), ctypes.POINTER(ctypes.c_void_p),
                                                      ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                                      ctypes.c_int32, ctypes.POINTER(CommDesc), ctypes.c_int64,
                                                      ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_gemm_grouped_exchange.restype = ctypes.c_int
        L.llmt_b200_cross_entropy_fwd.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int64] * 3 + [ctypes.c_void_p]
        L.llmt_b200_cross_entropy_fwd.restype = ctypes.c_int
        L.llmt_b200_lm_head_ce_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_void_p, ctypes.c_void_p]
        L.llmt_b200_lm_head_ce_workspace_bytes.restype = ctypes.c_uint64
        L.llmt_b200_lm_head_ce_fwd.argtypes = [ctypes.POINTER(GemmDesc)] + [ctypes.c_void_p] * 8
        L.llmt_b200_lm_head_ce_fwd.restype = ctypes.c_int
        L.llmt_b200_cross_entropy_bwd.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_float] + [ctypes.c_int64] * 4 + [ctypes.c_void_p]
        L.llmt_b200_cross_entropy_bwd.restype = ctypes.c_int
        L.llmt_b200_lm_head_ce_bwd.argtypes = [ctypes.POINTER(GemmDesc)] + [ctypes.c_void_p] * 5 + [ctypes.c_float, ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_lm_head_ce_bwd.restype = ctypes.c_int
        L.llmt_b200_gemm_softmax_workspace_bytes.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_void_p, ctypes.c_void_p]
        L.llmt_b200_gemm_softmax_workspace_bytes.restype = ctypes.c_uint64
        L.llmt_b200_gemm_softmax_fwd.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                 ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
        L.llmt_b200_gemm_softmax_fwd.restype = ctypes.c_int
        L.llmt_b200_gemm_softmax_bwd.argtypes = [ctypes.POINTER(GemmDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_gemm_softmax_bwd.restype = ctypes.c_int
        L.llmt_b200_rowdot.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int64] * 4 + [ctypes.c_int32, ctypes.c_void_p]
        L.llmt_b200_rowdot.restype = ctypes.c_int
        L.llmt_b200_exchange_begin_step.argtypes = [ctypes.POINTER(CommDesc), ctypes.c_void_p]
        L.llmt_b200_exchange_begin_step.restype = ctypes.c_int
        L.llmt_b200_zero_grads.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        L.llmt_b200_zero_grads.restype = ctypes.c_int
        L.llmt_b200_set_sm_budget.argtypes = [ctypes.c_int32]
        L.llmt_b200_set_sm_budget.restype = ctypes.c_int
        L.llmt_b200_last_error.restype = ctypes.c_char_p
        L.llmt_b200_abi_version.restype = ctypes.c_int
        _lib = L
    return _lib


def last_error() -> str:
    return lib().llmt_b200_last_error().decode()


def _check(status: int) -> None:
    if status != OK:
        raise LlmtB200Error(status, last_error())


def _stream(stream):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def _dtype_code(t) -> int:
    import torch
    if t.dtype == torch.float32:
        return FP32
    if t.dtype == torch.bfloat16:
        return BF16
    raise LlmtB200Error(ERR_UNSUPPORTED, f"dtype {t.dtype} not supported")


def _row_pitch(t) -> int:
    if t.stride(-1) != 1 and t.shape[-1] != 1:
        raise LlmtB200Error(ERR_INVALID, "innermost dimension must be contiguous")
    return t.stride(-2)


def make_desc(c, a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, bias=None, gelu=False,
              dbias=None, dbias_beta=0.0, workspace=None, tile_n=0, splits=0, cta_pairs=0, gelu_bwd_of=None,
              save_pre=None) -> GemmDesc:
    """Builds the descriptor for C = epilogue(alpha*op(A)*op(B) + beta*C) from rank-2
    or rank-3 torch tensors (row-major views with a contiguous last dimension)."""
    if not (a.dim() == b.dim() == c.dim()) or a.dim() not in (2, 3):
        raise LlmtB200Error(ERR_INVALID, "matmul: expected rank-2 or rank-3 tensors of one rank")
    d = GemmDesc()
    ar, ac = a.shape[-2], a.shape[-1]
    br, bc = b.shape[-2], b.shape[-1]
    d.m, d.k = (ac, ar) if trans_a else (ar, ac)
    kb, d.n = (bc, br) if trans_b else (br, bc)
    if kb != d.k:
        raise LlmtB200Error(ERR_INVALID, f"matmul: inner dims disagree: {d.k} vs {kb}")
    if tuple(c.shape[-2:]) != (d.m, d.n):
        raise LlmtB200Error(ERR_INVALID, "matmul: C shape mismatch")
    if a.dim() == 3:
        d.batch = a.shape[0]
        if b.shape[0] != d.batch or c.shape[0] != d.batch:
            raise LlmtB200Error(ERR_INVALID, "matmul: batch sizes disagree")
        d.stride_a, d.stride_b, d.stride_c = a.stride(0), b.stride(0), c.stride(0)
    else:
        d.batch = 1
    d.lda, d.ldb, d.ldc = _row_pitch(a), _row_pitch(b), _row_pitch(c)
    d.trans_a, d.trans_b = int(trans_a), int(trans_b)
    if a.dtype != b.dtype:
        raise LlmtB200Error(ERR_INVALID, "matmul: mixed dtypes in one matmul")
    d.dtype_ab, d.dtype_c = _dtype_code(a), _dtype_code(c)
    d.alpha, d.beta = float(alpha), float(beta)
    d.epilogue = (EPI_BIAS if bias is not None else 0) | (EPI_GELU if gelu else 0)
    if bias is not None:
        d.bias = bias.data_ptr()
        d.bias_dtype = _dtype_code(bias)
    if dbias is not None:
        d.dbias = dbias.data_ptr()
        d.dbias_beta = float(dbias_beta)
    d.plan_tile_n, d.plan_splits, d.plan_cta_pairs = int(tile_n), int(splits), int(cta_pairs)
    if gelu_bwd_of is not None:
        # C = (alpha * op(A) * op(B)) * gelu'(pre): `gelu_bwd_of` is the saved pre-activation, laid out like C
        if gelu_bwd_of.shape != c.shape or gelu_bwd_of.dtype != c.dtype or gelu_bwd_of.stride() != c.stride():
            raise LlmtB200Error(ERR_INVALID, "matmul: the pre-activation must have C's shape, type and strides")
        d.epilogue |= EPI_GELU_BWD
        d.aux = gelu_bwd_of.data_ptr()
    if save_pre is not None:
        # with gelu=True: the value the GELU sees is stored in `save_pre` (laid out like C) as well
        if save_pre.shape != c.shape or save_pre.dtype != c.dtype or save_pre.stride() != c.stride():
            raise LlmtB200Error(ERR_INVALID, "matmul: the pre-activation must have C's shape, type and strides")
        d.epilogue |= EPI_SAVE_PRE
        d.aux = save_pre.data_ptr()
    if workspace is not None:
        d.workspace = workspace.data_ptr()
        d.workspace_bytes = workspace.numel() * workspace.element_size()
    return d


def workspace_bytes(desc: GemmDesc, a=None, b=None) -> int:
    """Scratch the problem needs; pass the operand tensors when their base address may be odd."""
    if a is None or b is None:
        return int(lib().llmt_b200_gemm_workspace_bytes(ctypes.byref(desc)))
    return int(lib().llmt_b200_gemm_workspace_bytes_for(ctypes.byref(desc), a.data_ptr(), b.data_ptr()))


def set_wait_limit_ns(gemm_ns: int = 0, exchange_ns: int = 0) -> None:
    """Bound of the waits inside the kernels (0 = leave unchanged)."""
    _check(lib().llmt_b200_set_wait_limit_ns(int(gemm_ns), int(exchange_ns)))


def tensor_map_cache_stats():
    """(hits, misses) of the host-side cache of encoded TMA descriptors."""
    h, m = ctypes.c_uint64(0), ctypes.c_uint64(0)
    lib().llmt_b200_tensor_map_cache_stats(ctypes.byref(h), ctypes.byref(m))
    return int(h.value), int(m.value)


def plan(desc: GemmDesc) -> str:
    buf = ctypes.create_string_buffer(256)
    _check(lib().llmt_b200_gemm_plan(ctypes.byref(desc), buf, 256))
    return buf.value.decode()


def gemm_desc(desc: GemmDesc, c, a, b, stream=None) -> None:
    """Enqueues one llmt_b200_gemm call; `stream` is a torch.cuda.Stream (default: current)."""
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    _check(lib().llmt_b200_gemm(ctypes.byref(desc), c.data_ptr(), a.data_ptr(), b.data_ptr(),
                                ctypes.c_void_p(s.cuda_stream)))


class Group:
    """A fixed list of independent bf16 problems launched as one kernel
    (llmt_b200_gemm_grouped). Built once from (desc, c, a, b) tuples; run() enqueues it."""

    def __init__(self, problems):
        n = len(problems)
        self.n = n
        self.descs = (GemmDesc * n)(*[p[0] for p in problems])
        self.tensors = [p[1:] for p in problems]  # keep the tensors alive
        self.c = (ctypes.c_void_p * n)(*[p[1].data_ptr() for p in problems])
        self.a = (ctypes.c_void_p * n)(*[p[2].data_ptr() for p in problems])
        self.b = (ctypes.c_void_p * n)(*[p[3].data_ptr() for p in problems])

    def workspace_bytes(self):
        out = (ctypes.c_uint64 * self.n)()
        _check(lib().llmt_b200_gemm_grouped_workspace_bytes(self.descs, self.n, out))
        return [int(v) for v in out]

    def set_workspaces(self, buffers):
        """buffers: one torch uint8 tensor (or None) per problem."""
        self._ws = buffers
        for d, buf in zip(self.descs, buffers):
            if buf is not None:
                d.workspace, d.workspace_bytes = buf.data_ptr(), buf.numel()

    def run(self, stream=None):
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        _check(lib().llmt_b200_gemm_grouped(self.descs, self.c, self.a, self.b, self.n,
                                            ctypes.c_void_p(s.cuda_stream)))

    def run_with_exchange(self, comm: "CommDesc", offset: int, count: int, index: int, stream=None):
        """llmt_b200_gemm_grouped_exchange: the same launch, whose epilogue warps also sum floats
        [offset, offset + count) of the gradient span over the ranks through the NVSwitch
        multicast mapping.  The range must be complete before the launch starts."""
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        _check(lib().llmt_b200_gemm_grouped_exchange(self.descs, self.c, self.a, self.b, self.n, ctypes.byref(comm),
                                                     ctypes.c_int64(int(offset)), ctypes.c_int64(int(count)),
                                                     ctypes.c_int32(int(index)), ctypes.c_void_p(s.cuda_stream)))


STATIC_SCRATCH_BYTES = 32 << 20


def gemm_static_scratch(desc: GemmDesc, c, a, b, stream=None) -> None:
    """llmt_b200_gemm_static_scratch: same result as gemm_desc, but split-K partial sums go to
    the fixed array built into the library, so the call allocates nothing and needs no
    workspace from the caller. Problems needing more than STATIC_SCRATCH_BYTES are refused.
    Calls that may overlap on the GPU share (and race on) that one array."""
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    _check(lib().llmt_b200_gemm_static_scratch(ctypes.byref(desc), c.data_ptr(), a.data_ptr(),
                                               b.data_ptr(), ctypes.c_void_p(s.cuda_stream)))


def gemm(c, a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, bias=None, gelu=False,
         dbias=None, dbias_beta=0.0, workspace=None, stream=None, tile_n=0, splits=0, cta_pairs=0) -> None:
    """C = epilogue(alpha*op(A)*op(B) + beta*C) on device tensors, in place in C.

    Same argument meaning as llmt's kernels::matmul
    (include/llmt/kernels/matmul.h:12-24) plus the fused bias / GELU / dbias
    extensions. If the problem needs split-K scratch and none is passed, a
    torch buffer is allocated for this call."""
    import torch
    d = make_desc(c, a, b, trans_a, trans_b, alpha, beta, bias, gelu, dbias, dbias_beta, workspace,
                  tile_n, splits, cta_pairs)
    if workspace is None:
        need = workspace_bytes(d, a, b)
        if need:
            ws = torch.empty(need, dtype=torch.uint8, device=c.device)
            d.workspace = ws.data_ptr()
            d.workspace_bytes = need
    gemm_desc(d, c, a, b, stream)


def softmax_fwd(y, x, causal: bool, stream=None) -> None:
    """Row softmax of [batch, Tq, Tk] with llmt's causal rule; y may be x."""
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    tq, tk = x.shape[-2], x.shape[-1]
    _check(lib().llmt_b200_softmax_fwd(y.data_ptr(), x.data_ptr(), x.numel() // tk, tq, tk,
                                       _dtype_code(x), int(causal), ctypes.c_void_p(s.cuda_stream)))


def softmax_bwd(ds, p, dp, stream=None) -> None:
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    tk = p.shape[-1]
    _check(lib().llmt_b200_softmax_bwd(ds.data_ptr(), p.data_ptr(), dp.data_ptr(), p.numel() // tk, tk,
                                       _dtype_code(p), ctypes.c_void_p(s.cuda_stream)))


def head_merge(y, x, stream=None) -> None:
    """y[b, t, h*hd + d] = x[b, h, t, d] (llmt permute_merge): x [B,H,T,hd] -> y [B,T,H*hd]."""
    b, h, t, hd = x.shape
    _check(lib().llmt_b200_head_merge(y.data_ptr(), x.data_ptr(), b, h, t, hd, _dtype_code(x), _stream(stream)))


def head_split(q, k, v, qkv, stream=None) -> None:
    """q|k|v[b, h, t, d] = qkv[b, t, part*A + h*hd + d] (llmt permute_split): qkv [B,T,3A] -> 3 x [B,H,T,hd]."""
    b, h, t, hd = q.shape
    _check(lib().llmt_b200_head_split(q.data_ptr(), k.data_ptr(), v.data_ptr(), qkv.data_ptr(), b, h, t, hd,
                                      _dtype_code(qkv), _stream(stream)))


def device_status():
    """Synchronises and returns (code, detail) of the device health word; raises if non-zero."""
    code, detail = ctypes.c_int32(0), ctypes.c_int32(0)
    st = lib().llmt_b200_device_status(ctypes.byref(code), ctypes.byref(detail))
    if st != OK:
        raise LlmtB200Error(st, last_error())
    return code.value, detail.value


def grad_allreduce(desc: "CommDesc", offset: int, count: int, ctas: int = 8, stream=None) -> None:
    """Sums floats [offset, offset + count) of the span over the ranks of `desc`, in place."""
    _check(lib().llmt_b200_grad_allreduce(ctypes.byref(desc), int(offset), int(count), int(ctas), _stream(stream)))


def cross_entropy_fwd(loss, row_nll, logits, targets, mask, stream=None) -> None:
    """llmt's cross_entropy_fwd (include/llmt/kernels/cross_entropy.h:36-37) on fp32 logits [..., V]:
    row_nll = mask * (lse - logit of the target), loss = sum(row_nll) / sum(mask)."""
    import torch
    v = logits.shape[-1]
    rows = logits.numel() // v
    if logits.dtype != torch.float32 or targets.dtype != torch.int32 or mask.dtype != torch.float32:
        raise LlmtB200Error(ERR_INVALID, "cross_entropy_fwd: fp32 logits and mask, int32 targets")
    _check(lib().llmt_b200_cross_entropy_fwd(loss.data_ptr(), row_nll.data_ptr(), logits.data_ptr(), targets.data_ptr(),
                                             mask.data_ptr(), rows, v, logits.stride(-2) if logits.dim() > 1 else v,
                                             _stream(stream)))


def lm_head_ce_workspace_bytes(desc: GemmDesc, a=None, b=None) -> int:
    return int(lib().llmt_b200_lm_head_ce_workspace_bytes(ctypes.byref(desc), a.data_ptr() if a is not None else None,
                                                          b.data_ptr() if b is not None else None))


def lm_head_ce_fwd(desc: GemmDesc, logits, a, b, targets, mask, row_nll, loss, stream=None) -> None:
    """The LM-head product and its cross-entropy in one pass (llmt_b200_lm_head_ce_fwd); `logits`
    may be None: then the [rows, vocab] tensor is never written."""
    _check(lib().llmt_b200_lm_head_ce_fwd(ctypes.byref(desc), logits.data_ptr() if logits is not None else None,
                                          a.data_ptr(), b.data_ptr(), targets.data_ptr(), mask.data_ptr(),
                                          row_nll.data_ptr(), loss.data_ptr(), _stream(stream)))


def cross_entropy_bwd(dlogits, logits, targets, mask, dloss: float = 1.0, stream=None) -> None:
    """dlogits = (softmax(logits) - onehot(targets)) * dloss * mask / sum(mask) on fp32 logits [..., V];
    dlogits may be `logits` itself (in place)."""
    v = logits.shape[-1]
    rows = logits.numel() // v
    if _dtype_code(logits) != FP32 or _dtype_code(dlogits) != FP32 or dlogits.shape != logits.shape:
        raise LlmtB200Error(ERR_INVALID, "cross_entropy_bwd: fp32 logits and dlogits of one shape")
    _check(lib().llmt_b200_cross_entropy_bwd(dlogits.data_ptr(), logits.data_ptr(), targets.data_ptr(), mask.data_ptr(),
                                             float(dloss), rows, v, logits.stride(-2) if logits.dim() > 1 else v,
                                             dlogits.stride(-2) if dlogits.dim() > 1 else v, _stream(stream)))


def lm_head_ce_bwd(desc: GemmDesc, dlogits, a, b, targets, mask, dloss: float = 1.0, stats_valid: bool = False,
                   stream=None) -> None:
    """dLogits of the LM head's cross-entropy from the product itself (llmt_b200_lm_head_ce_bwd)."""
    _check(lib().llmt_b200_lm_head_ce_bwd(ctypes.byref(desc), dlogits.data_ptr(), a.data_ptr(), b.data_ptr(),
                                          targets.data_ptr(), mask.data_ptr(), float(dloss), 1 if stats_valid else 0,
                                          _stream(stream)))


def gemm_softmax_workspace_bytes(desc: GemmDesc, a=None, b=None) -> int:
    return int(lib().llmt_b200_gemm_softmax_workspace_bytes(ctypes.byref(desc), a.data_ptr() if a is not None else None,
                                                            b.data_ptr() if b is not None else None))


def gemm_softmax_fwd(desc: GemmDesc, probs, a, b, causal: bool, lse=None, stream=None) -> None:
    """probs = row softmax of alpha * op(a) * op(b), the scores never stored (llmt_b200_gemm_softmax_fwd)."""
    _check(lib().llmt_b200_gemm_softmax_fwd(ctypes.byref(desc), probs.data_ptr(), a.data_ptr(), b.data_ptr(),
                                            1 if causal else 0, lse.data_ptr() if lse is not None else None,
                                            _stream(stream)))


def gemm_softmax_bwd(desc: GemmDesc, ds, a, b, probs, row_dot, causal: bool, stream=None) -> None:
    """ds = probs * (alpha * op(a) * op(b) - row_dot[row]), dP never stored (llmt_b200_gemm_softmax_bwd)."""
    _check(lib().llmt_b200_gemm_softmax_bwd(ctypes.byref(desc), ds.data_ptr(), a.data_ptr(), b.data_ptr(),
                                            probs.data_ptr(), row_dot.data_ptr(), 1 if causal else 0, _stream(stream)))


def rowdot(out, x, y, stream=None) -> None:
    """out[r] = sum_j x[r, j] * y[r, j] (fp32) over the last dimension of two same-shaped tensors."""
    cols = x.shape[-1]
    rows = x.numel() // cols
    if x.shape != y.shape or x.dtype != y.dtype or _dtype_code(out) != FP32 or out.numel() != rows:
        raise LlmtB200Error(ERR_INVALID, "rowdot: x and y of one shape and type, out fp32 with one value per row")
    if not (x.is_contiguous() and y.is_contiguous()):
        raise LlmtB200Error(ERR_INVALID, "rowdot: contiguous tensors")
    _check(lib().llmt_b200_rowdot(out.data_ptr(), x.data_ptr(), y.data_ptr(), rows, cols, cols, cols,
                                  _dtype_code(x), _stream(stream)))


def exchange_begin_step(desc: "CommDesc", stream=None) -> None:
    """Starts a step of ride-along exchanges (Group.run_with_exchange) on this rank's stream."""
    _check(lib().llmt_b200_exchange_begin_step(ctypes.byref(desc), _stream(stream)))


def grad_allreduce_emulated(descs, offset: int, count: int, ctas: int = 4, stream=None) -> None:
    """All ranks of the exchange on one device, one cooperative launch (tests)."""
    arr = (CommDesc * len(descs))(*descs)
    _check(lib().llmt_b200_grad_allreduce_emulated(arr, len(descs), int(offset), int(count), int(ctas),
                                                   _stream(stream)))


def zero_grads(span, stream=None) -> None:
    """Zeroes a contiguous fp32 tensor (the flat gradient span) on its device."""
    import torch
    if span.dtype != torch.float32 or not span.is_contiguous():
        raise LlmtB200Error(ERR_INVALID, "zero_grads: contiguous fp32 tensor expected")
    _check(lib().llmt_b200_zero_grads(span.data_ptr(), span.numel(), _stream(stream)))


def set_sm_budget(sms: int) -> int:
    """SMs the persistent GEMM kernels may occupy (0 = all); returns the previous value."""
    return int(lib().llmt_b200_set_sm_budget(int(sms)))


def launch_count() -> int:
    return int(lib().llmt_b200_launch_count())
