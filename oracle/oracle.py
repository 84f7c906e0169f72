"""ctypes front end of oracle.c (fp64 CPU restatement of llmt's matmul path).

TEST INFRASTRUCTURE, NOT PRODUCT. Only tests/, the smoke check and the
benchmark's CPU-baseline leg import this module.

Every function takes/returns numpy arrays. bf16 tensors are represented as
float32 arrays whose values are exactly bf16-representable (see round_bf16).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i64 = ctypes.c_int64


def build(force: bool = False) -> str:
    """Compile oracle.c with the Makefile next to it (gcc + OpenMP)."""
    src = os.path.join(_HERE, "oracle.c")
    if (force or not os.path.exists(_LIB_PATH)
            or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)):
        subprocess.check_call(["make", "-s", "-C", _HERE])
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.oracle_num_threads.restype = ctypes.c_int
        L.oracle_gemm_f64.argtypes = [_i64, _i64, _i64, _i64,
                                      _f32p, _i64, _i64, ctypes.c_int,
                                      _f32p, _i64, _i64, ctypes.c_int,
                                      _f64p, _i64, _i64, ctypes.c_double, ctypes.c_double]
        L.oracle_gemm_f32.argtypes = [_i64, _i64, _i64,
                                      _f32p, _i64, ctypes.c_int,
                                      _f32p, _i64, ctypes.c_int,
                                      _f32p, _i64, ctypes.c_float, ctypes.c_float]
        L.oracle_epilogue_f64.argtypes = [_f64p, _i64, _i64, _i64, _f32p, ctypes.c_int]
        L.oracle_rowsum_f64.argtypes = [_i64, _i64, _f32p, _i64, ctypes.c_int, _f64p,
                                        ctypes.c_double]
        L.oracle_softmax_f64.argtypes = [_f64p, _f64p, _i64, _i64, _i64, ctypes.c_int]
        L.oracle_softmax_bwd_f64.argtypes = [_f64p, _f64p, _f64p, _i64, _i64]
        L.oracle_round_bf16.argtypes = [_f32p, _f32p, _i64]
        L.oracle_gelu_f64.argtypes = [ctypes.c_double]
        L.oracle_gelu_f64.restype = ctypes.c_double
        L.oracle_gelu_f32.argtypes = [ctypes.c_float]
        L.oracle_gelu_f32.restype = ctypes.c_float
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def _f32(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def _p32(x):
    return x.ctypes.data_as(_f32p)


def _p64(x):
    return x.ctypes.data_as(_f64p)


def round_bf16(x) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned widened back to float32."""
    x = _f32(x)
    out = np.empty_like(x)
    lib().oracle_round_bf16(_p32(x), _p32(out), x.size)
    return out


def gemm(a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None) -> np.ndarray:
    """C = alpha*op(A)*op(B) + beta*C in fp64; rank 2 or rank 3 (batched).

    Follows kernels::matmul (include/llmt/kernels/matmul.h:12-24): all tensors
    share one rank, rank 3 means one independent GEMM per leading index.
    """
    a = _f32(a)
    b = _f32(b)
    if a.ndim != b.ndim or a.ndim not in (2, 3):
        raise ValueError("expected rank-2 or rank-3 tensors of equal rank")
    batch = a.shape[0] if a.ndim == 3 else 1
    ar, ac = a.shape[-2], a.shape[-1]
    br, bc = b.shape[-2], b.shape[-1]
    m, k = (ac, ar) if trans_a else (ar, ac)
    kb, n = (bc, br) if trans_b else (br, bc)
    if k != kb:
        raise ValueError(f"inner dims disagree: {k} vs {kb}")
    if a.ndim == 3 and b.shape[0] != batch:
        raise ValueError("batch sizes disagree")
    shape = (batch, m, n) if a.ndim == 3 else (m, n)
    if c is None:
        out = np.zeros(shape, dtype=np.float64)
        beta = 0.0
    else:
        out = np.array(c, dtype=np.float64, order="C", copy=True).reshape(shape)
    lib().oracle_gemm_f64(m, n, k, batch,
                          _p32(a), ac, ar * ac, int(trans_a),
                          _p32(b), bc, br * bc, int(trans_b),
                          _p64(out), n, m * n, float(alpha), float(beta))
    return out


def gemm_f32(a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None) -> np.ndarray:
    """fp32-arithmetic blocked host GEMM (the timed CPU baseline), rank 2."""
    a = _f32(a)
    b = _f32(b)
    ar, ac = a.shape
    br, bc = b.shape
    m, k = (ac, ar) if trans_a else (ar, ac)
    n = br if trans_b else bc
    out = np.zeros((m, n), np.float32) if c is None else _f32(c).copy()
    lib().oracle_gemm_f32(m, n, k, _p32(a), ac, int(trans_a), _p32(b), bc, int(trans_b),
                          _p32(out), n, float(alpha), float(beta if c is not None else 0.0))
    return out


def epilogue(c64, bias=None, gelu=False) -> np.ndarray:
    """matmul result -> + bias[j] -> tanh-GELU (src/kernels/gelu.cu:23-26), in fp64."""
    out = np.array(c64, dtype=np.float64, order="C", copy=True)
    m2 = out.reshape(-1, out.shape[-1])
    flags = (1 if bias is not None else 0) | (2 if gelu else 0)
    bb = _f32(bias) if bias is not None else np.zeros(1, np.float32)
    lib().oracle_epilogue_f64(_p64(m2), m2.shape[0], m2.shape[1], m2.shape[1], _p32(bb), flags)
    return out


def rowsum(a, trans_a=False, out=None, out_beta=0.0) -> np.ndarray:
    """out[i] = out_beta*out[i] + sum_p op(A)[i,p] (the dbias extension)."""
    a = _f32(a)
    ar, ac = a.shape
    m, k = (ac, ar) if trans_a else (ar, ac)
    res = np.zeros(m, np.float64) if out is None else np.array(out, np.float64).copy()
    lib().oracle_rowsum_f64(m, k, _p32(a), ac, int(trans_a), _p64(res),
                            float(out_beta if out is not None else 0.0))
    return res


def softmax(x, causal: bool) -> np.ndarray:
    """Row softmax of [batch, Tq, Tk] with llmt's causal rule (softmax.cu:33-50)."""
    x = np.ascontiguousarray(x, dtype=np.float64)
    y = np.empty_like(x)
    tq, tk = x.shape[-2], x.shape[-1]
    lib().oracle_softmax_f64(_p64(x), _p64(y), x.size // tk, tq, tk, int(causal))
    return y


def softmax_bwd(p, dp) -> np.ndarray:
    """dS = P*(dP - rowsum(dP*P)) (docs/TODO.md:227)."""
    p = np.ascontiguousarray(p, dtype=np.float64)
    dp = np.ascontiguousarray(dp, dtype=np.float64)
    ds = np.empty_like(p)
    tk = p.shape[-1]
    lib().oracle_softmax_bwd_f64(_p64(p), _p64(dp), _p64(ds), p.size // tk, tk)
    return ds


def cross_entropy(logits, targets, mask):
    """Masked cross-entropy from raw logits [..., V] in fp64 (llmt
    src/kernels/cross_entropy.cu:26-49 per row, :57-77 the mask-weighted mean):
    row_nll = mask * (logsumexp(logits) - logits[target]); loss = sum(row_nll) / sum(mask).
    Returns (loss, row_nll)."""
    x = np.asarray(logits, dtype=np.float64)
    v = x.shape[-1]
    x2 = x.reshape(-1, v)
    t = np.asarray(targets).reshape(-1).astype(np.int64)
    w = np.asarray(mask, dtype=np.float64).reshape(-1)
    m = x2.max(axis=1)
    lse = m + np.log(np.exp(x2 - m[:, None]).sum(axis=1))
    nll = w * (lse - x2[np.arange(x2.shape[0]), t])
    return nll.sum() / w.sum(), nll.reshape(np.asarray(targets).shape)


def cross_entropy_bwd(logits, targets, mask, dloss=1.0) -> np.ndarray:
    """Gradient of the masked mean cross-entropy with respect to the logits, in fp64 (llmt
    docs/TODO.md:216-217: dlogits = (softmax - onehot) * mask / sum(mask))."""
    x = np.asarray(logits, dtype=np.float64)
    v = x.shape[-1]
    x2 = x.reshape(-1, v)
    t = np.asarray(targets).reshape(-1).astype(np.int64)
    w = np.asarray(mask, dtype=np.float64).reshape(-1)
    m = x2.max(axis=1, keepdims=True)
    e = np.exp(x2 - m)
    g = e / e.sum(axis=1, keepdims=True)
    g[np.arange(x2.shape[0]), t] -= 1.0
    g *= (dloss * w / w.sum())[:, None]
    return g.reshape(x.shape)


def gelu(x) -> np.ndarray:
    x = np.asarray(x, dtype=np.float64)
    k0, k1 = 0.7978845608028654, 0.044715
    return 0.5 * x * (1.0 + np.tanh(k0 * (x + k1 * x ** 3)))


def gelu_bwd(x) -> np.ndarray:
    """Derivative of the tanh-GELU (src/kernels/gelu.cu:23-26 gives the function; llmt plans
    gelu_bwd in docs/TODO.md:223) in fp64."""
    x = np.asarray(x, dtype=np.float64)
    k0, k1 = 0.7978845608028654, 0.044715
    t = np.tanh(k0 * (x + k1 * x ** 3))
    return 0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * k0 * (1.0 + 3.0 * k1 * x * x)


def rel_fro(x, ref) -> float:
    """Relative Frobenius error ||x-ref|| / ||ref|| in fp64."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref.ravel())
    return float(np.linalg.norm((x - ref).ravel()) / (den if den > 0 else 1.0))
