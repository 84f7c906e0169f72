"""ctypes front end of oracle/_build/libcublaslt_bf16.so: llmt's cuBLASLt call pattern
(operand swap, 32 MiB workspace, cached top-1 heuristic) with bf16 operands and fp32
accumulation. TEST / BASELINE INFRASTRUCTURE, NOT PRODUCT: an accuracy and speed
comparator on the GPU, used by tests/ and bench.py only."""
from __future__ import annotations

import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_build", "libcublaslt_bf16.so")
_lib = None


def build() -> str:
    src = os.path.join(_HERE, "cublaslt_bf16.cu")
    if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "cmp"])
    return LIB_PATH


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        for cand in ("/usr/local/cuda/lib64/libcublasLt.so.12",):
            if os.path.exists(cand):
                try:
                    ctypes.CDLL(cand, mode=ctypes.RTLD_GLOBAL)
                except OSError:
                    pass
        L = ctypes.CDLL(LIB_PATH)
        L.cmp_create.restype = ctypes.c_void_p
        L.cmp_destroy.argtypes = [ctypes.c_void_p]
        L.cmp_matmul_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                      ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                      ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                                      ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        L.cmp_matmul_bf16.restype = ctypes.c_int
        _lib = L
    return _lib


class CublasLtBf16:
    def __init__(self):
        self.h = lib().cmp_create()
        if not self.h:
            raise RuntimeError("cublasLtCreate failed")

    def close(self):
        if self.h:
            lib().cmp_destroy(self.h)
            self.h = None

    def matmul(self, c, a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, bias=None, gelu=False,
               stream=None, dbias=None):
        """C = alpha*op(A)*op(B) + beta*C on contiguous bf16 A/B and bf16-or-fp32 C (rank 2 or 3).
        dbias (fp32 [M] for fp32 C): Lt's bias-gradient epilogue writes sum_p op(A)[i, p] into it."""
        import torch
        assert a.is_contiguous() and b.is_contiguous() and c.is_contiguous()
        assert a.dtype == b.dtype == torch.bfloat16
        batch = a.shape[0] if a.dim() == 3 else 1
        ar, ac = a.shape[-2], a.shape[-1]
        br, bc = b.shape[-2], b.shape[-1]
        m, k = (ac, ar) if trans_a else (ar, ac)
        n = br if trans_b else bc
        epi = 0
        if dbias is not None:
            assert bias is None and not gelu
            epi, bias = 4, dbias
        elif bias is not None:
            epi = 3 if gelu else 1
        elif gelu:
            raise ValueError("GELU without bias is not an Lt epilogue used here")
        s = stream if stream is not None else torch.cuda.current_stream()
        rc = lib().cmp_matmul_bf16(self.h, c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, batch,
                                   int(trans_a), int(trans_b), float(alpha), float(beta),
                                   int(c.dtype == torch.float32), epi,
                                   bias.data_ptr() if bias is not None else None,
                                   ctypes.c_void_p(s.cuda_stream))
        if rc != 0:
            raise RuntimeError(f"cuBLASLt comparator failed with status {rc}")
