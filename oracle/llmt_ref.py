"""ctypes front end of oracle/_ref/libllmt_ref.so — the UNMODIFIED llmt library
(cuBLASLt, strict fp32) compiled from its own sources by `make -C oracle ref`.

TEST / BASELINE INFRASTRUCTURE, NOT PRODUCT. Needs a GPU to run. Used by the
GPU parity tests as a second checker and by the benchmark's reference arm.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libllmt_ref.so")
_lib = None


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
        L.ref_create.restype = ctypes.c_void_p
        L.ref_create.argtypes = [ctypes.c_int]
        L.ref_destroy.argtypes = [ctypes.c_void_p]
        i64p = ctypes.POINTER(ctypes.c_int64)
        L.ref_matmul.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                 ctypes.c_int, i64p, i64p, i64p, ctypes.c_int, ctypes.c_int,
                                 ctypes.c_float, ctypes.c_float, ctypes.c_void_p]
        L.ref_gelu.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                               ctypes.c_void_p]
        L.ref_softmax.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                  ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
        L.ref_linear.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                 ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        L.ref_synchronize.argtypes = [ctypes.c_void_p]
        _lib = L
    return _lib


class Llmt:
    """One llmt Device + RunCtx (fp32 policy)."""

    def __init__(self, device: int = 0):
        self.h = lib().ref_create(device)

    def close(self):
        if self.h:
            lib().ref_destroy(self.h)
            self.h = None

    @staticmethod
    def _dims(t):
        return (ctypes.c_int64 * t.dim())(*t.shape)

    def matmul(self, c, a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, stream=None):
        """llmt::kernels::matmul on contiguous fp32 torch tensors (rank 2 or 3)."""
        import torch
        for t in (c, a, b):
            assert t.is_contiguous() and t.dtype == torch.float32
        s = stream if stream is not None else torch.cuda.current_stream()
        lib().ref_matmul(self.h, c.data_ptr(), a.data_ptr(), b.data_ptr(), c.dim(),
                         self._dims(c), self._dims(a), self._dims(b), int(trans_a), int(trans_b),
                         float(alpha), float(beta), ctypes.c_void_p(s.cuda_stream))

    def gelu(self, y, x, stream=None):
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        lib().ref_gelu(self.h, y.data_ptr(), x.data_ptr(), x.numel(), ctypes.c_void_p(s.cuda_stream))

    def softmax(self, y, x, causal, stream=None):
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        lib().ref_softmax(self.h, y.data_ptr(), x.data_ptr(), x.shape[0], x.shape[1], x.shape[2],
                          int(causal), ctypes.c_void_p(s.cuda_stream))

    def linear(self, w, x, dy, backward_calls=1):
        """llmt::Linear forward + backward; returns (y, dx, dW)."""
        import torch
        torch.cuda.synchronize()
        m, in_f = x.shape
        out_f = w.shape[0]
        y = torch.empty(m, out_f, device=x.device)
        dx = torch.empty(m, in_f, device=x.device)
        dw = torch.empty(out_f, in_f, device=x.device)
        lib().ref_linear(self.h, m, in_f, out_f, w.data_ptr(), x.data_ptr(), dy.data_ptr(),
                         y.data_ptr(), dx.data_ptr(), dw.data_ptr(), backward_calls)
        return y, dx, dw
