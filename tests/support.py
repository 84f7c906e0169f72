"""Shared helpers for the tests: llmt golden-file reader and comparison rules."""
from __future__ import annotations

import os
import struct

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
LLMT_GOLDEN_DIR = os.path.join(GOLDEN_DIR, "llmt")

_MAGIC = 0x544D4C4C  # "LLMT"
_DTYPES = {0: np.float32, 1: np.uint16, 2: np.int32}  # code 1 = bf16 bit patterns


def read_golden(path: str) -> np.ndarray:
    """Reads one llmt golden tensor (docs/golden.md:8-21 of llmt: 16-byte header
    magic/version/dtype/rank, then int64 dims, then the row-major payload)."""
    with open(path, "rb") as f:
        raw = f.read()
    magic, version, dtype, rank = struct.unpack_from("<IIII", raw, 0)
    if magic != _MAGIC or version != 1 or rank > 4 or dtype not in _DTYPES:
        raise ValueError(f"{path}: not an llmt golden tensor")
    dims = struct.unpack_from(f"<{rank}q", raw, 16)
    off = 16 + 8 * rank
    arr = np.frombuffer(raw, dtype=_DTYPES[dtype], offset=off)
    return arr.reshape(dims).copy()


def write_golden(path: str, arr: np.ndarray) -> None:
    """Writes a tensor in the same format (float32 / int32 only)."""
    arr = np.ascontiguousarray(arr)
    code = {np.dtype(np.float32): 0, np.dtype(np.uint16): 1, np.dtype(np.int32): 2}[arr.dtype]
    with open(path, "wb") as f:
        f.write(struct.pack("<IIII", _MAGIC, 1, code, arr.ndim))
        f.write(struct.pack(f"<{arr.ndim}q", *arr.shape))
        f.write(arr.tobytes())


class GoldenCase:
    def __init__(self, name: str, root: str = LLMT_GOLDEN_DIR):
        self.dir = os.path.join(root, name)

    def tensor(self, name: str) -> np.ndarray:
        return read_golden(os.path.join(self.dir, name + ".bin"))


def assert_close(actual, expected, rtol=1e-5, atol=1e-6, what=""):
    """llmt's comparison rule (tests/support/golden_io.cpp:66-88 of llmt):
    |a-e| <= atol + rtol*|e| elementwise, NaN always a mismatch."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    bad = ~(np.abs(a - e) <= atol + rtol * np.abs(e))
    if bad.any():
        idx = np.argwhere(bad)[0]
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{a.size} mismatches; first at {tuple(idx)}: "
            f"got {a[tuple(idx)]!r} want {e[tuple(idx)]!r}")
