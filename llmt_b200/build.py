"""Builds libllmt_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m llmt_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. Objects go to llmt_b200/_build/, the shared
library to llmt_b200/lib/libllmt_b200.so.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "_build")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libllmt_b200.so")

SOURCES = ["capi.cu", "gemm_grouped_sm100.cu", "gemm_fp32_simt.cu", "grad_allreduce_sm100.cu", "cross_entropy.cu"]
HEADERS = ["common.h", "ptx_sm100.cuh", os.path.join("..", "..", "include", "llmt_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build llmt_b200")
    return path


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    hdrs = [os.path.normpath(os.path.join(CSRC, h)) for h in HEADERS]
    jobs = []
    objs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s, *hdrs, os.path.abspath(__file__)]):
            cmd = [nvcc(), *NVCC_FLAGS, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    with concurrent.futures.ThreadPoolExecutor(max_workers=4) as ex:
        for cmd, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    if force or jobs or _stale(LIB_PATH, objs):
        # The public symbols are the extern "C" ones marked default-visible below.
        cmd = [nvcc(), "-shared", "-o", LIB_PATH, *objs, "-Xcompiler", "-fPIC",
               "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


CPP_DIR = os.path.join(HERE, "cpp")
CPP_SOURCES = ["runtime.cpp", "matmul.cpp", "layers.cpp", "attention.cpp", "peer_exchange.cpp", "cross_entropy.cpp"]
HOST_LIB = os.path.join(LIB_DIR, "libllmt_b200_host.so")
ROOT = os.path.dirname(HERE)
CPP_TEST_SRC = os.path.join(ROOT, "tests", "cpp", "test_llmt_goldens.cpp")
CPP_TEST_BIN = os.path.join(ROOT, "tests", "cpp", "_build", "test_llmt_goldens")
CPP_TESTS = {"test_llmt_goldens": CPP_TEST_BIN,
             "test_peer_exchange": os.path.join(ROOT, "tests", "cpp", "_build", "test_peer_exchange")}


def build_cpp(force: bool = False) -> str:
    """Builds the C++ interface library (llmt's matmul / Linear / MLP / attention
    API over the C ABI) and the golden-test binary that exercises it."""
    build_library()
    inc = [os.path.join(CPP_DIR, "include"), os.path.join(ROOT, "include")]
    srcs = [os.path.join(CPP_DIR, "src", s) for s in CPP_SOURCES]
    hdrs = []
    for base, _d, files in os.walk(inc[0]):
        hdrs += [os.path.join(base, f) for f in files]
    flags = ["-std=c++20", "-O2", "-Wno-deprecated-gpu-targets", "-Xcompiler", "-fPIC,-Wall,-Wextra"] + [f"-I{i}" for i in inc]
    rpath = ["-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    if force or _stale(HOST_LIB, srcs + hdrs + [LIB_PATH]):
        cmd = [nvcc(), *flags, "-shared", "-o", HOST_LIB, *srcs, f"-L{LIB_DIR}", "-lllmt_b200", *rpath]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("C++ interface library failed to build")
    os.makedirs(os.path.dirname(CPP_TEST_BIN), exist_ok=True)
    for name, binary in CPP_TESTS.items():
        src = os.path.join(ROOT, "tests", "cpp", name + ".cpp")
        if force or _stale(binary, [src, HOST_LIB]):
            cmd = [nvcc(), *flags, "-o", binary, src, f"-L{LIB_DIR}", "-lllmt_b200_host",
                   "-lllmt_b200", "-Xlinker", "-rpath", "-Xlinker", LIB_DIR,
                   "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../llmt_b200/lib"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
                raise RuntimeError(f"C++ test {name} failed to build")
    return CPP_TEST_BIN


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    print(build_cpp(force="--force" in sys.argv))
