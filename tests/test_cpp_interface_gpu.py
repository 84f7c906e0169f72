"""Runs the C++ golden-test binary: llmt's own known-answer tests (matmul,
rank-3, Linear fwd/bwd with accumulation, MLP, attention stages) written against
llmt's C++ interface and linked with the llmt_b200 implementation."""
import os
import subprocess

import pytest

from tests.support import LLMT_GOLDEN_DIR

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "_build", "test_llmt_goldens")


@pytest.mark.gpu
def test_llmt_cpp_interface_goldens():
    assert os.path.exists(BIN), "run `python -m llmt_b200.build` (or __graft_entry__.build()) first"
    r = subprocess.run([BIN, LLMT_GOLDEN_DIR], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "0 failures" in r.stdout


@pytest.mark.gpu
def test_cpp_param_store_allreduce_over_cuda_ipc_two_processes():
    """The C++ host side of the exchange: ParamStore (aliases, four spans, gradient span placed in
    a dist::PeerExchange allocation) + allreduce_grads over CUDA IPC, two processes on two GPUs."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    binary = os.path.join(ROOT, "tests", "cpp", "_build", "test_peer_exchange")
    assert os.path.exists(binary), "run `python -m llmt_b200.build` (or __graft_entry__.build()) first"
    r = subprocess.run([binary, "2"], capture_output=True, text=True, timeout=300)
    if r.returncode == 77:
        pytest.skip("fewer GPUs than ranks")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "0 failures" in r.stdout


def test_cpp_interface_is_built_and_links_the_c_abi():
    """CPU check: the interface library exists and resolves against the C-ABI library."""
    host = os.path.join(ROOT, "llmt_b200", "lib", "libllmt_b200_host.so")
    if not os.path.exists(host):
        pytest.skip("C++ interface library not built yet")
    out = subprocess.run(["ldd", host], capture_output=True, text=True).stdout
    assert "libllmt_b200.so" in out and "not found" not in out.split("libllmt_b200.so")[1].split("\n")[0]
