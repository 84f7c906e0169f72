"""The allocation-free entry point, llmt_b200_gemm_static_scratch.

It exists for hosts that have nowhere to get a workspace from when they need a
GEMM (a frozen memory plan where cudaMalloc would stall the device, a plugin
that receives tensors but no allocator). Its split-K scratch is a fixed array
inside the library. The test drives it through the C ABI on a split-K problem
(a Linear dW + dbias shape), twice in a row, and requires the same output as the
ordinary entry point gives with a caller-supplied workspace.
"""
import ctypes

import numpy as np
import pytest

import llmt_b200 as L


def _problem(torch, dev):
    # dW[out,in] += dy^T x with dbias: 36 output tiles and a 4096-long reduction -> split-K
    tokens, out_f, in_f = 4096, 768, 768
    g = torch.Generator(device=dev).manual_seed(123)
    dy = (torch.randn(tokens, out_f, device=dev, generator=g) * 0.01).to(torch.bfloat16)
    x = torch.randn(tokens, in_f, device=dev, generator=g).to(torch.bfloat16)
    dw0 = torch.randn(out_f, in_f, device=dev, generator=g)
    db0 = torch.randn(out_f, device=dev, generator=g)
    return dy, x, dw0, db0


@pytest.mark.gpu
def test_static_scratch_matches_the_workspace_entry_point_twice_in_a_row():
    import torch
    dev = "cuda:0"
    dy, x, dw0, db0 = _problem(torch, dev)

    # reference: the ordinary entry point with a caller-supplied workspace
    dw_ref, db_ref = dw0.clone(), db0.clone()
    d_ref = L.make_desc(dw_ref, dy, x, True, False, beta=1.0, dbias=db_ref, dbias_beta=1.0)
    need = L.workspace_bytes(d_ref)
    assert 0 < need <= L.STATIC_SCRATCH_BYTES, "the test problem must use split-K scratch"
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    d_ref.workspace, d_ref.workspace_bytes = ws.data_ptr(), need
    L.gemm_desc(d_ref, dw_ref, dy, x)
    torch.cuda.synchronize()

    before = torch.cuda.memory_allocated()
    for call in range(2):
        dw, db = dw0.clone(), db0.clone()
        d = L.make_desc(dw, dy, x, True, False, beta=1.0, dbias=db, dbias_beta=1.0)
        assert d.workspace is None and d.workspace_bytes == 0  # nothing handed in
        L.gemm_static_scratch(d, dw, dy, x)
        torch.cuda.synchronize()
        assert L.device_status() == (0, 0)
        # same plan, same fixed summation order: the tolerance of the other bf16 tests
        # (relative Frobenius <= 1e-3) is met with room to spare -- the bits are equal
        err = float((dw.double() - dw_ref.double()).norm() / dw_ref.double().norm())
        assert err <= 1e-3, f"call {call}: dW differs from the workspace entry point ({err:.3e})"
        assert torch.equal(dw, dw_ref), f"call {call}: dW not bitwise equal"
        assert torch.equal(db, db_ref), f"call {call}: dbias not bitwise equal"
        del dw, db
    assert torch.cuda.memory_allocated() <= before + 1024


@pytest.mark.gpu
def test_static_scratch_without_split_k_and_fp32_path():
    """Problems that need no scratch run through the same entry point unchanged."""
    import torch
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(5)
    a = torch.randn(512, 256, device=dev, generator=g)
    b = torch.randn(384, 256, device=dev, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        a2, b2 = a.to(dt), b.to(dt)
        c1 = torch.empty(512, 384, device=dev)
        c2 = torch.empty(512, 384, device=dev)
        d = L.make_desc(c1, a2, b2, False, True)
        L.gemm_desc(d, c1, a2, b2)
        L.gemm_static_scratch(L.make_desc(c2, a2, b2, False, True), c2, a2, b2)
        torch.cuda.synchronize()
        assert torch.equal(c1, c2)


def test_static_scratch_refuses_oversized_plans_before_touching_the_gpu():
    d = L.GemmDesc()
    d.m, d.n, d.k, d.batch = 4096, 4096, 65536, 1          # 8 splits x 64 MiB of partial sums
    d.lda, d.ldb, d.ldc = 4096, 4096, 4096
    d.trans_a = 1
    d.dtype_ab, d.dtype_c = L.BF16, L.FP32
    d.alpha = 1.0
    d.plan_tile_n, d.plan_splits = 256, 8
    st = L.lib().llmt_b200_gemm_static_scratch(
        ctypes.byref(d), ctypes.c_void_p(0x7000000000), ctypes.c_void_p(0x1000000000),
        ctypes.c_void_p(0x3000000000), None)
    assert st == L.ERR_WORKSPACE
    msg = L.last_error()
    assert "built-in scratch" in msg and str(L.STATIC_SCRATCH_BYTES) in msg
