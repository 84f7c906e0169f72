"""The softmax of an attention layer fused around its GEMMs (llmt src/kernels/attention.cpp:60-62,
src/kernels/softmax.cu:25-51, docs/TODO.md:226-228): probs = softmax(alpha q k^T) without the scores
ever being stored, dS = probs * (dO v^T - D) without dP ever being stored.  Checked against the fp64
oracle on the same bf16-rounded operands and against the unfused composition on the GPU."""
import numpy as np
import pytest
import torch

import llmt_b200 as L
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)

# a bf16 result carries its own rounding (2^-9 relative) on top of the fp32 arithmetic
TOL_BF16_OUT_FRO = 4e-3
TOL_F32_OUT_FRO = 2e-5


def dev_bf16(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(DEV).to(torch.bfloat16)


def host(t):
    return t.detach().to(torch.float32).cpu().numpy()


def _fwd(q, k, alpha, causal, out_dtype, want_lse=True):
    """probs [B, Tq, Tk] and lse [B, Tq] from q [B, Tq, hd], k [B, Tk, hd] on the device."""
    B, tq, tk = q.shape[0], q.shape[1], k.shape[1]
    p = torch.full((B, tq, tk), float("nan"), device=DEV, dtype=out_dtype)
    d = L.make_desc(p, q, k, False, True, alpha=alpha)
    need = L.gemm_softmax_workspace_bytes(d, q, k)
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    lse = torch.full((B, tq), float("nan"), device=DEV) if want_lse else None
    L.gemm_softmax_fwd(d, p, q, k, causal, lse)
    L.device_status()
    return p, lse


@pytest.mark.parametrize("B,tq,tk,hd,causal,out", [
    (1, 128, 128, 64, True, torch.bfloat16),
    (3, 256, 256, 64, True, torch.bfloat16),
    (2, 1024, 1024, 64, True, torch.bfloat16),
    (2, 1024, 1024, 64, False, torch.bfloat16),
    (2, 200, 200, 64, True, torch.bfloat16),     # ragged tiles
    (2, 100, 333, 40, False, torch.bfloat16),    # Tq != Tk, pitch TMA cannot address for C
    (2, 320, 320, 128, True, torch.float32),
    (1, 1, 1, 8, True, torch.bfloat16),
    (5, 37, 37, 24, True, torch.float32),
])
def test_fused_softmax_forward_against_the_oracle(B, tq, tk, hd, causal, out):
    rng = np.random.default_rng(B * 1000 + tq + tk + hd)
    q = oracle.round_bf16(rng.standard_normal((B, tq, hd)) * 2.0)
    k = oracle.round_bf16(rng.standard_normal((B, tk, hd)) * 2.0)
    q[0, 0, :] *= 6.0  # a row with scores far from zero: exponentials need the maximum
    q = oracle.round_bf16(q)
    alpha = 1.0 / np.sqrt(hd)
    p, lse = _fwd(dev_bf16(q), dev_bf16(k), alpha, causal, out)
    s_ref = oracle.gemm(q, k, False, True, alpha)
    p_ref = oracle.softmax(s_ref, causal)
    ph = host(p)
    assert np.isfinite(ph).all()
    tol = TOL_BF16_OUT_FRO if out == torch.bfloat16 else TOL_F32_OUT_FRO
    assert oracle.rel_fro(ph, p_ref) <= tol
    if causal:
        iu = np.triu_indices(tq, 1, tk)
        assert (ph[:, iu[0], iu[1]] == 0.0).all(), "masked probabilities must be exact zeros"
    # rows sum to one within the result type's rounding
    assert np.abs(ph.sum(-1) - 1.0).max() <= (2e-2 if out == torch.bfloat16 else 1e-5)
    # the rows' log-sum-exp
    s_m = s_ref.copy()
    if causal:
        s_m[:, iu[0], iu[1]] = -np.inf
    mx = s_m.max(-1)
    lse_ref = mx + np.log(np.exp(s_m - mx[..., None]).sum(-1))
    assert np.abs(host(lse) - lse_ref).max() <= 1e-4 * max(1.0, np.abs(lse_ref).max())


def test_fused_softmax_reruns_bitwise_and_matches_the_unfused_composition():
    B, T, hd = 4, 512, 64
    rng = np.random.default_rng(11)
    q = dev_bf16(rng.standard_normal((B, T, hd)))
    k = dev_bf16(rng.standard_normal((B, T, hd)))
    p1, l1 = _fwd(q, k, 0.125, True, torch.bfloat16)
    p2, l2 = _fwd(q, k, 0.125, True, torch.bfloat16, want_lse=False)
    assert l2 is None
    assert torch.equal(p1, p2)
    # llmt's composition: scores rounded to bf16, then the softmax kernel
    s = torch.empty(B, T, T, device=DEV, dtype=torch.bfloat16)
    L.gemm(s, q, k, False, True, alpha=0.125)
    L.softmax_fwd(s, s, causal=True)
    assert oracle.rel_fro(host(p1), host(s).astype(np.float64)) <= 2 * TOL_BF16_OUT_FRO


def test_fused_softmax_on_the_packed_qkv_layout():
    """q and k read straight out of the [B, T, 3*H*hd] projection output (two-level batch)."""
    B, H, T, hd = 2, 3, 256, 64
    A = H * hd
    rng = np.random.default_rng(21)
    qkv = oracle.round_bf16(rng.standard_normal((B, T, 3 * A)))
    qkv_d = dev_bf16(qkv)
    p = torch.empty(B, H, T, T, device=DEV, dtype=torch.bfloat16)
    d = L.GemmDesc()
    d.m, d.n, d.k, d.batch, d.batch_inner = T, T, hd, B * H, H
    d.lda, d.ldb, d.ldc = 3 * A, 3 * A, T
    d.stride_a, d.stride_b, d.stride_c = hd, hd, T * T
    d.stride_a_outer, d.stride_b_outer, d.stride_c_outer = T * 3 * A, T * 3 * A, H * T * T
    d.trans_a, d.trans_b = 0, 1
    d.dtype_ab, d.dtype_c = L.BF16, L.BF16
    d.alpha, d.beta = 0.125, 0.0
    a_ptr, b_ptr = qkv_d, qkv_d[0, 0, A:]
    need = L.gemm_softmax_workspace_bytes(d, a_ptr, b_ptr)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    lse = torch.empty(B * H, T, device=DEV)
    L.gemm_softmax_fwd(d, p, a_ptr, b_ptr, True, lse)
    L.device_status()
    x = qkv.reshape(B, T, 3, H, hd)
    qh = x[:, :, 0].transpose(0, 2, 1, 3).reshape(B * H, T, hd)
    kh = x[:, :, 1].transpose(0, 2, 1, 3).reshape(B * H, T, hd)
    p_ref = oracle.softmax(oracle.gemm(np.ascontiguousarray(qh), np.ascontiguousarray(kh), False, True, 0.125), True)
    assert oracle.rel_fro(host(p).reshape(B * H, T, T), p_ref) <= TOL_BF16_OUT_FRO


@pytest.mark.parametrize("B,T,hd,causal,out", [
    (2, 256, 64, True, torch.bfloat16),
    (2, 1024, 64, True, torch.bfloat16),
    (3, 200, 40, True, torch.bfloat16),
    (2, 192, 64, False, torch.float32),
])
def test_fused_softmax_backward_against_the_oracle(B, T, hd, causal, out):
    """dS = P * (dO V^T - D), D = rowsum(dO * O): against the oracle's softmax backward on the same P."""
    rng = np.random.default_rng(B + T + hd)
    q = oracle.round_bf16(rng.standard_normal((B, T, hd)))
    k = oracle.round_bf16(rng.standard_normal((B, T, hd)))
    v = oracle.round_bf16(rng.standard_normal((B, T, hd)))
    d_o = oracle.round_bf16(rng.standard_normal((B, T, hd)) * 0.01)
    p, _ = _fwd(dev_bf16(q), dev_bf16(k), 1.0 / np.sqrt(hd), causal, out)
    ph = host(p)
    vd, dod = dev_bf16(v), dev_bf16(d_o)
    # O in fp32 from the stored P (bf16 P needs bf16 operands for the product: take the oracle's O)
    o_ref = oracle.gemm(ph, v)
    o = torch.from_numpy(o_ref.astype(np.float32)).to(DEV)
    dof = dod.to(torch.float32)
    dvec = torch.empty(B, T, device=DEV)
    L.rowdot(dvec, dof, o)
    L.device_status()
    d_ref = (d_o.astype(np.float64) * o_ref).sum(-1)
    assert np.abs(host(dvec) - d_ref).max() <= 1e-5 * max(1.0, np.abs(d_ref).max()) + 1e-7
    ds = torch.full((B, T, T), float("nan"), device=DEV, dtype=out)
    d = L.make_desc(ds, dod, vd, False, True)
    need = L.workspace_bytes(d, dod, vd)
    ws = torch.empty(max(need, 256), dtype=torch.uint8, device=DEV)
    d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
    L.gemm_softmax_bwd(d, ds, dod, vd, p, dvec, causal)
    L.device_status()
    dp_ref = oracle.gemm(d_o, v, False, True)
    ds_ref = oracle.softmax_bwd(ph.astype(np.float64), dp_ref)
    dsh = host(ds)
    assert np.isfinite(dsh).all()
    assert oracle.rel_fro(dsh, ds_ref) <= (TOL_BF16_OUT_FRO if out == torch.bfloat16 else 1e-4)
    if causal:
        iu = np.triu_indices(T, 1)
        assert (dsh[:, iu[0], iu[1]] == 0.0).all()


def test_rowdot_bf16_rows():
    rng = np.random.default_rng(5)
    x = oracle.round_bf16(rng.standard_normal((3, 50, 72)))
    y = oracle.round_bf16(rng.standard_normal((3, 50, 72)))
    out = torch.empty(3, 50, device=DEV)
    L.rowdot(out, dev_bf16(x), dev_bf16(y))
    want = (x.astype(np.float64) * y.astype(np.float64)).sum(-1)
    assert np.abs(host(out) - want).max() <= 1e-4


def test_fused_softmax_rejects_what_it_cannot_do():
    q = torch.zeros(2, 64, 64, device=DEV, dtype=torch.bfloat16)
    p = torch.zeros(2, 64, 128, device=DEV, dtype=torch.bfloat16)
    k = torch.zeros(2, 128, 64, device=DEV, dtype=torch.bfloat16)
    d = L.make_desc(p, q, k, False, True)
    ws = torch.empty(1 << 20, dtype=torch.uint8, device=DEV)
    d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
    with pytest.raises(L.LlmtB200Error, match="causal mask requires square scores"):
        L.gemm_softmax_fwd(d, p, q, k, True)
    d.workspace_bytes = 0
    with pytest.raises(L.LlmtB200Error, match="workspace"):
        L.gemm_softmax_fwd(d, p, q, k, False)
    d.workspace_bytes = ws.numel()
    d.beta = 1.0
    with pytest.raises(L.LlmtB200Error, match="beta must be 0"):
        L.gemm_softmax_fwd(d, p, q, k, False)
    qf = torch.zeros(2, 64, 64, device=DEV)
    kf = torch.zeros(2, 128, 64, device=DEV)
    pf = torch.zeros(2, 64, 128, device=DEV)
    df = L.make_desc(pf, qf, kf, False, True)
    df.workspace, df.workspace_bytes = ws.data_ptr(), ws.numel()
    with pytest.raises(L.LlmtB200Error, match="bf16 operands only"):
        L.gemm_softmax_fwd(df, pf, qf, kf, False)
