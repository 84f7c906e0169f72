"""The benchmark configurations at their full sizes, through the C ABI, checked on sampled
output rows against the fp64 oracle of the same bf16-rounded inputs.

  config 2  GPT-2-small linears at M = 8192: QKV, attention out-proj, MLP fc (bias + GELU),
            MLP proj; each forward, dX and dW + dbias (llmt src/layers/linear.cpp:16-30)
  config 3  LM head at M = 8192, vocabulary 50257: row pitch 50264 and contiguous
  config 4  the six attention products at B*H = 96, T = 1024, hd = 64
            (llmt src/kernels/attention.cpp:60-62, docs/TODO.md:226-228)
  config 5  GPT-2-XL MLP (1600 <-> 6400) on one 8192-token shard: fc and proj, forward, dX, dW

Tolerances: fp32 outputs <= 1e-3 relative Frobenius, bf16 outputs <= 4e-3 (rounding the exact
result to bf16 is itself 1.7e-3 away), as in test_gemm_gpu.py.
"""
import numpy as np
import pytest
import torch

import llmt_b200 as L
from oracle import oracle

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL_F32, TOL_BF16 = 1e-3, 4e-3


@pytest.fixture(autouse=True)
def _healthy_device():
    yield
    assert L.device_status() == (0, 0)


def _gen(seed):
    return torch.Generator(device=DEV).manual_seed(seed)


def _randn_bf16(g, *shape, scale=1.0):
    return (torch.randn(*shape, device=DEV, generator=g) * scale).to(torch.bfloat16)


def _np(t):
    return t.float().cpu().numpy()


def _rows(g, n, count):
    """A sample of row indices that always holds the first and the last row."""
    idx = torch.randperm(n, device=DEV, generator=g)[:count].tolist()
    return sorted(set(idx + [0, n - 1]))


def _check(c, a_rows64, b, tb, rows, tol, post=None, alpha=1.0):
    """c[rows] against oracle(a_rows64 (x) b)."""
    ref = oracle.gemm(a_rows64, b, False, tb, alpha)
    if post is not None:
        ref = post(ref)
    got = _np(c[torch.as_tensor(rows, device=DEV)])
    err = oracle.rel_fro(got, ref)
    assert err <= tol, err


def _linear_layer_full(m, i, o, seed, gelu, bias=True, pairs_note=""):
    g = _gen(seed)
    x = _randn_bf16(g, m, i)
    w = _randn_bf16(g, o, i, scale=0.02)
    dy = _randn_bf16(g, m, o, scale=0.01)
    b = torch.randn(o, device=DEV, generator=g) * 0.02 if bias else None
    xh, wh, dyh = _np(x), _np(w), _np(dy)
    bh = _np(b) if bias else None
    rows = _rows(g, m, 24)
    # forward: y = epilogue(x W^T + b)
    y = torch.empty(m, o, device=DEV, dtype=torch.bfloat16)
    L.gemm(y, x, w, False, True, bias=b, gelu=gelu)
    _check(y, xh[rows], wh, True, rows, TOL_BF16, post=lambda r: oracle.epilogue(r, bias=bh, gelu=gelu))
    # Linear::backward as one launch: dx = dy W, dW += dy^T x, dbias += column sums of dy
    dx = torch.empty(m, i, device=DEV, dtype=torch.bfloat16)
    dw = torch.zeros(o, i, device=DEV)
    db = torch.zeros(o, device=DEV) if bias else None
    grp = L.Group([(L.make_desc(dx, dy, w, False, False), dx, dy, w),
                   (L.make_desc(dw, dy, x, True, False, beta=1.0, dbias=db, dbias_beta=1.0), dw, dy, x)])
    grp.set_workspaces([torch.empty(max(n, 256), dtype=torch.uint8, device=DEV) for n in grp.workspace_bytes()])
    grp.run()
    _check(dx, dyh[rows], wh, False, rows, TOL_BF16)
    orows = _rows(g, o, 16)
    _check(dw, np.ascontiguousarray(dyh.T[orows]), xh, False, orows, TOL_F32)
    if bias:
        assert oracle.rel_fro(_np(db), oracle.rowsum(dyh, trans_a=True)) <= TOL_F32
    # accumulation contract (llmt tests/unit/test_linear.cu:49-56): a second backward doubles dW
    dw1 = dw.clone()
    db1 = db.clone() if bias else None
    grp.run()
    assert torch.allclose(dw, 2.0 * dw1, rtol=1e-6, atol=0)
    if bias:
        assert torch.allclose(db, 2.0 * db1, rtol=1e-6, atol=0)
    # determinism (llmt tests/unit/test_matmul.cu:86-103): the same launch again from the same
    # start gives the same bits
    dw.copy_(dw1)
    if bias:
        db.copy_(db1)
    grp.run()
    dw2 = dw.clone()
    dw.copy_(dw1)
    if bias:
        db.copy_(db1)
    grp.run()
    assert torch.equal(dw, dw2)


@pytest.mark.parametrize("name,i,o,gelu", [("qkv", 768, 2304, False), ("attn_out", 768, 768, False),
                                           ("mlp_fc", 768, 3072, True), ("mlp_proj", 3072, 768, False)])
def test_config2_every_layer_forward_dx_dw(name, i, o, gelu):
    _linear_layer_full(8192, i, o, seed=200 + i + o, gelu=gelu)


@pytest.mark.parametrize("name,i,o,gelu", [("mlp_fc", 1600, 6400, True), ("mlp_proj", 6400, 1600, False)])
def test_config5_xl_mlp_forward_dx_dw(name, i, o, gelu):
    _linear_layer_full(8192, i, o, seed=500 + i, gelu=gelu)


@pytest.mark.parametrize("contiguous", [False, True])
def test_config3_lm_head_full_size(contiguous):
    """M = 8192 tokens, vocabulary 50257: fp32 logits, dX = dLogits W, dW = dLogits^T X.
    Row pitch 50264 (TMA reads and writes in place) or contiguous 50257 (pitch of 100514 /
    201028 bytes: logits leave through registers, dLogits is first copied to an aligned pitch)."""
    M, C, V = 8192, 768, 50257
    LD = V if contiguous else 50264
    g = _gen(3 + contiguous)
    x = _randn_bf16(g, M, C)
    w = _randn_bf16(g, V, C, scale=0.02)
    xh, wh = _np(x), _np(w)
    rows = _rows(g, M, 10)
    logits = torch.empty(M, LD, device=DEV)[:, :V]
    L.gemm(logits, x, w, False, True)
    _check(logits, xh[rows], wh, True, rows, TOL_F32)
    del logits
    dl = torch.zeros(M, LD, device=DEV, dtype=torch.bfloat16)
    dl[:, :V] = _randn_bf16(g, M, V, scale=1e-4)
    dl = dl[:, :V]
    dlh_rows = _np(dl[torch.as_tensor(rows, device=DEV)])
    dx = torch.empty(M, C, device=DEV, dtype=torch.bfloat16)
    L.gemm(dx, dl, w, False, False)
    _check(dx, dlh_rows, wh, False, rows, TOL_BF16)
    dw = torch.zeros(V, C, device=DEV)
    L.gemm(dw, dl, x, True, False, beta=1.0)
    vrows = sorted(set(_rows(g, V, 10) + [V - 2]))
    a_rows = np.ascontiguousarray(_np(dl[:, torch.as_tensor(vrows, device=DEV)]).T)
    _check(dw, a_rows, xh, False, vrows, TOL_F32)


def test_config4_attention_products_full_batch():
    """B*H = 96: S = QK^T/8, P = causal softmax(S), O = PV, dV = P^T dO, dP = dO V^T,
    dS = softmax backward, dQ = dS K / 8, dK = dS^T Q / 8; six sampled (batch, head) items are
    checked in full, every product against the oracle of its own inputs."""
    BH, T, HD = 96, 1024, 64
    alpha = 0.125
    g = _gen(4)
    q, k, v = (_randn_bf16(g, BH, T, HD) for _ in range(3))
    d_o = _randn_bf16(g, BH, T, HD, scale=0.01)
    bf = torch.bfloat16
    s = torch.empty(BH, T, T, device=DEV, dtype=bf)
    L.gemm(s, q, k, False, True, alpha=alpha)
    p = torch.empty_like(s)
    L.softmax_fwd(p, s, causal=True)
    o = torch.empty(BH, T, HD, device=DEV, dtype=bf)
    L.gemm(o, p, v, False, False)
    dv = torch.empty_like(o)
    L.gemm(dv, p, d_o, True, False)
    dp = torch.empty_like(s)
    L.gemm(dp, d_o, v, False, True)
    ds = torch.empty_like(s)
    L.softmax_bwd(ds, p, dp)
    dq, dk = torch.empty_like(o), torch.empty_like(o)
    L.gemm(dq, ds, k, False, False, alpha=alpha)
    L.gemm(dk, ds, q, True, False, alpha=alpha)
    iu = np.triu_indices(T, 1)
    for b in sorted(set(_rows(g, BH, 4))):
        qh, kh, vh, doh = (_np(t[b]) for t in (q, k, v, d_o))
        sh, ph, dph, dsh = (_np(t[b]) for t in (s, p, dp, ds))
        assert oracle.rel_fro(sh, oracle.gemm(qh, kh, False, True, alpha)) <= TOL_BF16
        assert oracle.rel_fro(ph, oracle.softmax(sh.astype(np.float64)[None], causal=True)[0]) <= TOL_BF16
        assert (ph[iu[0], iu[1]] == 0.0).all(), "masked probabilities must be exact zeros"
        assert oracle.rel_fro(_np(o[b]), oracle.gemm(ph, vh)) <= TOL_BF16
        assert oracle.rel_fro(_np(dv[b]), oracle.gemm(ph, doh, True, False)) <= TOL_BF16
        assert oracle.rel_fro(dph, oracle.gemm(doh, vh, False, True)) <= TOL_BF16
        ds_ref = oracle.softmax_bwd(ph.astype(np.float64)[None], dph.astype(np.float64)[None])[0]
        assert oracle.rel_fro(dsh, ds_ref) <= TOL_BF16
        assert oracle.rel_fro(_np(dq[b]), oracle.gemm(dsh, kh, False, False, alpha)) <= TOL_BF16
        assert oracle.rel_fro(_np(dk[b]), oracle.gemm(dsh, qh, True, False, alpha)) <= TOL_BF16
