"""dX through a GELU: the dX product of the layer after a tanh-GELU with gelu'(pre) as its epilogue
(llmt docs/TODO.md:223 plans gelu_bwd as a kernel of its own), alone and in a grouped launch with dW."""
import numpy as np
import pytest
import torch

import llmt_b200 as L
from oracle import oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def dev_bf16(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(DEV).to(torch.bfloat16)


def host(t):
    return t.detach().to(torch.float32).cpu().numpy()


@pytest.mark.parametrize("m,f,c,out", [(256, 512, 128, torch.bfloat16), (300, 1000, 192, torch.bfloat16),
                                       (1024, 3072, 768, torch.bfloat16), (200, 264, 64, torch.float32)])
def test_dx_through_gelu_against_the_oracle(m, f, c, out):
    """d_pre = (dy W_down) * gelu'(pre) with dy [m, c], W_down [c, f] (stored [out, in]), pre [m, f]."""
    rng = np.random.default_rng(m + f + c)
    dy = oracle.round_bf16(rng.standard_normal((m, c)) * 0.1)
    w = oracle.round_bf16(rng.standard_normal((c, f)) * 0.05)
    pre = rng.standard_normal((m, f)) * 2.0
    pre = oracle.round_bf16(pre) if out == torch.bfloat16 else pre.astype(np.float32)
    pre_d = dev_bf16(pre) if out == torch.bfloat16 else torch.from_numpy(pre).to(DEV)
    dyd, wd = dev_bf16(dy), dev_bf16(w)
    dpre = torch.full((m, f), float("nan"), device=DEV, dtype=out)
    d = L.make_desc(dpre, dyd, wd, False, False, gelu_bwd_of=pre_d)
    ws = torch.empty(max(L.workspace_bytes(d, dyd, wd), 256), dtype=torch.uint8, device=DEV)
    d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
    L.gemm_desc(d, dpre, dyd, wd)
    L.device_status()
    want = oracle.gemm(dy, w) * oracle.gelu_bwd(pre)
    got = host(dpre)
    assert np.isfinite(got).all()
    assert oracle.rel_fro(got, want) <= (4e-3 if out == torch.bfloat16 else 1e-4)
    # the same bits as the plain product followed by the multiplication, for an fp32 result
    dpre2 = torch.empty_like(dpre)
    L.gemm_desc(d, dpre2, dyd, wd)
    assert torch.equal(dpre, dpre2)


def test_dx_through_gelu_in_a_grouped_launch_with_dw():
    """The backward pass of the down projection as ONE launch: d_pre = (dy W) * gelu'(pre) and
    dW += dy^T h (+ dbias)."""
    m, f, c = 2048, 3072, 768
    rng = np.random.default_rng(9)
    dy = oracle.round_bf16(rng.standard_normal((m, c)) * 0.1)
    w = oracle.round_bf16(rng.standard_normal((c, f)) * 0.05)
    pre = oracle.round_bf16(rng.standard_normal((m, f)) * 2.0)
    h = oracle.round_bf16(oracle.gelu(pre))
    dyd, wd, pre_d, hd = dev_bf16(dy), dev_bf16(w), dev_bf16(pre), dev_bf16(h)
    dpre = torch.empty(m, f, device=DEV, dtype=torch.bfloat16)
    dw = torch.zeros(c, f, device=DEV)
    db = torch.zeros(c, device=DEV)
    d_dx = L.make_desc(dpre, dyd, wd, False, False, gelu_bwd_of=pre_d)
    d_dw = L.make_desc(dw, dyd, hd, True, False, beta=1.0, dbias=db, dbias_beta=1.0)
    grp = L.Group([(d_dx, dpre, dyd, wd), (d_dw, dw, dyd, hd)])
    bufs = [torch.empty(max(n, 256), dtype=torch.uint8, device=DEV) for n in grp.workspace_bytes()]
    grp.set_workspaces(bufs)
    grp.run()
    L.device_status()
    rows = rng.choice(m, 32, replace=False)
    want = oracle.gemm(dy[rows], w) * oracle.gelu_bwd(pre[rows])
    assert oracle.rel_fro(host(dpre)[rows], want) <= 4e-3
    crows = rng.choice(c, 16, replace=False)
    assert oracle.rel_fro(host(dw)[crows], oracle.gemm(np.ascontiguousarray(dy[:, crows]), h, True, False)) <= 1e-3
    assert oracle.rel_fro(host(db), oracle.rowsum(dy, trans_a=True)) <= 1e-3


def test_gelu_bwd_flag_is_checked():
    a = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    c = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    d = L.make_desc(c, a, a, False, False, gelu_bwd_of=c.clone())
    d.aux = None
    with pytest.raises(L.LlmtB200Error, match="aux is null"):
        L.gemm_desc(d, c, a, a)
    d = L.make_desc(c, a, a, False, False, gelu_bwd_of=c.clone())
    d.epilogue |= L.EPI_GELU
    with pytest.raises(L.LlmtB200Error, match="stands alone"):
        L.gemm_desc(d, c, a, a)
    af = torch.zeros(64, 64, device=DEV)
    cf = torch.zeros(64, 64, device=DEV)
    d = L.make_desc(cf, af, af, False, False, gelu_bwd_of=cf.clone())
    with pytest.raises(L.LlmtB200Error, match="bf16 operands"):
        L.gemm_desc(d, cf, af, af)


@pytest.mark.parametrize("m,f,c,out", [(256, 512, 128, torch.bfloat16), (300, 1000, 192, torch.bfloat16),
                                       (2048, 3072, 768, torch.bfloat16), (200, 264, 64, torch.float32)])
def test_forward_keeps_the_pre_activation(m, f, c, out):
    """h = gelu(x W^T + b) and pre = x W^T + b from one launch; h must equal the launch without
    the second result bit for bit, pre must equal the bias-only launch bit for bit."""
    rng = np.random.default_rng(m * 3 + f + c)
    x = oracle.round_bf16(rng.standard_normal((m, c)))
    w = oracle.round_bf16(rng.standard_normal((f, c)) * 0.05)
    bias = (rng.standard_normal(f) * 0.1).astype(np.float32)
    xd, wd, bd = dev_bf16(x), dev_bf16(w), torch.from_numpy(bias).to(DEV)
    h = torch.full((m, f), float("nan"), device=DEV, dtype=out)
    pre = torch.full((m, f), float("nan"), device=DEV, dtype=out)
    d = L.make_desc(h, xd, wd, False, True, bias=bd, gelu=True, save_pre=pre)
    ws = torch.empty(max(L.workspace_bytes(d, xd, wd), 256), dtype=torch.uint8, device=DEV)
    d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
    L.gemm_desc(d, h, xd, wd)
    L.device_status()
    h_only = torch.empty_like(h)
    L.gemm(h_only, xd, wd, False, True, bias=bd, gelu=True)
    pre_only = torch.empty_like(pre)
    L.gemm(pre_only, xd, wd, False, True, bias=bd)
    assert torch.equal(pre, pre_only)
    assert torch.equal(h, h_only)
    want_pre = oracle.gemm(x, w, False, True) + bias.astype(np.float64)
    assert oracle.rel_fro(host(pre), want_pre) <= (4e-3 if out == torch.bfloat16 else 1e-5)
    assert oracle.rel_fro(host(h), oracle.gelu(want_pre)) <= (4e-3 if out == torch.bfloat16 else 1e-5)


def test_mlp_forward_and_backward_chain():
    """x -> fc (+bias, GELU, pre kept) -> proj; backward: proj's dX through the GELU in one launch
    with proj's dW, then fc's dX and dW: against the oracle's chain on the same bf16 tensors."""
    m, c, f = 512, 256, 1024
    rng = np.random.default_rng(77)
    x = oracle.round_bf16(rng.standard_normal((m, c)))
    w1 = oracle.round_bf16(rng.standard_normal((f, c)) * 0.05)
    b1 = (rng.standard_normal(f) * 0.1).astype(np.float32)
    w2 = oracle.round_bf16(rng.standard_normal((c, f)) * 0.05)
    dy = oracle.round_bf16(rng.standard_normal((m, c)) * 0.1)
    xd, w1d, w2d, dyd, b1d = dev_bf16(x), dev_bf16(w1), dev_bf16(w2), dev_bf16(dy), torch.from_numpy(b1).to(DEV)
    bf = torch.bfloat16
    h = torch.empty(m, f, device=DEV, dtype=bf)
    pre = torch.empty(m, f, device=DEV, dtype=bf)
    d = L.make_desc(h, xd, w1d, False, True, bias=b1d, gelu=True, save_pre=pre)
    L.gemm_desc(d, h, xd, w1d)
    y = torch.empty(m, c, device=DEV, dtype=bf)
    L.gemm(y, h, w2d, False, True)
    dpre = torch.empty(m, f, device=DEV, dtype=bf)
    dw2 = torch.zeros(c, f, device=DEV)
    grp = L.Group([(L.make_desc(dpre, dyd, w2d, False, False, gelu_bwd_of=pre), dpre, dyd, w2d),
                   (L.make_desc(dw2, dyd, h, True, False, beta=1.0), dw2, dyd, h)])
    bufs = [torch.empty(max(n, 256), dtype=torch.uint8, device=DEV) for n in grp.workspace_bytes()]
    grp.set_workspaces(bufs)
    grp.run()
    dx = torch.empty(m, c, device=DEV, dtype=bf)
    dw1 = torch.zeros(f, c, device=DEV)
    db1 = torch.zeros(f, device=DEV)
    L.gemm(dx, dpre, w1d, False, False)
    L.gemm(dw1, dpre, xd, True, False, beta=1.0, dbias=db1, dbias_beta=1.0)
    L.device_status()
    # the oracle's chain, rounding where the device stores bf16
    pre_r = oracle.gemm(x, w1, False, True) + b1.astype(np.float64)
    pre_b = oracle.round_bf16(pre_r)
    h_b = oracle.round_bf16(oracle.gelu(pre_r))
    assert oracle.rel_fro(host(y), oracle.gemm(h_b, w2, False, True)) <= 6e-3
    dpre_r = oracle.gemm(dy, w2) * oracle.gelu_bwd(pre_b)
    assert oracle.rel_fro(host(dpre), dpre_r) <= 6e-3
    dpre_b = host(dpre)
    assert oracle.rel_fro(host(dx), oracle.gemm(dpre_b, w1)) <= 6e-3
    assert oracle.rel_fro(host(dw1), oracle.gemm(dpre_b, x, True, False)) <= 1e-3
    assert oracle.rel_fro(host(db1), oracle.rowsum(dpre_b, trans_a=True)) <= 1e-3
    assert oracle.rel_fro(host(dw2), oracle.gemm(dy, host(h), True, False)) <= 1e-3
