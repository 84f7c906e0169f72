"""The consumer of the LM-head logits: cross-entropy forward, from logits in memory (llmt's
cross_entropy_fwd) and fused into the LM-head GEMM's epilogue (no [rows, vocab] tensor)."""
import numpy as np
import pytest
import torch

import llmt_b200 as L
from oracle import oracle
from tests.support import GoldenCase, assert_close

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _ce(logits, targets, mask):
    rows = targets.numel()
    loss = torch.empty(1, device=DEV)
    nll = torch.empty(rows, device=DEV)
    L.cross_entropy_fwd(loss, nll, logits, targets, mask)
    L.device_status()
    return loss.cpu().numpy(), nll.cpu().numpy()


def test_cross_entropy_matches_llmt_golden_and_reruns_bitwise():
    # llmt tests/unit/test_cross_entropy.cu:19-54, same tolerance (1e-5 / 1e-6)
    g = GoldenCase("cross_entropy")
    logits = torch.from_numpy(g.tensor("logits")).to(DEV)
    targets = torch.from_numpy(g.tensor("targets")).to(DEV)
    mask = torch.from_numpy(g.tensor("mask")).to(DEV)
    loss, nll = _ce(logits, targets, mask)
    assert_close(nll.reshape(2, 4), g.tensor("wnll"), what="row_nll")
    assert_close(loss, g.tensor("loss"), what="loss")
    loss2, nll2 = _ce(logits, targets, mask)
    assert loss.tobytes() == loss2.tobytes() and nll.tobytes() == nll2.tobytes()


@pytest.mark.parametrize("rows,vocab", [(1, 1), (7, 33), (64, 50257), (300, 1000)])
def test_cross_entropy_against_the_oracle(rows, vocab):
    rng = np.random.default_rng(rows * 131 + vocab)
    x = (rng.standard_normal((rows, vocab)) * 3.0).astype(np.float32)
    x[0, :] += 80.0  # a row whose exponentials would overflow without the maximum
    t = rng.integers(0, vocab, size=rows).astype(np.int32)
    w = rng.random(rows).astype(np.float32)
    w[rows // 2] = 0.0 if rows > 1 else 1.0
    loss, nll = _ce(torch.from_numpy(x).to(DEV), torch.from_numpy(t).to(DEV), torch.from_numpy(w).to(DEV))
    want_loss, want_nll = oracle.cross_entropy(x, t, w)
    assert_close(nll, want_nll, rtol=1e-5, atol=1e-5, what="row_nll")
    assert_close(loss, np.array([want_loss]), rtol=1e-5, atol=1e-6, what="loss")


@pytest.mark.parametrize("m,vocab,k,store", [(256, 512, 128, True), (300, 1000, 192, False),
                                             (1024, 50257, 768, False), (1024, 50257, 768, True)])
def test_lm_head_with_fused_cross_entropy(m, vocab, k, store):
    """logits = X W^T (+ bias) never has to exist: the loss and the per-row NLL from the GEMM's epilogue
    against the fp64 oracle on the same bf16-rounded operands; with `store` the logits are written
    too and must equal a plain GEMM bit for bit."""
    rng = np.random.default_rng(m + vocab + k)
    x = oracle.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    w = oracle.round_bf16((rng.standard_normal((vocab, k)) * 0.2).astype(np.float32))
    bias = (rng.standard_normal(vocab) * 0.5).astype(np.float32)
    t = rng.integers(0, vocab, size=m).astype(np.int32)
    msk = rng.random(m).astype(np.float32)
    xd = torch.from_numpy(x).to(DEV).to(torch.bfloat16)
    wd = torch.from_numpy(w).to(DEV).to(torch.bfloat16)
    bd = torch.from_numpy(bias).to(DEV)
    td, md = torch.from_numpy(t).to(DEV), torch.from_numpy(msk).to(DEV)
    logits = torch.empty(m, vocab, device=DEV) if store else None
    # the descriptor by hand: C dtype fp32, contiguous pitch
    d = L.GemmDesc()
    d.m, d.n, d.k, d.batch = m, vocab, k, 1
    d.lda, d.ldb, d.ldc = k, k, vocab
    d.trans_a, d.trans_b = 0, 1
    d.dtype_ab, d.dtype_c = L.BF16, L.FP32
    d.alpha, d.beta = 1.0, 0.0
    d.epilogue, d.bias, d.bias_dtype = L.EPI_BIAS, bd.data_ptr(), L.FP32
    need = L.lm_head_ce_workspace_bytes(d, xd, wd)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    loss = torch.empty(1, device=DEV)
    nll = torch.empty(m, device=DEV)
    L.lm_head_ce_fwd(d, logits, xd, wd, td, md, nll, loss)
    L.device_status()
    ref_logits = oracle.gemm(x, w, False, True) + bias.astype(np.float64)
    want_loss, want_nll = oracle.cross_entropy(ref_logits, t, msk)
    assert_close(nll.cpu().numpy(), want_nll, rtol=2e-4, atol=2e-4, what="row_nll")
    assert_close(loss.cpu().numpy(), np.array([want_loss]), rtol=1e-4, atol=1e-5, what="loss")
    # a second run: the same bits
    loss2, nll2 = torch.empty(1, device=DEV), torch.empty(m, device=DEV)
    L.lm_head_ce_fwd(d, logits, xd, wd, td, md, nll2, loss2)
    assert torch.equal(loss, loss2) and torch.equal(nll, nll2)
    if store:
        plain = torch.empty(m, vocab, device=DEV)
        L.gemm(plain, xd, wd, False, True, bias=bd)
        assert torch.equal(plain, logits)
        # and llmt's cross_entropy_fwd on those logits agrees with the fused result
        l3, n3 = _ce(logits, td, md)
        assert_close(nll.cpu().numpy(), n3, rtol=1e-5, atol=1e-5, what="fused vs from-memory row_nll")


def test_lm_head_ce_refuses_what_it_cannot_do():
    d = L.GemmDesc()
    d.m, d.n, d.k, d.batch = 64, 64, 64, 1
    d.lda, d.ldb, d.ldc = 64, 64, 64
    d.trans_b = 1
    d.dtype_ab, d.dtype_c = L.FP32, L.FP32
    d.alpha = 1.0
    x = torch.zeros(64, 64, device=DEV)
    t = torch.zeros(64, dtype=torch.int32, device=DEV)
    o = torch.zeros(64, device=DEV)
    with pytest.raises(L.LlmtB200Error) as ei:
        L.lm_head_ce_fwd(d, None, x, x, t, o, o, o)
    assert ei.value.status == L.ERR_UNSUPPORTED
    d.dtype_ab = L.BF16
    xb = x.to(torch.bfloat16)
    with pytest.raises(L.LlmtB200Error) as ei:
        L.lm_head_ce_fwd(d, None, xb, xb, t, o, o, o)  # no workspace
    assert ei.value.status == L.ERR_WORKSPACE


@pytest.mark.parametrize("rows,vocab,in_place", [(1, 1, True), (7, 33, False), (64, 50257, True), (300, 1000, False)])
def test_cross_entropy_bwd_against_the_oracle(rows, vocab, in_place):
    """llmt's planned cross_entropy_bwd (docs/TODO.md:216-217): (softmax - onehot) * mask / sum(mask),
    in place of the logits or into another tensor."""
    rng = np.random.default_rng(rows * 7 + vocab)
    x = (rng.standard_normal((rows, vocab)) * 3.0).astype(np.float32)
    x[0, :] += 80.0
    t = rng.integers(0, vocab, size=rows).astype(np.int32)
    w = rng.random(rows).astype(np.float32) + 0.1
    w[rows // 2] = 0.0 if rows > 1 else 1.0
    xd = torch.from_numpy(x).to(DEV)
    out = xd if in_place else torch.full_like(xd, float("nan"))
    L.cross_entropy_bwd(out, xd, torch.from_numpy(t).to(DEV), torch.from_numpy(w).to(DEV), dloss=0.5)
    L.device_status()
    want = oracle.cross_entropy_bwd(x, t, w, dloss=0.5)
    assert_close(out.cpu().numpy(), want, rtol=5e-5, atol=1e-7, what="dlogits")


@pytest.mark.parametrize("m,vocab,k,out_dtype,reuse", [(256, 512, 128, torch.bfloat16, True), (300, 1000, 192, torch.float32, False),
                                                       (1024, 50257, 768, torch.bfloat16, True)])
def test_lm_head_dlogits_from_the_product(m, vocab, k, out_dtype, reuse):
    """dLogits of the LM head's cross-entropy without logits in memory: the product made again,
    leaving as (softmax - onehot) * weight.  `reuse`: the statistics of the forward call are still
    in the workspace and the statistics pass is skipped; both ways must give the same bits."""
    rng = np.random.default_rng(m + vocab + k + 1)
    x = oracle.round_bf16(rng.standard_normal((m, k)).astype(np.float32))
    w = oracle.round_bf16((rng.standard_normal((vocab, k)) * 0.2).astype(np.float32))
    t = rng.integers(0, vocab, size=m).astype(np.int32)
    msk = rng.random(m).astype(np.float32)
    xd = torch.from_numpy(x).to(DEV).to(torch.bfloat16)
    wd = torch.from_numpy(w).to(DEV).to(torch.bfloat16)
    td, md = torch.from_numpy(t).to(DEV), torch.from_numpy(msk).to(DEV)
    ld = (vocab + 7) // 8 * 8
    dl = torch.full((m, ld), float("nan"), device=DEV, dtype=out_dtype)[:, :vocab]
    d = L.GemmDesc()
    d.m, d.n, d.k, d.batch = m, vocab, k, 1
    d.lda, d.ldb, d.ldc = k, k, ld
    d.trans_a, d.trans_b = 0, 1
    d.dtype_ab, d.dtype_c = L.BF16, (L.BF16 if out_dtype == torch.bfloat16 else L.FP32)
    d.alpha, d.beta = 1.0, 0.0
    need = L.lm_head_ce_workspace_bytes(d, xd, wd)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    d.workspace, d.workspace_bytes = ws.data_ptr(), need
    if reuse:
        loss, nll = torch.empty(1, device=DEV), torch.empty(m, device=DEV)
        L.lm_head_ce_fwd(d, None, xd, wd, td, md, nll, loss)
    L.lm_head_ce_bwd(d, dl, xd, wd, td, md, dloss=1.0, stats_valid=reuse)
    L.device_status()
    want = oracle.cross_entropy_bwd(oracle.gemm(x, w, False, True), t, msk)
    got = dl.float().cpu().numpy()
    assert np.isfinite(got).all()
    tol = 4e-3 if out_dtype == torch.bfloat16 else 2e-4
    assert oracle.rel_fro(got, want) <= tol
    # the gradient of every row sums to zero (softmax minus one-hot), up to the result type's rounding
    assert np.abs(got.sum(-1)).max() <= (5e-3 if out_dtype == torch.bfloat16 else 1e-6)
    # the other way round gives the same bits
    dl2 = torch.full((m, ld), float("nan"), device=DEV, dtype=out_dtype)[:, :vocab]
    L.lm_head_ce_bwd(d, dl2, xd, wd, td, md, dloss=1.0, stats_valid=False)
    assert torch.equal(dl, dl2)
