"""Pins the CPU oracle against every known-answer tensor llmt's own tests hold
for the matmul path, at llmt's own tolerance (rtol 1e-5, atol 1e-6)."""
import numpy as np

from oracle import oracle
from tests.support import GoldenCase, assert_close


def test_matmul_four_transpose_combos():
    # llmt tests/unit/test_matmul.cu:20-47
    g = GoldenCase("matmul")
    a, at, b, bt = (g.tensor(n) for n in ("a", "at", "b", "bt"))
    assert_close(oracle.gemm(a, b), g.tensor("c_nn"), what="c_nn")
    assert_close(oracle.gemm(a, bt, trans_b=True), g.tensor("c_nt"), what="c_nt")
    assert_close(oracle.gemm(at, b, trans_a=True), g.tensor("c_tn"), what="c_tn")
    assert_close(oracle.gemm(at, bt, trans_a=True, trans_b=True), g.tensor("c_tt"), what="c_tt")


def test_matmul_beta_accumulates():
    # llmt tests/unit/test_matmul.cu:49-62
    g = GoldenCase("matmul")
    c = oracle.gemm(g.tensor("a"), g.tensor("b"), beta=1.0, c=g.tensor("c0"))
    assert_close(c, g.tensor("c_beta"), what="c_beta")


def test_matmul_rank3():
    # llmt tests/unit/test_matmul.cu:64-84
    g = GoldenCase("matmul_rank3")
    assert_close(oracle.gemm(g.tensor("a"), g.tensor("b")), g.tensor("c"), what="c")
    assert_close(oracle.gemm(g.tensor("q"), g.tensor("k"), trans_b=True), g.tensor("scores"),
                 what="scores")


def test_linear_forward_backward_accumulate():
    # llmt tests/unit/test_linear.cu:19-57 ; operand roles from src/layers/linear.cpp:16-30
    g = GoldenCase("linear")
    x, w, dy = g.tensor("x"), g.tensor("weight"), g.tensor("dy")
    assert_close(oracle.gemm(x, w, trans_b=True), g.tensor("y"), what="y")
    assert_close(oracle.gemm(dy, w), g.tensor("dx"), what="dx")
    dw = oracle.gemm(dy, x, trans_a=True, beta=1.0, c=np.zeros_like(w))
    assert_close(dw, g.tensor("dw"), what="dw")
    dw2 = oracle.gemm(dy, x, trans_a=True, beta=1.0, c=dw)
    assert_close(dw2, 2.0 * g.tensor("dw").astype(np.float64), what="dw twice")


def test_mlp_forward():
    # llmt tests/unit/test_mlp.cu:16-42 ; src/layers/mlp.cpp:14-18
    g = GoldenCase("mlp")
    h = oracle.epilogue(oracle.gemm(g.tensor("x"), g.tensor("wu"), trans_b=True), gelu=True)
    y = oracle.gemm(h.astype(np.float32), g.tensor("wd"), trans_b=True)
    assert_close(y, g.tensor("y"), what="mlp y")


def test_gelu_formula():
    # llmt tests/unit/test_kernels_fwd.cu:74-89 ; src/kernels/gelu.cu:23-26
    g = GoldenCase("gelu")
    assert_close(oracle.gelu(g.tensor("x")), g.tensor("y"), what="gelu")
    x = g.tensor("x")
    via_c = oracle.epilogue(x.astype(np.float64), gelu=True)
    assert_close(via_c, g.tensor("y"), what="gelu via oracle.c")


def test_attention_stages():
    # llmt tests/unit/test_attention.cu:58-99 ; src/kernels/attention.cpp:54-62
    g = GoldenCase("attention")
    q, k, v = (g.tensor(n) for n in ("q", "k", "v"))
    B, H, T, hd = q.shape
    q3, k3, v3 = (t.reshape(B * H, T, hd) for t in (q, k, v))
    scores = oracle.gemm(q3, k3, trans_b=True, alpha=1.0 / np.sqrt(np.float32(hd)))
    assert_close(scores.reshape(B, H, T, T), g.tensor("scores"), what="scores")
    probs = oracle.softmax(scores, causal=True)
    assert_close(probs.reshape(B, H, T, T), g.tensor("probs"), what="probs")
    assert (probs[:, np.triu_indices(T, 1)[0], np.triu_indices(T, 1)[1]] == 0.0).all()
    out = oracle.gemm(probs.astype(np.float32), v3)
    assert_close(out.reshape(B, H, T, hd), g.tensor("out"), what="out")
    merged = out.reshape(B, H, T, hd).transpose(0, 2, 1, 3).reshape(B, T, H * hd)
    assert_close(merged, g.tensor("merged"), what="merged")


def test_softmax_bwd_matches_finite_difference():
    rng = np.random.default_rng(3)
    s = rng.standard_normal((2, 5, 5))
    dp = rng.standard_normal((2, 5, 5))
    p = oracle.softmax(s, causal=False)
    ds = oracle.softmax_bwd(p, dp)
    eps = 1e-6
    num = np.zeros_like(s)
    for idx in np.ndindex(*s.shape):
        sp = s.copy(); sp[idx] += eps
        sm = s.copy(); sm[idx] -= eps
        num[idx] = ((oracle.softmax(sp, False) - oracle.softmax(sm, False)) * dp).sum() / (2 * eps)
    assert np.allclose(ds, num, rtol=1e-5, atol=1e-8)


def test_bf16_rounding_is_rne():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.0e38, 1e-40, 0.0], np.float32)
    r = oracle.round_bf16(x)
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7: ties to even -> 1.0
    assert r[0] == 1.0 and r[1] == 1.0
    # 1 + 3*2^-8 is a tie between 1+2^-7 (odd) and 1+2^-6 (even) -> 1 + 2^-6
    assert r[2] == np.float32(1.015625)
    bits = r.view(np.uint32)
    assert (bits & 0xFFFF == 0).all()


def test_f32_port_matches_f64():
    rng = np.random.default_rng(0)
    a = rng.standard_normal((37, 53)).astype(np.float32)
    b = rng.standard_normal((29, 53)).astype(np.float32)
    ref = oracle.gemm(a, b, trans_b=True)
    got = oracle.gemm_f32(a, b, trans_b=True)
    assert oracle.rel_fro(got, ref) < 1e-6
    at = np.ascontiguousarray(a.T)
    bn = np.ascontiguousarray(b.T)
    got2 = oracle.gemm_f32(at, bn, trans_a=True, trans_b=False)
    assert oracle.rel_fro(got2, ref) < 1e-6


def test_oracle_cross_entropy_matches_llmt_golden():
    # the consumer of the LM-head logits: llmt tests/unit/test_cross_entropy.cu:19-35
    g = GoldenCase("cross_entropy")
    loss, nll = oracle.cross_entropy(g.tensor("logits"), g.tensor("targets"), g.tensor("mask"))
    assert_close(nll, g.tensor("wnll"), what="cross_entropy row_nll")
    assert_close(np.array([loss]), g.tensor("loss"), what="cross_entropy loss")


def test_oracle_cross_entropy_bwd_matches_torch_autograd():
    # llmt has no cross_entropy_bwd yet (docs/TODO.md:216-217 gives the formula); its golden
    # generator differentiates through torch, so the oracle is pinned against torch autograd on
    # llmt's own cross_entropy inputs and on a larger seeded case.
    import torch
    g = GoldenCase("cross_entropy")
    cases = [(g.tensor("logits"), g.tensor("targets"), g.tensor("mask"))]
    rng = np.random.default_rng(3)
    cases.append(((rng.standard_normal((3, 5, 97)) * 4).astype(np.float32), rng.integers(0, 97, (3, 5)).astype(np.int32),
                  rng.random((3, 5)).astype(np.float32)))
    for logits, targets, mask in cases:
        x = torch.tensor(logits, dtype=torch.float64, requires_grad=True)
        v = x.shape[-1]
        nll = torch.nn.functional.cross_entropy(x.reshape(-1, v), torch.tensor(targets).reshape(-1).long(), reduction="none")
        w = torch.tensor(mask, dtype=torch.float64).reshape(-1)
        loss = (nll * w).sum() / w.sum()
        loss.backward()
        got = oracle.cross_entropy_bwd(logits, targets, mask)
        assert_close(got, x.grad.numpy(), rtol=1e-9, atol=1e-12, what="cross_entropy_bwd")
        got2 = oracle.cross_entropy_bwd(logits, targets, mask, dloss=0.5)
        assert_close(got2, 0.5 * x.grad.numpy(), rtol=1e-9, atol=1e-12, what="cross_entropy_bwd scaled")


def test_oracle_gelu_bwd_matches_torch_autograd():
    # llmt plans gelu_bwd (docs/TODO.md:223); its goldens come from torch, so the oracle's derivative
    # of the tanh-GELU is pinned against torch autograd.
    import torch
    x = torch.linspace(-8.0, 8.0, 4001, dtype=torch.float64, requires_grad=True)
    torch.nn.functional.gelu(x, approximate="tanh").sum().backward()
    assert_close(oracle.gelu_bwd(x.detach().numpy()), x.grad.numpy(), rtol=1e-12, atol=1e-14, what="gelu_bwd")
