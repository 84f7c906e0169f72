"""Parity of the CUDA path (called through the C ABI) against the CPU oracle,
llmt's golden tensors and — where it was built — the unmodified llmt library.

Tolerances (stated once, used below):
  * strict fp32 path vs llmt goldens: llmt's own rtol 1e-5 / atol 1e-6 elementwise;
    vs the fp64 oracle on larger cases: relative Frobenius <= 1e-5.
  * bf16 inputs, fp32 accumulation, fp32 output vs the fp64 product of the same
    bf16-rounded inputs: relative Frobenius <= 1e-3 (observed ~1e-6).
  * bf16 output: relative Frobenius <= 4e-3 (rounding the exact result to bf16 is
    itself ~1.7e-3 away) and >= 99.9 % of elements within one bf16 ulp of
    round_bf16(oracle).
"""
import numpy as np
import pytest
import torch

import llmt_b200 as L
from oracle import llmt_ref, oracle
from tests.support import GoldenCase, assert_close

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL_F32_FRO = 1e-5
TOL_BF16_ACC_FRO = 1e-3
TOL_BF16_OUT_FRO = 4e-3


def dev_f32(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(DEV)


def dev_bf16(x):
    return dev_f32(x).to(torch.bfloat16)


def host(t):
    return t.float().cpu().numpy()


def bf16_ulp_ok_fraction(got, ref64):
    """Fraction of elements within one bf16 ulp of round_bf16(ref)."""
    want = oracle.round_bf16(ref64.astype(np.float32))
    ulp = np.maximum(np.abs(want), 2.0 ** -126) * 2.0 ** -7
    return float((np.abs(got.astype(np.float64) - want) <= ulp).mean())


@pytest.fixture(autouse=True)
def _healthy_device():
    yield
    assert L.device_status() == (0, 0)


# --------------------------------------------------------------- strict fp32 ---

def test_fp32_llmt_golden_matmul():
    # llmt tests/unit/test_matmul.cu:20-62
    g = GoldenCase("matmul")
    a, at, b, bt = (dev_f32(g.tensor(n)) for n in ("a", "at", "b", "bt"))
    c = torch.empty(7, 9, device=DEV)
    for ta, tb, x, y, name in [(0, 0, a, b, "c_nn"), (0, 1, a, bt, "c_nt"),
                               (1, 0, at, b, "c_tn"), (1, 1, at, bt, "c_tt")]:
        L.gemm(c, x, y, bool(ta), bool(tb))
        assert_close(host(c), g.tensor(name), what=name)
    c = dev_f32(g.tensor("c0"))
    L.gemm(c, a, b, beta=1.0)
    assert_close(host(c), g.tensor("c_beta"), what="c_beta")


def test_fp32_llmt_golden_rank3():
    # llmt tests/unit/test_matmul.cu:64-84
    g = GoldenCase("matmul_rank3")
    c = torch.empty(3, 4, 5, device=DEV)
    L.gemm(c, dev_f32(g.tensor("a")), dev_f32(g.tensor("b")))
    assert_close(host(c), g.tensor("c"), what="c")
    s = torch.empty(3, 4, 4, device=DEV)
    L.gemm(s, dev_f32(g.tensor("q")), dev_f32(g.tensor("k")), trans_b=True)
    assert_close(host(s), g.tensor("scores"), what="scores")


def test_fp32_llmt_golden_linear_accumulates():
    # llmt tests/unit/test_linear.cu:19-57 (operand roles: src/layers/linear.cpp:16-30)
    g = GoldenCase("linear")
    x, w, dy = (dev_f32(g.tensor(n)) for n in ("x", "weight", "dy"))
    y = torch.empty(8, 10, device=DEV)
    dx = torch.empty(8, 12, device=DEV)
    dw = torch.zeros(10, 12, device=DEV)
    L.gemm(y, x, w, trans_b=True)
    L.gemm(dx, dy, w)
    L.gemm(dw, dy, x, trans_a=True, beta=1.0)
    assert_close(host(y), g.tensor("y"), what="y")
    assert_close(host(dx), g.tensor("dx"), what="dx")
    assert_close(host(dw), g.tensor("dw"), what="dw")
    L.gemm(dw, dy, x, trans_a=True, beta=1.0)
    assert_close(host(dw), 2.0 * g.tensor("dw"), what="dw twice")


def test_fp32_llmt_golden_mlp_fused_gelu():
    # llmt tests/unit/test_mlp.cu:16-42; GELU runs in the up-projection's epilogue here
    g = GoldenCase("mlp")
    x, wu, wd = (dev_f32(g.tensor(n)) for n in ("x", "wu", "wd"))
    h = torch.empty(6, 16, device=DEV)
    y = torch.empty(6, 8, device=DEV)
    L.gemm(h, x, wu, trans_b=True, gelu=True)
    L.gemm(y, h, wd, trans_b=True)
    assert_close(host(y), g.tensor("y"), what="mlp y")


def test_fp32_llmt_golden_attention_stages():
    # llmt tests/unit/test_attention.cu:58-99
    g = GoldenCase("attention")
    q, k, v = (dev_f32(g.tensor(n).reshape(4, 4, 6)) for n in ("q", "k", "v"))
    s = torch.empty(4, 4, 4, device=DEV)
    L.gemm(s, q, k, trans_b=True, alpha=1.0 / np.sqrt(np.float32(6)))
    assert_close(host(s).reshape(2, 2, 4, 4), g.tensor("scores"), what="scores")
    L.softmax_fwd(s, s, causal=True)
    p = host(s).reshape(2, 2, 4, 4)
    assert_close(p, g.tensor("probs"), what="probs")
    assert (p[..., np.triu_indices(4, 1)[0], np.triu_indices(4, 1)[1]] == 0.0).all()
    o = torch.empty(4, 4, 6, device=DEV)
    L.gemm(o, s, v)
    assert_close(host(o).reshape(2, 2, 4, 6), g.tensor("out"), what="out")


def test_fp32_config1_linear_with_bias():
    # BASELINE config 1: Y = X W^T + b, X[256,768] ~ N(0,1), W[3072,768], b ~ N(0,0.02), seed 0
    rng = np.random.default_rng(0)
    x = rng.standard_normal((256, 768)).astype(np.float32)
    w = (rng.standard_normal((3072, 768)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(3072) * 0.02).astype(np.float32)
    y = torch.empty(256, 3072, device=DEV)
    L.gemm(y, dev_f32(x), dev_f32(w), trans_b=True, bias=dev_f32(b))
    ref = oracle.epilogue(oracle.gemm(x, w, trans_b=True), bias=b)
    assert oracle.rel_fro(host(y), ref) <= TOL_F32_FRO


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_fp32_ragged_all_transposes(ta, tb):
    rng = np.random.default_rng(10 + 2 * ta + tb)
    m, n, k, batch = 67, 130, 45, 3
    a = rng.standard_normal((batch, k, m) if ta else (batch, m, k)).astype(np.float32)
    b = rng.standard_normal((batch, n, k) if tb else (batch, k, n)).astype(np.float32)
    c0 = rng.standard_normal((batch, m, n)).astype(np.float32)
    c = dev_f32(c0)
    L.gemm(c, dev_f32(a), dev_f32(b), bool(ta), bool(tb), alpha=0.75, beta=-0.5)
    ref = oracle.gemm(a, b, bool(ta), bool(tb), 0.75, -0.5, c0)
    assert oracle.rel_fro(host(c), ref) <= TOL_F32_FRO


@pytest.mark.skipif(not llmt_ref.available(), reason="llmt itself was not compiled (make -C oracle ref)")
def test_fp32_matches_unmodified_llmt_on_gpu():
    """The real llmt (cuBLASLt, strict fp32) and this library on the same seeded inputs."""
    ref_lib = llmt_ref.Llmt(0)
    rng = np.random.default_rng(5)
    x = dev_f32(rng.standard_normal((256, 768)))
    w = dev_f32(rng.standard_normal((3072, 768)) * 0.02)
    dy = dev_f32(rng.standard_normal((256, 3072)) * 0.01)
    y_ref, dx_ref, dw_ref = ref_lib.linear(w, x, dy, backward_calls=2)
    y = torch.empty_like(y_ref); dx = torch.empty_like(dx_ref); dw = torch.zeros_like(dw_ref)
    L.gemm(y, x, w, trans_b=True)
    L.gemm(dx, dy, w)
    L.gemm(dw, dy, x, trans_a=True, beta=1.0)
    L.gemm(dw, dy, x, trans_a=True, beta=1.0)
    torch.cuda.synchronize()
    for got, want, name in [(y, y_ref, "y"), (dx, dx_ref, "dx"), (dw, dw_ref, "dw")]:
        assert oracle.rel_fro(host(got), host(want)) <= TOL_F32_FRO, name
    ref_lib.close()


# ------------------------------------------------------------ bf16 tensor path ---

def _bf16_case(m, n, k, ta, tb, seed, batch=0, scale_b=0.5):
    rng = np.random.default_rng(seed)
    bs = (batch,) if batch else ()
    a = oracle.round_bf16(rng.standard_normal(bs + ((k, m) if ta else (m, k))))
    b = oracle.round_bf16(rng.standard_normal(bs + ((n, k) if tb else (k, n))) * scale_b)
    return a, b, rng


@pytest.mark.parametrize("tile_n", [64, 128, 192, 256])
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
def test_bf16_all_transposes_all_tiles_ragged(ta, tb, tile_n):
    # ragged in m, n and k: 1, tile-1, tile+1 style extents
    m, n, k = 264, 2 * tile_n + 8, 200   # not multiples of the 128 x tile_n x 64 tile
    a, b, _ = _bf16_case(m, n, k, ta, tb, seed=100 + tile_n + 2 * ta + tb)
    c = torch.empty(m, n, device=DEV)
    L.gemm(c, dev_bf16(a), dev_bf16(b), bool(ta), bool(tb), tile_n=tile_n)
    ref = oracle.gemm(a, b, bool(ta), bool(tb))
    assert oracle.rel_fro(host(c), ref) <= TOL_BF16_ACC_FRO


@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (7, 16, 8), (127, 72, 64), (129, 264, 72), (128, 256, 64)])
def test_bf16_small_and_edge_extents(m, n, k):
    a, b, _ = _bf16_case(m, n, k, 0, 1, seed=m * 1000 + n)
    c = torch.empty(m, n, device=DEV)
    L.gemm(c, dev_bf16(a), dev_bf16(b), False, True)
    assert oracle.rel_fro(host(c), oracle.gemm(a, b, False, True)) <= TOL_BF16_ACC_FRO


def test_bf16_padded_pitches():
    """Row pitches larger than the row (the aligned-vocabulary layout of the LM head)."""
    m, n, k = 200, 257, 136
    a, b, rng = _bf16_case(m, n, k, 0, 1, seed=7)
    a_buf = torch.zeros(m, 144, device=DEV, dtype=torch.bfloat16); a_buf[:, :k] = dev_bf16(a)
    b_buf = torch.zeros(n, 152, device=DEV, dtype=torch.bfloat16); b_buf[:, :k] = dev_bf16(b)
    c_buf = torch.full((m, 264), 7.0, device=DEV)
    L.gemm(c_buf[:, :n], a_buf[:, :k], b_buf[:, :k], False, True)
    got = host(c_buf)
    assert oracle.rel_fro(got[:, :n], oracle.gemm(a, b, False, True)) <= TOL_BF16_ACC_FRO
    assert (got[:, n:] == 7.0).all(), "padding columns of C must not be written"


@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0)])
def test_bf16_unaligned_pitches_are_repacked(ta, tb):
    """Operands whose pitch is not a multiple of 8 elements (TMA cannot address them) are
    copied into the workspace with a padded pitch first; C with an odd pitch is written
    straight from registers."""
    m, n, k = 257, 203, 137  # every pitch is odd
    a, b, _ = _bf16_case(m, n, k, ta, tb, seed=71 + 2 * ta + tb)
    c = torch.full((m, n), -1.0, device=DEV)
    ad, bd = dev_bf16(a), dev_bf16(b)
    d = L.make_desc(c, ad, bd, bool(ta), bool(tb))
    need = L.workspace_bytes(d)
    assert need >= 2 * (a.size + b.size)  # both operands get an aligned copy
    with pytest.raises(L.LlmtB200Error) as e:
        L.gemm_desc(d, c, ad, bd)        # no scratch handed in
    assert e.value.status == L.ERR_WORKSPACE
    L.gemm(c, ad, bd, bool(ta), bool(tb))  # the wrapper allocates the scratch
    assert oracle.rel_fro(host(c), oracle.gemm(a, b, bool(ta), bool(tb))) <= TOL_BF16_ACC_FRO


def test_bf16_unaligned_batch_stride():
    batch, m, n, k = 3, 64, 72, 40
    rng = np.random.default_rng(73)
    a = oracle.round_bf16(rng.standard_normal((batch, m, k)))
    b = oracle.round_bf16(rng.standard_normal((batch, n, k)))
    # batch items 4 elements further apart than one matrix: stride not a multiple of 8
    abuf = torch.zeros(batch * (m * k + 4), device=DEV, dtype=torch.bfloat16)
    av = abuf.as_strided((batch, m, k), (m * k + 4, k, 1))
    av.copy_(dev_bf16(a))
    c = torch.empty(batch, m, n, device=DEV)
    L.gemm(c, av, dev_bf16(b), False, True)
    assert oracle.rel_fro(host(c), oracle.gemm(a, b, False, True)) <= TOL_BF16_ACC_FRO


def test_bf16_output_rounding_and_ulp():
    m, n, k = 512, 768, 768
    a, b, _ = _bf16_case(m, n, k, 0, 1, seed=11, scale_b=0.02)
    c = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    L.gemm(c, dev_bf16(a), dev_bf16(b), False, True)
    ref = oracle.gemm(a, b, False, True)
    assert oracle.rel_fro(host(c), ref) <= TOL_BF16_OUT_FRO
    assert bf16_ulp_ok_fraction(host(c), ref) >= 0.999


@pytest.mark.parametrize("cdt", [torch.float32, torch.bfloat16])
def test_bf16_alpha_beta_in_place(cdt):
    m, n, k = 300, 520, 192
    a, b, rng = _bf16_case(m, n, k, 0, 1, seed=13)
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    if cdt == torch.bfloat16:
        c0 = oracle.round_bf16(c0)
    c = dev_f32(c0).to(cdt)
    L.gemm(c, dev_bf16(a), dev_bf16(b), False, True, alpha=0.5, beta=1.0)
    ref = oracle.gemm(a, b, False, True, 0.5, 1.0, c0)
    tol = TOL_BF16_OUT_FRO if cdt == torch.bfloat16 else TOL_BF16_ACC_FRO
    assert oracle.rel_fro(host(c), ref) <= tol


@pytest.mark.parametrize("bias_dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("gelu", [False, True])
def test_bf16_fused_bias_gelu_epilogue(gelu, bias_dt):
    # epilogue order: alpha*acc + beta*C -> + bias -> tanh-GELU (llmt gelu.cu:23-26) -> cast
    m, n, k = 384, 3072 // 4 + 8, 768
    a, b, rng = _bf16_case(m, n, k, 0, 1, seed=17, scale_b=0.02)
    bias = (rng.standard_normal(n) * 0.5).astype(np.float32)
    if bias_dt == torch.bfloat16:
        bias = oracle.round_bf16(bias)
    ref = oracle.epilogue(oracle.gemm(a, b, False, True), bias=bias, gelu=gelu)
    c32 = torch.empty(m, n, device=DEV)
    L.gemm(c32, dev_bf16(a), dev_bf16(b), False, True, bias=dev_f32(bias).to(bias_dt), gelu=gelu)
    assert oracle.rel_fro(host(c32), ref) <= TOL_BF16_ACC_FRO
    c16 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    L.gemm(c16, dev_bf16(a), dev_bf16(b), False, True, bias=dev_f32(bias).to(bias_dt), gelu=gelu)
    assert oracle.rel_fro(host(c16), ref) <= TOL_BF16_OUT_FRO
    assert bf16_ulp_ok_fraction(host(c16), ref) >= 0.999


@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0)])
def test_bf16_strided_batched(ta, tb):
    # the per-head attention products of llmt attention.cpp:60-62 (NT, NN) and their TN duals
    batch, m, n, k = 6, 160, 96, 72
    a, b, _ = _bf16_case(m, n, k, ta, tb, seed=19 + ta + tb, batch=batch)
    c = torch.empty(batch, m, n, device=DEV)
    L.gemm(c, dev_bf16(a), dev_bf16(b), bool(ta), bool(tb), alpha=0.125)
    assert oracle.rel_fro(host(c), oracle.gemm(a, b, bool(ta), bool(tb), 0.125)) <= TOL_BF16_ACC_FRO


@pytest.mark.parametrize("splits", [0, 1, 3])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_bf16_dw_with_fused_dbias_on_cta_pairs(tile_n, splits):
    """The same product on CTA pairs (256-row tiles); each CTA of the pair that draws a dbias
    ticket reduces half of its rows."""
    tokens, out_f, in_f = 1024, 520, 2 * tile_n + 40
    rng = np.random.default_rng(53 + tile_n + splits)
    dy = oracle.round_bf16(rng.standard_normal((tokens, out_f)) * 0.01)
    x = oracle.round_bf16(rng.standard_normal((tokens, in_f)))
    dw0 = rng.standard_normal((out_f, in_f)).astype(np.float32)
    db0 = rng.standard_normal(out_f).astype(np.float32)
    dw, db = dev_f32(dw0), dev_f32(db0)
    L.gemm(dw, dev_bf16(dy), dev_bf16(x), trans_a=True, beta=1.0, dbias=db, dbias_beta=1.0,
           tile_n=tile_n, splits=splits, cta_pairs=2)
    assert oracle.rel_fro(host(dw), oracle.gemm(dy, x, trans_a=True, beta=1.0, c=dw0)) <= TOL_BF16_ACC_FRO
    assert oracle.rel_fro(host(db), oracle.rowsum(dy, trans_a=True, out=db0, out_beta=1.0)) <= TOL_BF16_ACC_FRO


@pytest.mark.parametrize("cta_pairs", [1, 2])
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
def test_bf16_single_cta_and_pair_kernels_agree(ta, tb, cta_pairs):
    """Both tensor-core kernels (128-row tiles on one CTA, 256-row tiles on a CTA pair) on
    every transpose combination, against the oracle."""
    m, n, k = 520, 392, 328
    a, b, _ = _bf16_case(m, n, k, ta, tb, seed=61 + 2 * ta + tb)
    c = torch.empty(m, n, device=DEV)
    L.gemm(c, dev_bf16(a), dev_bf16(b), bool(ta), bool(tb), cta_pairs=cta_pairs)
    assert oracle.rel_fro(host(c), oracle.gemm(a, b, bool(ta), bool(tb))) <= TOL_BF16_ACC_FRO


@pytest.mark.parametrize("splits", [0, 1, 3, 8])
@pytest.mark.parametrize("tile_n", [64, 128, 192, 256])
def test_bf16_dw_with_fused_dbias_and_splitk(tile_n, splits):
    # Linear backward: dW += dy^T x, dbias += sum_rows dy (llmt linear.cpp:27-29 + bias extension)
    tokens, out_f, in_f = 1024, 200, 2 * tile_n + 40
    rng = np.random.default_rng(23 + tile_n + splits)
    dy = oracle.round_bf16(rng.standard_normal((tokens, out_f)) * 0.01)
    x = oracle.round_bf16(rng.standard_normal((tokens, in_f)))
    dw0 = rng.standard_normal((out_f, in_f)).astype(np.float32)
    db0 = rng.standard_normal(out_f).astype(np.float32)
    dw, db = dev_f32(dw0), dev_f32(db0)
    L.gemm(dw, dev_bf16(dy), dev_bf16(x), trans_a=True, beta=1.0, dbias=db, dbias_beta=1.0,
           tile_n=tile_n, splits=splits)
    ref_dw = oracle.gemm(dy, x, trans_a=True, beta=1.0, c=dw0)
    ref_db = oracle.rowsum(dy, trans_a=True, out=db0, out_beta=1.0)
    assert oracle.rel_fro(host(dw), ref_dw) <= TOL_BF16_ACC_FRO
    assert oracle.rel_fro(host(db), ref_db) <= TOL_BF16_ACC_FRO


def test_bf16_bitwise_deterministic_and_scale_exact():
    """Same inputs -> same bits (llmt test_matmul.cu:86-103), with and without
    split-K; and scaling A by 2 (exact in bf16) scales C by exactly 2."""
    m, n, k = 768, 768, 4096
    a, b, _ = _bf16_case(m, n, k, 1, 0, seed=29, scale_b=0.02)
    ta, tb2 = dev_bf16(a), dev_bf16(b)
    outs = []
    for _ in range(3):
        c = torch.empty(m, n, device=DEV)
        L.gemm(c, ta, tb2, True, False)
        outs.append(c)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    c2 = torch.empty(m, n, device=DEV)
    L.gemm(c2, dev_bf16(2.0 * a), tb2, True, False)
    assert torch.equal(c2, 2.0 * outs[0])
    assert oracle.rel_fro(host(outs[0]), oracle.gemm(a, b, True, False)) <= TOL_BF16_ACC_FRO


def test_empty_reduction_and_empty_output():
    """k == 0 leaves C = beta*C (BLAS convention); m == 0 writes nothing. torch hands out
    null pointers for empty tensors, so the operands are addressed through a dummy buffer."""
    import ctypes
    dummy = torch.zeros(4096, device=DEV, dtype=torch.bfloat16)
    c = torch.full((64, 32), 3.0, device=DEV)
    d = L.GemmDesc()
    d.m, d.n, d.k, d.batch = 64, 32, 0, 1
    d.lda, d.ldb, d.ldc = 8, 8, 32
    d.trans_b = 1
    d.dtype_ab, d.dtype_c = L.BF16, L.FP32
    d.alpha, d.beta = 1.0, 0.5
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = L.lib().llmt_b200_gemm(ctypes.byref(d), c.data_ptr(), dummy.data_ptr(),
                                dummy.data_ptr() + 4096, s)
    assert st == L.OK, L.last_error()
    assert torch.equal(c, torch.full((64, 32), 1.5, device=DEV))
    d.m, d.k, d.beta = 0, 8, 0.0
    st = L.lib().llmt_b200_gemm(ctypes.byref(d), c.data_ptr(), dummy.data_ptr(),
                                dummy.data_ptr() + 4096, s)
    assert st == L.OK
    assert torch.equal(c, torch.full((64, 32), 1.5, device=DEV))


# ------------------------------------------- full-size configs, sampled rows ---

def _check_rows(c, a, b, ta, tb, rows, tol, post=None):
    """Oracle on a sample of output rows of a large product."""
    a64 = (a.T if ta else a)[rows]
    ref = oracle.gemm(np.ascontiguousarray(a64), b, False, tb)
    if post is not None:
        ref = post(ref)
    got = host(c[torch.as_tensor(rows, device=DEV)])
    assert oracle.rel_fro(got, ref) <= tol


def test_config2_gpt2_small_mlp_fc_layer_full_size():
    """BASELINE config 2, MLP fc layer at M=8192: fwd with bias+GELU -> bf16, dX, dW+dbias."""
    M, C, F = 8192, 768, 3072
    rng = np.random.default_rng(0)
    x = oracle.round_bf16(rng.standard_normal((M, C)))
    w = oracle.round_bf16(rng.standard_normal((F, C)) * 0.02)
    bias = (rng.standard_normal(F) * 0.02).astype(np.float32)
    dy = oracle.round_bf16(rng.standard_normal((M, F)) * 0.01)
    xd, wd, dyd = dev_bf16(x), dev_bf16(w), dev_bf16(dy)
    rows = rng.choice(M, 48, replace=False)
    h = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    L.gemm(h, xd, wd, False, True, bias=dev_f32(bias), gelu=True)
    _check_rows(h, x, w, False, True, rows, TOL_BF16_OUT_FRO,
                post=lambda r: oracle.epilogue(r, bias=bias, gelu=True))
    dx = torch.empty(M, C, device=DEV, dtype=torch.bfloat16)
    L.gemm(dx, dyd, wd, False, False)
    _check_rows(dx, dy, w, False, False, rows, TOL_BF16_OUT_FRO)
    dw = torch.zeros(F, C, device=DEV)
    db = torch.zeros(F, device=DEV)
    L.gemm(dw, dyd, xd, True, False, beta=1.0, dbias=db, dbias_beta=1.0)
    frows = rng.choice(F, 32, replace=False)
    _check_rows(dw, dy, x, True, False, frows, TOL_BF16_ACC_FRO)
    assert oracle.rel_fro(host(db), oracle.rowsum(dy, trans_a=True)) <= TOL_BF16_ACC_FRO
    # accumulation contract: a second backward doubles the gradient exactly
    dw1 = dw.clone()
    L.gemm(dw, dyd, xd, True, False, beta=1.0, dbias=db, dbias_beta=1.0)
    assert torch.allclose(dw, 2.0 * dw1, rtol=1e-6, atol=0)


def test_config3_lm_head_padded_vocab_sampled():
    """BASELINE config 3 at reduced M (the oracle is sampled): N = 50257 logits in fp32
    through a row pitch of 50264, dX and dW with the reduction over the vocabulary."""
    M, C, V, LD = 1024, 768, 50257, 50264
    rng = np.random.default_rng(3)
    x = oracle.round_bf16(rng.standard_normal((M, C)))
    w = oracle.round_bf16(rng.standard_normal((V, C)) * 0.02)
    xd, wd = dev_bf16(x), dev_bf16(w)
    logits = torch.empty(M, LD, device=DEV)[:, :V]
    L.gemm(logits, xd, wd, False, True)
    rows = rng.choice(M, 16, replace=False)
    _check_rows(logits, x, w, False, True, rows, TOL_BF16_ACC_FRO)
    dl_host = oracle.round_bf16(rng.standard_normal((M, V)) * 1e-4)
    dl = torch.zeros(M, LD, device=DEV, dtype=torch.bfloat16)
    dl[:, :V] = dev_bf16(dl_host)
    dl = dl[:, :V]
    dx = torch.empty(M, C, device=DEV, dtype=torch.bfloat16)
    L.gemm(dx, dl, wd, False, False)
    _check_rows(dx, dl_host, w, False, False, rows, TOL_BF16_OUT_FRO)
    dw = torch.zeros(V, C, device=DEV)
    L.gemm(dw, dl, xd, True, False, beta=1.0)
    vrows = np.concatenate([rng.choice(V, 14, replace=False), [V - 1, V - 2]])
    _check_rows(dw, dl_host, x, True, False, vrows, TOL_BF16_ACC_FRO)


def test_config3_lm_head_contiguous_vocab_50257():
    """BASELINE config 3 with the vocabulary NOT padded: logits and dLogits are contiguous
    [tokens, 50257] (pitch 100514 / 201028 bytes, which TMA cannot address).  fp32 logits are
    written from registers; the bf16 dLogits operand of dX and dW goes through the repack copy."""
    M, C, V = 512, 768, 50257
    rng = np.random.default_rng(33)
    x = oracle.round_bf16(rng.standard_normal((M, C)))
    w = oracle.round_bf16(rng.standard_normal((V, C)) * 0.02)
    dl_host = oracle.round_bf16(rng.standard_normal((M, V)) * 1e-4)
    xd, wd, dl = dev_bf16(x), dev_bf16(w), dev_bf16(dl_host)
    rows = rng.choice(M, 12, replace=False)
    logits = torch.empty(M, V, device=DEV)
    L.gemm(logits, xd, wd, False, True)
    _check_rows(logits, x, w, False, True, rows, TOL_BF16_ACC_FRO)
    dx = torch.empty(M, C, device=DEV, dtype=torch.bfloat16)
    L.gemm(dx, dl, wd, False, False)
    _check_rows(dx, dl_host, w, False, False, rows, TOL_BF16_OUT_FRO)
    dw = torch.zeros(V, C, device=DEV)
    L.gemm(dw, dl, xd, True, False, beta=1.0)
    vrows = np.concatenate([rng.choice(V, 10, replace=False), [V - 1, 0]])
    _check_rows(dw, dl_host, x, True, False, vrows, TOL_BF16_ACC_FRO)


def test_config4_attention_products_forward_and_backward():
    """BASELINE config 4 at reduced batch: S = QK^T/8, P = causal softmax, O = PV, and the
    backward products dV = P^T dO, dP = dO V^T, dQ = a dS K, dK = a dS^T Q (llmt TODO.md:226-228)."""
    B, T, hd = 4, 1024, 64
    alpha = 0.125
    rng = np.random.default_rng(4)
    q, k, v = (oracle.round_bf16(rng.standard_normal((B, T, hd))) for _ in range(3))
    d_o = oracle.round_bf16(rng.standard_normal((B, T, hd)) * 0.01)
    qd, kd, vd, dod = (dev_bf16(t) for t in (q, k, v, d_o))
    s = torch.empty(B, T, T, device=DEV, dtype=torch.bfloat16)
    L.gemm(s, qd, kd, False, True, alpha=alpha)
    s_ref = oracle.gemm(q, k, False, True, alpha)
    assert oracle.rel_fro(host(s), s_ref) <= TOL_BF16_OUT_FRO
    p = torch.empty_like(s)
    L.softmax_fwd(p, s, causal=True)
    p_ref = oracle.softmax(host(s).astype(np.float64), causal=True)
    assert oracle.rel_fro(host(p), p_ref) <= TOL_BF16_OUT_FRO
    iu = np.triu_indices(T, 1)
    assert (host(p)[:, iu[0], iu[1]] == 0.0).all(), "masked probabilities must be exact zeros"
    ph = host(p)
    o = torch.empty(B, T, hd, device=DEV, dtype=torch.bfloat16)
    L.gemm(o, p, vd, False, False)
    assert oracle.rel_fro(host(o), oracle.gemm(ph, v)) <= TOL_BF16_OUT_FRO
    dv = torch.empty(B, T, hd, device=DEV, dtype=torch.bfloat16)
    L.gemm(dv, p, dod, True, False)
    assert oracle.rel_fro(host(dv), oracle.gemm(ph, d_o, True, False)) <= TOL_BF16_OUT_FRO
    dp = torch.empty(B, T, T, device=DEV, dtype=torch.bfloat16)
    L.gemm(dp, dod, vd, False, True)
    assert oracle.rel_fro(host(dp), oracle.gemm(d_o, v, False, True)) <= TOL_BF16_OUT_FRO
    ds = torch.empty_like(dp)
    L.softmax_bwd(ds, p, dp)
    ds_ref = oracle.softmax_bwd(ph.astype(np.float64), host(dp).astype(np.float64))
    assert oracle.rel_fro(host(ds), ds_ref) <= TOL_BF16_OUT_FRO
    dsh = host(ds)
    dq = torch.empty(B, T, hd, device=DEV, dtype=torch.bfloat16)
    L.gemm(dq, ds, kd, False, False, alpha=alpha)
    assert oracle.rel_fro(host(dq), oracle.gemm(dsh, k, False, False, alpha)) <= TOL_BF16_OUT_FRO
    dk = torch.empty(B, T, hd, device=DEV, dtype=torch.bfloat16)
    L.gemm(dk, ds, qd, True, False, alpha=alpha)
    assert oracle.rel_fro(host(dk), oracle.gemm(dsh, q, True, False, alpha)) <= TOL_BF16_OUT_FRO


def test_config5_xl_mlp_shapes_sampled():
    """BASELINE config 5 shapes (C=1600, 4C=6400) on one 8192-token shard."""
    M, C, F = 8192, 1600, 6400
    rng = np.random.default_rng(5)
    x = oracle.round_bf16(rng.standard_normal((M, C)))
    w = oracle.round_bf16(rng.standard_normal((F, C)) * 0.02)
    bias = (rng.standard_normal(F) * 0.02).astype(np.float32)
    xd, wd = dev_bf16(x), dev_bf16(w)
    h = torch.empty(M, F, device=DEV, dtype=torch.bfloat16)
    L.gemm(h, xd, wd, False, True, bias=dev_f32(bias), gelu=True)
    rows = rng.choice(M, 24, replace=False)
    _check_rows(h, x, w, False, True, rows, TOL_BF16_OUT_FRO,
                post=lambda r: oracle.epilogue(r, bias=bias, gelu=True))
    dy = oracle.round_bf16(rng.standard_normal((M, F)) * 0.01)
    dw = torch.zeros(F, C, device=DEV)
    db = torch.zeros(F, device=DEV)
    L.gemm(dw, dev_bf16(dy), xd, True, False, beta=1.0, dbias=db, dbias_beta=1.0)
    frows = rng.choice(F, 16, replace=False)
    _check_rows(dw, dy, x, True, False, frows, TOL_BF16_ACC_FRO)
    assert oracle.rel_fro(host(db), oracle.rowsum(dy, trans_a=True)) <= TOL_BF16_ACC_FRO


# --------------------------------------------------- several problems, one launch ---

def test_grouped_linear_backward_matches_oracle():
    """Linear::backward as ONE launch: dx = dy W and dW += dy^T x (+ dbias) share a tile queue
    (llmt src/layers/linear.cpp:22-30 issues them as two matmul calls)."""
    tokens, out_f, in_f = 2048, 384, 520
    rng = np.random.default_rng(31)
    dy = oracle.round_bf16(rng.standard_normal((tokens, out_f)) * 0.01)
    x = oracle.round_bf16(rng.standard_normal((tokens, in_f)))
    w = oracle.round_bf16(rng.standard_normal((out_f, in_f)) * 0.02)
    dw0 = rng.standard_normal((out_f, in_f)).astype(np.float32)
    db0 = rng.standard_normal(out_f).astype(np.float32)
    dyd, xd, wd = dev_bf16(dy), dev_bf16(x), dev_bf16(w)
    dx = torch.empty(tokens, in_f, device=DEV, dtype=torch.bfloat16)
    dw, db = dev_f32(dw0), dev_f32(db0)
    grp = L.Group([
        (L.make_desc(dx, dyd, wd, False, False), dx, dyd, wd),
        (L.make_desc(dw, dyd, xd, True, False, beta=1.0, dbias=db, dbias_beta=1.0), dw, dyd, xd),
    ])
    need = grp.workspace_bytes()
    grp.set_workspaces([torch.empty(max(b, 256), dtype=torch.uint8, device=DEV) for b in need])
    grp.run()
    assert oracle.rel_fro(host(dx), oracle.gemm(dy, w)) <= TOL_BF16_OUT_FRO
    assert oracle.rel_fro(host(dw), oracle.gemm(dy, x, trans_a=True, beta=1.0, c=dw0)) <= TOL_BF16_ACC_FRO
    assert oracle.rel_fro(host(db), oracle.rowsum(dy, trans_a=True, out=db0, out_beta=1.0)) <= TOL_BF16_ACC_FRO
    # run-to-run: the dynamic tile queue must not change a single bit
    dx2 = torch.empty_like(dx)
    dw2, db2 = dev_f32(dw0), dev_f32(db0)
    grp2 = L.Group([
        (L.make_desc(dx2, dyd, wd, False, False), dx2, dyd, wd),
        (L.make_desc(dw2, dyd, xd, True, False, beta=1.0, dbias=db2, dbias_beta=1.0), dw2, dyd, xd),
    ])
    grp2.set_workspaces([torch.empty(max(b, 256), dtype=torch.uint8, device=DEV) for b in need])
    grp2.run()
    assert torch.equal(dx, dx2) and torch.equal(dw, dw2) and torch.equal(db, db2)


def test_grouped_mixed_shapes_transposes_and_epilogues():
    rng = np.random.default_rng(37)
    specs = [  # m, n, k, ta, tb, out dtype, bias, gelu, alpha, forced splits
        (300, 520, 200, 0, 1, torch.bfloat16, True, True, 1.0, 0),
        (136, 72, 1024, 1, 0, torch.float32, False, False, 0.5, 4),
        (64, 264, 72, 0, 0, torch.float32, True, False, 1.0, 0),
        (257 + 7, 64, 136, 1, 1, torch.bfloat16, False, False, 2.0, 0),
    ]
    probs, refs, outs = [], [], []
    for (m, n, k, ta, tb, cdt, bias, gelu, alpha, splits) in specs:
        a = oracle.round_bf16(rng.standard_normal((k, m) if ta else (m, k)))
        b = oracle.round_bf16(rng.standard_normal((n, k) if tb else (k, n)) * 0.3)
        bv = (rng.standard_normal(n) * 0.5).astype(np.float32) if bias else None
        c = torch.empty(m, n, device=DEV, dtype=cdt)
        ad, bd = dev_bf16(a), dev_bf16(b)
        bt = dev_f32(bv) if bias else None
        probs.append((L.make_desc(c, ad, bd, bool(ta), bool(tb), alpha=alpha, bias=bt, gelu=gelu,
                                  splits=splits), c, ad, bd, bt))
        refs.append(oracle.epilogue(oracle.gemm(a, b, bool(ta), bool(tb), alpha), bias=bv, gelu=gelu))
        outs.append((c, cdt))
    grp = L.Group([p[:4] for p in probs])
    need = grp.workspace_bytes()
    assert need[1] > 0  # the forced split needs scratch
    grp.set_workspaces([torch.empty(max(b, 256), dtype=torch.uint8, device=DEV) for b in need])
    grp.run()
    for (c, cdt), ref in zip(outs, refs):
        tol = TOL_BF16_OUT_FRO if cdt == torch.bfloat16 else TOL_BF16_ACC_FRO
        assert oracle.rel_fro(host(c), ref) <= tol


def test_grouped_rejects_dependent_problems():
    x = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(64, 64, device=DEV, dtype=torch.bfloat16)
    y = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    z = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    grp = L.Group([(L.make_desc(y, x, w, False, True), y, x, w),
                   (L.make_desc(z, y, w, False, True), z, y, w)])  # second reads what the first writes
    with pytest.raises(L.LlmtB200Error) as e:
        grp.run()
    assert e.value.status == L.ERR_INVALID and "independent" in str(e.value)


# ------------------------------------------- against cuBLASLt in bf16 (llmt's call pattern) ---

@pytest.mark.parametrize("shape", ["qkv_fwd", "fc_dx", "fc_dw"])
def test_error_no_worse_than_twice_cublaslt(shape):
    """BASELINE north star: on the same seeded inputs the error against the fp64 product is no
    worse than 2x that of cuBLASLt called the way llmt calls it (bf16 operands, fp32 accumulate)."""
    from oracle import cublaslt_ref
    if not cublaslt_ref.available():
        pytest.skip("comparator not built (make -C oracle cmp)")
    M = 2048
    cases = {"qkv_fwd": (M, 2304, 768, 0, 1, torch.bfloat16),
             "fc_dx": (M, 768, 3072, 0, 0, torch.bfloat16),
             "fc_dw": (3072, 768, M, 1, 0, torch.float32)}
    m, n, k, ta, tb, cdt = cases[shape]
    rng = np.random.default_rng(41)
    a = oracle.round_bf16(rng.standard_normal((k, m) if ta else (m, k)))
    b = oracle.round_bf16(rng.standard_normal((n, k) if tb else (k, n)) * 0.02)
    ad, bd = dev_bf16(a), dev_bf16(b)
    ref = oracle.gemm(a, b, bool(ta), bool(tb))
    ours = torch.empty(m, n, device=DEV, dtype=cdt)
    L.gemm(ours, ad, bd, bool(ta), bool(tb))
    lt = cublaslt_ref.CublasLtBf16()
    theirs = torch.empty(m, n, device=DEV, dtype=cdt)
    lt.matmul(theirs, ad, bd, bool(ta), bool(tb))
    torch.cuda.synchronize()
    e_ours, e_lt = oracle.rel_fro(host(ours), ref), oracle.rel_fro(host(theirs), ref)
    lt.close()
    assert e_ours <= 2.0 * e_lt + 1e-7, (e_ours, e_lt)
    assert e_ours <= (TOL_BF16_OUT_FRO if cdt == torch.bfloat16 else TOL_BF16_ACC_FRO)
