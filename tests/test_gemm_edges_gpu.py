"""Edges of the tensor-core path, through the C ABI: every extent at 1, tile-1, tile and
tile+1 in each of M, N and K, on every transpose combination, on single CTAs and CTA pairs,
with and without split-K, with guard words around everything the call may write (C, dbias,
the workspace); operands that TMA cannot address in place; the host-side tensor-map cache.

Tolerances are those of test_gemm_gpu.py: fp32 output of bf16 operands vs the fp64 product of
the same bf16-rounded inputs, relative Frobenius <= 1e-3.
"""
import numpy as np
import pytest
import torch

import llmt_b200 as L
from oracle import oracle

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = 1e-3
GUARD = 12345.0


@pytest.fixture(autouse=True)
def _healthy_device():
    yield
    assert L.device_status() == (0, 0)


def _bf16_dev(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(DEV).to(torch.bfloat16)


class Guarded:
    """A [rows, cols] fp32 view in the middle of a larger buffer filled with a sentinel."""

    def __init__(self, rows, cols, pad_rows=2, pad_cols=8, init=None):
        self.full = torch.full((rows + 2 * pad_rows, cols + 2 * pad_cols), GUARD, device=DEV)
        self.view = self.full[pad_rows:pad_rows + rows, pad_cols:pad_cols + cols]
        self.view.copy_(init if init is not None else torch.zeros(rows, cols, device=DEV))
        self.mask = torch.ones_like(self.full, dtype=torch.bool)
        self.mask[pad_rows:pad_rows + rows, pad_cols:pad_cols + cols] = False

    def intact(self):
        return bool((self.full[self.mask] == GUARD).all())


def _padded_operand(x):
    """bf16 copy of x with a row pitch that TMA accepts (multiple of 8) but that is larger than the row."""
    rows, cols = x.shape
    ld = (cols + 7) // 8 * 8 + 8
    buf = torch.zeros(rows, ld, device=DEV, dtype=torch.bfloat16)
    buf[:, :cols] = _bf16_dev(x)
    return buf[:, :cols]


def _extents(tile):
    return [1, tile - 1, tile, tile + 1]


@pytest.mark.parametrize("pairs", [1, 2])
@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
def test_ragged_grid_with_guard_words(ta, tb, pairs):
    tile_m = 128 * pairs
    rng = np.random.default_rng(1000 + 10 * pairs + 2 * ta + tb)
    cases = 0
    for tile_n in ([128, 256] if pairs == 2 else [64, 192, 256]):
        for m in _extents(tile_m):
            if pairs == 2 and m <= 128:
                continue  # CTA pairs need more than one 128-row block
            for n in _extents(tile_n):
                for k in [1, 63, 64, 65, 200]:
                    for splits in ([1, 2] if k > 64 else [1]):
                        a = oracle.round_bf16(rng.standard_normal((k, m) if ta else (m, k)))
                        b = oracle.round_bf16(rng.standard_normal((n, k) if tb else (k, n)) * 0.5)
                        c0 = rng.standard_normal((m, n)).astype(np.float32)
                        ad, bd = _padded_operand(a), _padded_operand(b)
                        c = Guarded(m, n, init=torch.from_numpy(c0).to(DEV))
                        want_dbias = ta == 1
                        db = Guarded(1, m) if want_dbias else None
                        d = L.make_desc(c.view, ad, bd, bool(ta), bool(tb), alpha=0.5, beta=1.0,
                                        dbias=db.view[0] if want_dbias else None, dbias_beta=0.0,
                                        tile_n=tile_n, splits=splits, cta_pairs=pairs)
                        need = L.workspace_bytes(d, ad, bd)
                        ws = torch.full((need // 4 + 64,), GUARD, device=DEV)
                        if need:
                            d.workspace, d.workspace_bytes = ws.data_ptr(), need
                        L.gemm_desc(d, c.view, ad, bd)
                        what = (m, n, k, tile_n, splits)
                        ref = oracle.gemm(a, b, bool(ta), bool(tb), 0.5, 1.0, c0)
                        assert oracle.rel_fro(c.view.cpu().numpy(), ref) <= TOL, what
                        assert c.intact(), ("C guard", what)
                        assert bool((ws[need // 4:] == GUARD).all()), ("workspace guard", what)
                        if want_dbias:
                            got = db.view[0].cpu().numpy()
                            assert oracle.rel_fro(got, oracle.rowsum(a, trans_a=True)) <= TOL, ("dbias", what)
                            assert db.intact(), ("dbias guard", what)
                        cases += 1
    assert cases >= 100


@pytest.mark.parametrize("pairs", [1, 2])
def test_pair_and_single_split_ragged_mn_major_b_with_dbias_accumulation(pairs):
    """dW-shaped product (both operands MN-major), ragged in every extent, split-K, dbias with
    beta = 1 onto a prior value, twice in a row: the second call doubles the increment."""
    m, n, k = 520, 392, 1000
    rng = np.random.default_rng(77 + pairs)
    dy = oracle.round_bf16(rng.standard_normal((k, m)) * 0.01)
    x = oracle.round_bf16(rng.standard_normal((k, n)))
    dw0 = rng.standard_normal((m, n)).astype(np.float32)
    db0 = rng.standard_normal(m).astype(np.float32)
    dyd, xd = _padded_operand(dy), _padded_operand(x)
    dw = Guarded(m, n, init=torch.from_numpy(dw0).to(DEV))
    db = Guarded(1, m, init=torch.from_numpy(db0).to(DEV)[None, :])
    for rep in (1, 2):
        L.gemm(dw.view, dyd, xd, True, False, beta=1.0, dbias=db.view[0], dbias_beta=1.0, splits=3,
               tile_n=256 if pairs == 2 else 192, cta_pairs=pairs)
        inc_w = oracle.gemm(dy, x, trans_a=True)
        inc_b = oracle.rowsum(dy, trans_a=True)
        assert oracle.rel_fro(dw.view.cpu().numpy() - dw0, rep * inc_w) <= 5e-3  # difference of close numbers
        assert oracle.rel_fro(db.view[0].cpu().numpy() - db0, rep * inc_b) <= 5e-3
        assert dw.intact() and db.intact()


@pytest.mark.parametrize("ta", [0, 1])
def test_dbias_without_transposition_and_with(ta):
    """dbias[i] = sum_p op(A)[i, p] for both storage orders of A (row sums of an [m, k] matrix,
    column sums of a [k, m] one), ragged k, on the default plan."""
    m, n, k = 333, 264, 1234
    rng = np.random.default_rng(88 + ta)
    a = oracle.round_bf16(rng.standard_normal((k, m) if ta else (m, k)))
    b = oracle.round_bf16(rng.standard_normal((k, n)))
    ad, bd = _padded_operand(a), _padded_operand(b)
    c = torch.empty(m, n, device=DEV)
    db = torch.full((m,), 7.0, device=DEV)
    L.gemm(c, ad, bd, bool(ta), False, dbias=db, dbias_beta=0.0)
    assert oracle.rel_fro(c.cpu().numpy(), oracle.gemm(a, b, bool(ta), False)) <= TOL
    assert oracle.rel_fro(db.cpu().numpy(), oracle.rowsum(a, trans_a=bool(ta))) <= TOL


def test_fp32_path_bias_gradient():
    """Strict-fp32 Linear backward with a bias: dbias += column sums of dy (fixed order)."""
    rng = np.random.default_rng(91)
    dy = rng.standard_normal((300, 70)).astype(np.float32)
    x = rng.standard_normal((300, 50)).astype(np.float32)
    db0 = rng.standard_normal(70).astype(np.float32)
    dw = torch.zeros(70, 50, device=DEV)
    db = torch.from_numpy(db0).to(DEV)
    L.gemm(dw, torch.from_numpy(dy).to(DEV), torch.from_numpy(x).to(DEV), True, False, beta=1.0,
           dbias=db, dbias_beta=1.0)
    assert oracle.rel_fro(dw.cpu().numpy(), oracle.gemm(dy, x, trans_a=True)) <= 1e-5
    assert oracle.rel_fro(db.cpu().numpy(), db0 + dy.astype(np.float64).sum(axis=0)) <= 1e-5


def test_operands_that_start_at_odd_addresses_are_repacked():
    """Slices such as x[:, 1:] start 2 bytes off a 16-byte boundary (and have an odd pitch view):
    they are copied into the workspace first; the result is that of the aligned operands."""
    m, n, k = 200, 136, 264
    rng = np.random.default_rng(93)
    a = oracle.round_bf16(rng.standard_normal((m, k)))
    b = oracle.round_bf16(rng.standard_normal((n, k)))
    abuf = torch.zeros(m, k + 8, device=DEV, dtype=torch.bfloat16)
    bbuf = torch.zeros(n, k + 8, device=DEV, dtype=torch.bfloat16)
    abuf[:, 1:k + 1] = _bf16_dev(a)
    bbuf[:, 3:k + 3] = _bf16_dev(b)
    av, bv = abuf[:, 1:k + 1], bbuf[:, 3:k + 3]
    assert av.data_ptr() % 16 != 0 and bv.data_ptr() % 16 != 0
    c = torch.empty(m, n, device=DEV)
    d = L.make_desc(c, av, bv, False, True)
    assert L.workspace_bytes(d) == 0 and L.workspace_bytes(d, av, bv) >= 2 * (m + n) * k
    L.gemm(c, av, bv, False, True)
    assert oracle.rel_fro(c.cpu().numpy(), oracle.gemm(a, b, False, True)) <= TOL


def test_tensor_map_cache_replays_descriptors():
    """The second call on the same buffers encodes nothing and gives the same bits."""
    m, n, k = 512, 384, 256
    g = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randn(m, k, device=DEV, generator=g).to(torch.bfloat16)
    b = torch.randn(n, k, device=DEV, generator=g).to(torch.bfloat16)
    c1 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    d = L.make_desc(c1, a, b, False, True)
    L.gemm_desc(d, c1, a, b)
    h0, m0 = L.tensor_map_cache_stats()
    first = c1.clone()
    c1.zero_()
    L.gemm_desc(d, c1, a, b)
    h1, m1 = L.tensor_map_cache_stats()
    assert m1 == m0 and h1 >= h0 + 3   # A, B and C maps all came from the cache
    assert torch.equal(c1, first)
    # a different shape on the same base addresses must not be answered from the cache
    c2 = torch.empty(m // 2, n, device=DEV, dtype=torch.bfloat16)
    L.gemm(c2, a[: m // 2], b, False, True)
    assert torch.equal(c2, first[: m // 2])


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_head_split_and_merge_match_llmt_goldens(dt):
    """llmt tests/unit/test_attention.cu:23-43 (golden case `permute`, exact data movement)."""
    from tests.support import GoldenCase
    g = GoldenCase("permute")
    dev = lambda n: torch.from_numpy(g.tensor(n)).to(DEV).to(dt)
    qkv = dev("qkv")
    q, k, v = (torch.empty(2, 2, 3, 4, device=DEV, dtype=dt) for _ in range(3))
    L.head_split(q, k, v, qkv)
    for got, name in ((q, "q"), (k, "k"), (v, "v")):
        assert torch.equal(got, dev(name)), name
    y = torch.empty(2, 3, 8, device=DEV, dtype=dt)
    L.head_merge(y, dev("x"))
    assert torch.equal(y, dev("y"))
    with pytest.raises(L.LlmtB200Error):
        L.head_merge(qkv.view(-1)[: 2 * 3 * 8].view(2, 3, 8), qkv.view(-1)[: 2 * 2 * 3 * 4].view(2, 2, 3, 4))  # aliasing


def test_head_split_and_merge_at_model_size_vectorised():
    """GPT-2-small attention shapes (B = 8, H = 12, T = 1024, hd = 64), bf16: the 16-byte path."""
    B, H, T, hd = 8, 12, 1024, 64
    g = torch.Generator(device=DEV).manual_seed(9)
    qkv = torch.randn(B, T, 3 * H * hd, device=DEV, generator=g).to(torch.bfloat16)
    q, k, v = (torch.empty(B, H, T, hd, device=DEV, dtype=torch.bfloat16) for _ in range(3))
    L.head_split(q, k, v, qkv)
    want = qkv.view(B, T, 3, H, hd).permute(2, 0, 3, 1, 4)
    assert torch.equal(q, want[0]) and torch.equal(k, want[1]) and torch.equal(v, want[2])
    y = torch.empty(B, T, H * hd, device=DEV, dtype=torch.bfloat16)
    L.head_merge(y, q)
    assert torch.equal(y, q.permute(0, 2, 1, 3).reshape(B, T, H * hd))


def _packed_desc(c, a, b, m, n, k, batch, inner, ld, st, st_outer, trans_b, alpha=1.0):
    """Descriptor of a batch laid out on two levels: (lda, ldb, ldc), (stride_a, stride_b, stride_c) and
    (stride_a_outer, ...) in elements; c, a, b are the tensors that own the memory."""
    d = L.GemmDesc()
    d.m, d.n, d.k, d.batch, d.batch_inner = m, n, k, batch, inner
    d.lda, d.ldb, d.ldc = ld
    d.stride_a, d.stride_b, d.stride_c = st
    d.stride_a_outer, d.stride_b_outer, d.stride_c_outer = st_outer
    d.trans_a, d.trans_b = 0, int(trans_b)
    d.dtype_ab, d.dtype_c = L._dtype_code(a), L._dtype_code(c)
    d.alpha, d.beta = alpha, 0.0
    return d


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float32])
def test_attention_products_on_the_packed_qkv_layout(dt):
    """S = Q K^T / sqrt(hd) and O = P V with Q, K, V read straight out of the [B, T, 3*H*hd] output of the
    QKV projection and O written straight into [B, T, H*hd] token rows (batch_inner / stride_*_outer):
    the same bits as head split -> per-head products -> head merge."""
    import ctypes
    B, H, T, hd = (2, 12, 256, 64) if dt == torch.bfloat16 else (2, 3, 40, 8)
    A = H * hd
    g = torch.Generator(device=DEV).manual_seed(21)
    qkv = torch.randn(B, T, 3 * A, device=DEV, generator=g).to(dt)
    alpha = 1.0 / float(np.sqrt(hd))
    # reference route: explicit split, batched products on contiguous [B*H, T, hd] tensors, explicit merge
    q, k, v = (torch.empty(B, H, T, hd, device=DEV, dtype=dt) for _ in range(3))
    L.head_split(q, k, v, qkv)
    s_ref = torch.empty(B * H, T, T, device=DEV, dtype=dt)
    L.gemm(s_ref, q.view(B * H, T, hd), k.view(B * H, T, hd), False, True, alpha=alpha)
    L.softmax_fwd(s_ref, s_ref, causal=True)
    o_heads = torch.empty(B * H, T, hd, device=DEV, dtype=dt)
    L.gemm(o_heads, s_ref, v.view(B * H, T, hd), False, False)
    y_ref = torch.empty(B, T, A, device=DEV, dtype=dt)
    L.head_merge(y_ref, o_heads.view(B, H, T, hd))
    # packed route
    es = qkv.element_size()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    scores = torch.empty(B, H, T, T, device=DEV, dtype=dt)
    d = _packed_desc(scores, qkv, qkv, T, T, hd, B * H, H, (3 * A, 3 * A, T), (hd, hd, T * T),
                     (T * 3 * A, T * 3 * A, H * T * T), True, alpha)
    st = L.lib().llmt_b200_gemm(ctypes.byref(d), scores.data_ptr(), qkv.data_ptr(), qkv.data_ptr() + A * es, stream)
    assert st == L.OK, L.last_error()
    L.softmax_fwd(scores.view(B * H, T, T), scores.view(B * H, T, T), causal=True)
    y = torch.full((B, T, A), 7.0, device=DEV, dtype=dt)
    d2 = _packed_desc(y, scores, qkv, T, hd, T, B * H, H, (T, 3 * A, A), (T * T, hd, hd),
                      (H * T * T, T * 3 * A, T * A), False)
    st = L.lib().llmt_b200_gemm(ctypes.byref(d2), y.data_ptr(), scores.data_ptr(), qkv.data_ptr() + 2 * A * es, stream)
    assert st == L.OK, L.last_error()
    assert torch.equal(scores.view(B * H, T, T), s_ref)
    assert torch.equal(y, y_ref)
    # and against the oracle, one (batch, head) item
    b_, h_ = 1, H - 1
    qh, kh, vh = (qkv[b_, :, part * A + h_ * hd: part * A + (h_ + 1) * hd].float().cpu().numpy() for part in range(3))
    p_ref = oracle.softmax(oracle.gemm(oracle.round_bf16(qh) if dt == torch.bfloat16 else qh, kh, False, True, alpha)[None],
                           causal=True)[0]
    tol = 4e-3 if dt == torch.bfloat16 else 1e-5
    assert oracle.rel_fro(scores[b_, h_].float().cpu().numpy(), p_ref) <= 2 * tol
    o_ref = oracle.gemm(scores[b_, h_].float().cpu().numpy(), vh)
    assert oracle.rel_fro(y[b_, :, h_ * hd:(h_ + 1) * hd].float().cpu().numpy(), o_ref) <= tol
