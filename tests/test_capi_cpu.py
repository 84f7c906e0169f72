"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
public header declares, and rejects contract violations with status codes
(never aborts) — no compute call is made here."""
import ctypes
import os
import re

import pytest

import llmt_b200 as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "llmt_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return re.findall(r"LLMT_B200_API\s+[\w\s\*]+?\b(llmt_b200_\w+)\s*\(", text)


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    assert "llmt_b200_gemm" in syms and "llmt_b200_gemm_workspace_bytes" in syms
    assert len(syms) == len(set(syms)) >= 9


def test_library_exports_every_declared_symbol():
    lib = L.lib()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(set(declared_symbols())) == sorted(set(L.EXPORTS) | set(declared_symbols()))
    assert lib.llmt_b200_abi_version() == 5


def test_descriptor_layout_matches_the_header():
    # field order and sizes of struct llmt_b200_gemm_desc as the C compiler lays them out
    assert ctypes.sizeof(L.GemmDesc) == 10 * 8 + 4 * 4 + 2 * 4 + 2 * 4 + 2 * 8 + 4 * 4 + 2 * 8 + 4 * 8 + 8
    assert L.GemmDesc.batch_inner.offset == L.GemmDesc.workspace_bytes.offset + 8
    assert L.GemmDesc.plan_cta_pairs.offset == L.GemmDesc.plan_splits.offset + 4
    assert L.GemmDesc.workspace.offset % 8 == 0
    assert L.GemmDesc.aux.offset == L.GemmDesc.stride_c_outer.offset + 8
    # and what gcc makes of the header itself
    import shutil
    import subprocess
    import tempfile
    if shutil.which("gcc"):
        src = ('#include <stddef.h>\n#include <stdio.h>\n#include "llmt_b200.h"\n'
               'int main(void) { printf("%zu %zu %zu %zu\\n", sizeof(llmt_b200_gemm_desc), offsetof(llmt_b200_gemm_desc, bias), '
               'offsetof(llmt_b200_gemm_desc, workspace), offsetof(llmt_b200_gemm_desc, aux)); return 0; }\n')
        with tempfile.TemporaryDirectory() as tmp:
            c = os.path.join(tmp, "layout.c")
            with open(c, "w") as f:
                f.write(src)
            exe = os.path.join(tmp, "layout")
            subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
            got = [int(x) for x in subprocess.check_output([exe]).split()]
        assert got == [ctypes.sizeof(L.GemmDesc), L.GemmDesc.bias.offset, L.GemmDesc.workspace.offset, L.GemmDesc.aux.offset]


def _desc(**kw):
    d = L.GemmDesc()
    d.m, d.n, d.k, d.batch = 128, 128, 64, 1
    d.lda, d.ldb, d.ldc = 64, 64, 128
    d.trans_b = 1
    d.dtype_ab, d.dtype_c = L.BF16, L.FP32
    d.alpha = 1.0
    for k, v in kw.items():
        setattr(d, k, v)
    return d


A, B, C = 0x10000, 0x20000, 0x40000  # fake, non-overlapping, 16-byte aligned device addresses


def _call(d, c=C, a=A, b=B):
    return L.lib().llmt_b200_gemm(ctypes.byref(d), ctypes.c_void_p(c), ctypes.c_void_p(a),
                                  ctypes.c_void_p(b), None)


@pytest.mark.parametrize("kw,status,needle", [
    (dict(lda=32), L.ERR_INVALID, "row pitch"),
    (dict(m=-1), L.ERR_INVALID, "negative"),
    (dict(dtype_ab=7), L.ERR_UNSUPPORTED, "dtype code 7"),
    (dict(dtype_ab=L.FP32, dtype_c=L.BF16), L.ERR_UNSUPPORTED, "mixed dtypes"),
    (dict(epilogue=16), L.ERR_INVALID, "epilogue"),
    (dict(epilogue=L.EPI_SAVE_PRE), L.ERR_INVALID, "EPI_SAVE_PRE goes with EPI_GELU"),
    (dict(epilogue=L.EPI_GELU_BWD), L.ERR_INVALID, "aux is null"),
    (dict(epilogue=L.EPI_GELU_BWD | L.EPI_GELU), L.ERR_INVALID, "stands alone"),
    (dict(epilogue=L.EPI_BIAS), L.ERR_INVALID, "bias is null"),
    (dict(plan_tile_n=100), L.ERR_INVALID, "plan_tile_n"),
    (dict(plan_cta_pairs=3), L.ERR_INVALID, "plan_cta_pairs"),
    (dict(plan_cta_pairs=2), L.ERR_INVALID, "CTA pairs need m > 128"),
    (dict(lda=68), L.ERR_WORKSPACE, "repacked operands"),  # odd pitch: needs scratch for an aligned copy
    (dict(batch=2, stride_a=10, stride_b=128 * 64, stride_c=128 * 128), L.ERR_INVALID, "batch stride"),
])
def test_contract_violations_return_status(kw, status, needle):
    assert _call(_desc(**kw)) == status
    assert needle in L.last_error()


def test_null_and_overlapping_pointers_are_rejected():
    d = _desc()
    assert _call(d, a=0) == L.ERR_INVALID and "null data" in L.last_error()
    assert L.lib().llmt_b200_gemm(None, ctypes.c_void_p(C), ctypes.c_void_p(A), ctypes.c_void_p(B),
                                  None) == L.ERR_INVALID
    assert _call(d, c=A + 64) == L.ERR_INVALID and "overlaps" in L.last_error()


def test_unaligned_bf16_base_needs_scratch_for_an_aligned_copy():
    # a slice such as x[:, 1:] starts at an odd address: TMA cannot read it in place
    d = _desc()
    assert _call(d, a=A + 2) == L.ERR_WORKSPACE and "repacked operands" in L.last_error()
    lib = L.lib()
    assert lib.llmt_b200_gemm_workspace_bytes(ctypes.byref(d)) == 0
    need = lib.llmt_b200_gemm_workspace_bytes_for(ctypes.byref(d), ctypes.c_void_p(A + 2), ctypes.c_void_p(B))
    assert need == 128 * 64 * 2  # one aligned copy of A


def test_dbias_contract():
    d = _desc(dbias=0x80000, batch=2, stride_a=128 * 64, stride_b=128 * 64, stride_c=128 * 128)
    assert _call(d) == L.ERR_UNSUPPORTED and "batched" in L.last_error()


def test_dimensions_above_int32_are_refused():
    big = 1 << 31
    d = _desc(m=big, ldc=128)
    assert _call(d) == L.ERR_UNSUPPORTED and "2^31" in L.last_error()
    d = _desc(k=big, lda=big, ldb=big)
    assert _call(d) == L.ERR_UNSUPPORTED and "2^31" in L.last_error()


def test_written_ranges_must_not_overlap_anything_else():
    # C is 128 x 128 fp32 at C; A and B are 128 x 64 bf16
    assert _call(_desc(dbias=C + 256)) == L.ERR_INVALID and "dbias overlaps C" in L.last_error()
    assert _call(_desc(dbias=A + 16)) == L.ERR_INVALID and "dbias overlaps A" in L.last_error()
    d = _desc(workspace=B + 1024, workspace_bytes=4096)
    assert _call(d) == L.ERR_INVALID and "workspace overlaps B" in L.last_error()
    d = _desc(epilogue=L.EPI_BIAS, bias=0x90000, bias_dtype=L.FP32, workspace=0x90000 + 256, workspace_bytes=4096)
    assert _call(d) == L.ERR_INVALID and "workspace overlaps bias" in L.last_error()
    d = _desc(dbias=0x90000, workspace=0x90000, workspace_bytes=4096)
    assert _call(d) == L.ERR_INVALID and "dbias overlaps workspace" in L.last_error()


def _grouped(descs, cs, as_, bs):
    n = len(descs)
    arr = (L.GemmDesc * n)(*descs)
    vp = lambda xs: (ctypes.c_void_p * n)(*xs)
    return L.lib().llmt_b200_gemm_grouped(arr, vp(cs), vp(as_), vp(bs), n, None)


def test_grouped_problems_are_checked_by_address_range():
    d0, d1 = _desc(), _desc()
    # problem 1 reads, as its A, a view into the middle of what problem 0 writes
    assert _grouped([d0, d1], [C, 0x80000], [A, C + 4096], [B, B]) == L.ERR_INVALID
    assert "not independent" in L.last_error()
    # two C views into one buffer at different offsets
    assert _grouped([d0, d1], [C, C + 512], [A, A], [B, B]) == L.ERR_INVALID
    assert "not independent" in L.last_error()
    # a dbias of one problem inside the C of the other
    assert _grouped([_desc(dbias=0x80000 + 64), d1], [C, 0x80000], [A, A], [B, B]) == L.ERR_INVALID


def test_forced_pairs_are_refused_in_a_launch_that_cannot_pair():
    # plan_cta_pairs = 2 on a problem that shares its launch with one that has m <= 128: the launch
    # would fall back to single CTAs; that is reported, not done silently
    wide = _desc(m=512, n=256, k=64, ldc=256, plan_cta_pairs=2, plan_tile_n=256, dbias=0x5000000)
    small = _desc()
    assert _grouped([wide, small], [0x1000000, 0x2000000], [A, A], [B, B]) == L.ERR_INVALID
    assert "asks for CTA pairs" in L.last_error()


def test_two_level_batch_layout_contract():
    # the per-head products of attention on the packed QKV buffer: B = 2, H = 3, T = 128, hd = 64
    H, T, hd, B = 3, 128, 64, 2
    A3 = 3 * H * hd
    d = _desc(m=T, n=T, k=hd, batch=B * H, batch_inner=H, lda=A3, ldb=A3, ldc=T, trans_b=1,
              stride_a=hd, stride_b=hd, stride_c=T * T, stride_a_outer=T * A3, stride_b_outer=T * A3,
              stride_c_outer=H * T * T, dtype_c=L.BF16)
    qkv, scores = 0x1000000, 0x3000000
    # (strides between heads smaller than a matrix are what this layout is for; the valid case runs
    # in the GPU tests - nothing here may reach a launch)
    assert L.plan(d).startswith("tcgen05")
    bad = _desc(m=T, n=T, k=hd, batch=B * H, batch_inner=4, lda=A3, ldb=A3, ldc=T, trans_b=1)
    assert _call(bad, c=scores, a=qkv, b=qkv + 2 * H * hd) == L.ERR_INVALID and "batch_inner" in L.last_error()
    odd = _desc(m=T, n=T, k=hd, batch=B * H, batch_inner=H, lda=A3, ldb=A3, ldc=T, trans_b=1,
                stride_a=hd + 1, stride_b=hd, stride_c=T * T, stride_a_outer=T * A3, stride_b_outer=T * A3,
                stride_c_outer=H * T * T)
    assert _call(odd, c=scores, a=qkv, b=qkv + 2 * H * hd) == L.ERR_UNSUPPORTED and "two-level" in L.last_error()


def test_empty_output_is_a_no_op():
    assert _call(_desc(m=0)) == L.OK
    assert _call(_desc(batch=0)) == L.OK


def test_plan_is_a_pure_function_of_the_problem():
    # the determinism device: one problem -> one plan, every time
    # (role of llmt's AlgoCache, include/llmt/kernels/algo_cache.h:18-42)
    d = _desc(m=8192, n=2304, k=768, lda=768, ldb=768, ldc=2304)
    p1, p2 = L.plan(d), L.plan(d)
    assert p1 == p2 and "tcgen05 cta-pair tile=256x256x64" in p1  # pairs by default (no fused dbias)
    d.plan_cta_pairs = 1  # single CTAs on request: 128-row tiles
    assert "1-cta tile=128x256x64" in L.plan(d)
    d.plan_cta_pairs = 2
    assert "cta-pair tile=256x256x64" in L.plan(d)
    d.plan_cta_pairs = 0
    assert L.workspace_bytes(d) == 0
    dw = _desc(m=768, n=768, k=8192, trans_a=1, trans_b=0, lda=768, ldb=768, ldc=768)
    assert "splits=" in L.plan(dw)
    ws = L.workspace_bytes(dw)
    assert ws > 0 and ws % 256 == 0
    # workspace shortfall is reported before anything is launched
    dw.workspace, dw.workspace_bytes = 0x100000, 16
    assert _call(dw, c=0x7000000000, a=0x1000000000, b=0x2000000000) == L.ERR_WORKSPACE
    forced = _desc(m=768, n=768, k=8192, plan_tile_n=64, plan_splits=1)  # 64-wide tiles: single CTAs
    assert "1-cta tile=128x64x64" in L.plan(forced) and "splits=1 " in L.plan(forced)


def test_softmax_contract():
    lib = L.lib()
    assert lib.llmt_b200_softmax_fwd(ctypes.c_void_p(A), ctypes.c_void_p(A), 8, 4, 5, 0, 1, None) \
        == L.ERR_INVALID
    assert "square" in L.last_error()
    assert lib.llmt_b200_softmax_fwd(None, ctypes.c_void_p(A), 8, 4, 4, 0, 1, None) == L.ERR_INVALID
    assert lib.llmt_b200_softmax_fwd(ctypes.c_void_p(A), ctypes.c_void_p(A), 8, 4, 4, 2, 0, None) \
        == L.ERR_UNSUPPORTED


# ---- gradient exchange: host-side contract (no launch happens on these paths) --------------

def _comm(world=2, rank=0, slot=64):
    d = L.CommDesc()
    d.rank, d.world, d.slot_elems = rank, world, slot
    for r in range(min(world, L.COMM_MAX_RANKS)):
        d.grad[r], d.stage[r], d.flags[r] = 0x100000 * (r + 1), 0x100000 * (r + 1) + 0x40000, 0x100000 * (r + 1) + 0x80000
    d.epoch = 0x900000
    return d


def test_comm_descriptor_layout_matches_the_header():
    assert ctypes.sizeof(L.CommDesc) == 2 * 4 + 3 * 8 * 8 + 8 + 8 + 8
    text = open(HEADER).read()
    assert f"#define LLMT_B200_COMM_MAX_RANKS {L.COMM_MAX_RANKS}" in text
    assert f"#define LLMT_B200_COMM_MAX_CTAS {L.COMM_MAX_CTAS}" in text  # 128
    assert f"#define LLMT_B200_DEV_WAIT_PEER {L.DEV_WAIT_PEER}" in text


def test_allreduce_rejects_contract_violations():
    f = L.lib().llmt_b200_grad_allreduce
    assert f(None, 0, 8, 4, None) == L.ERR_INVALID
    assert f(ctypes.byref(_comm(world=9)), 0, 8, 4, None) == L.ERR_INVALID
    assert f(ctypes.byref(_comm(rank=2)), 0, 8, 4, None) == L.ERR_INVALID
    assert f(ctypes.byref(_comm()), 0, 8, 0, None) == L.ERR_INVALID
    assert f(ctypes.byref(_comm()), 0, 8, L.COMM_MAX_CTAS + 1, None) == L.ERR_INVALID
    assert f(ctypes.byref(_comm()), 2, 8, 4, None) == L.ERR_UNSUPPORTED
    assert f(ctypes.byref(_comm()), 0, 10, 4, None) == L.ERR_UNSUPPORTED
    assert f(ctypes.byref(_comm(slot=64)), 0, 4096, 4, None) == L.ERR_WORKSPACE
    assert "staging slot" in L.last_error()
    d = _comm()
    d.stage[1] = None
    assert f(ctypes.byref(d), 0, 8, 4, None) == L.ERR_INVALID
    d = _comm()
    d.grad[0] = 0x100004
    assert f(ctypes.byref(d), 0, 8, 4, None) == L.ERR_UNSUPPORTED


def test_sm_budget_round_trips():
    lib = L.lib()
    prev = lib.llmt_b200_set_sm_budget(140)
    assert lib.llmt_b200_set_sm_budget(prev) == 140
    assert lib.llmt_b200_set_sm_budget(-1) < 0 and "sm budget" in L.last_error()
    assert lib.llmt_b200_set_sm_budget(prev) == prev


def test_exchange_layout_is_aligned_and_large_enough():
    from llmt_b200.dp import exchange_layout
    for numel in (4, 64, 7080960, 4 * 1237):
        for world in (1, 2, 3, 8):
            lay = exchange_layout(numel, world)
            assert lay["slot_elems"] % 64 == 0 and lay["slot_elems"] * world >= numel
            assert lay["stage_off"] % 256 == 0 and lay["flags_off"] % 256 == 0
            assert lay["stage_off"] >= numel * 4
            assert lay["total"] == lay["flags_off"] + L.COMM_FLAG_BYTES
    with pytest.raises(ValueError):
        exchange_layout(6, 2)


def test_fused_dbias_products_run_on_pairs_with_full_width_tiles():
    # dW + dbias of one (unbatched) product: the epilogue warps add up the A stages in shared memory, so
    # the product keeps 256-wide tiles on CTA pairs and there are no dbias tickets (the QKV layer of
    # GPT-2-small: 2304 x 768 over 8192 tokens, split in two so that its 27 tiles fill the 74 pairs)
    d = _desc(m=2304, n=768, k=8192, trans_a=1, trans_b=0, lda=2304, ldb=768, ldc=768,
              dtype_c=L.FP32, beta=1.0, dbias=0x5000000, dbias_beta=1.0)
    plan = L.plan(d)
    assert "cta-pair tile=256x256x64" in plan and "splits=2 " in plan
    assert "dbias_tickets=0 " in plan
    # one row of sums per split lives in the workspace, after the split-K partial sums
    assert L.workspace_bytes(d) == 2 * 2304 * 768 * 4 + 2 * 2304 * 4
    d.plan_cta_pairs = 1
    assert "1-cta tile=128x" in L.plan(d) and "dbias_tickets=0 " in L.plan(d)
    d.plan_cta_pairs = 0
    d.plan_splits = 1
    assert L.workspace_bytes(d) == 0  # unsplit: the tiles write dbias themselves
    # a batch keeps the ticket form: chunks of 64 rows of A over all columns, then finishing tickets
    bt = _desc(m=2304, n=768, k=8192, batch=2, trans_a=1, trans_b=0, lda=2304, ldb=768, ldc=768,
               stride_a=8192 * 2304, stride_b=8192 * 768, stride_c=2304 * 768,
               dtype_c=L.FP32, dbias=0x5000000)
    assert "dbias_tickets=133 " in L.plan(bt)
    # row sums (A stored [m, k]) need no second phase and no workspace
    r = _desc(m=2304, n=768, k=512, lda=512, ldb=512, ldc=768, dbias=0x5000000)
    assert "dbias_tickets=72 " in L.plan(r) and L.workspace_bytes(r) == 0


def test_ride_along_exchange_arguments_are_checked_before_anything_is_planned():
    """llmt_b200_gemm_grouped_exchange: a missing multicast mapping, a bad range, a bad index and a
    launch that writes the range it is asked to carry are refused on the host."""
    d = _desc(m=256, n=256, k=256, trans_a=0, trans_b=1, lda=256, ldb=256, ldc=256, dtype_c=L.FP32)
    descs = (L.GemmDesc * 1)(d)
    span = 0x7000000  # fake device addresses: no call below reaches a launch
    c = (ctypes.c_void_p * 1)(span + 4096)
    a = (ctypes.c_void_p * 1)(0x1000000)
    b = (ctypes.c_void_p * 1)(0x2000000)
    comm = L.CommDesc()
    comm.rank, comm.world = 0, 2
    for r in range(2):
        comm.grad[r] = span + r * 0x1000000
        comm.flags[r] = 0x9000000 + r * 0x10000
    lib = L.lib()

    def call(off, cnt, idx):
        return lib.llmt_b200_gemm_grouped_exchange(descs, c, a, b, 1, ctypes.byref(comm), off, cnt, idx, None)

    assert lib.llmt_b200_gemm_grouped_exchange(descs, c, a, b, 1, None, 0, 4, 0, None) == L.ERR_INVALID
    assert call(0, 1024, 0) == L.ERR_UNSUPPORTED and "multicast" in L.last_error()
    comm.grad_mc = 0xA000000
    assert call(2, 1024, 0) == L.ERR_INVALID and "multiples of 4" in L.last_error()
    assert call(0, 0, 0) == L.ERR_INVALID
    assert call(0, 1024, 16) == L.ERR_INVALID and "index" in L.last_error()
    # C of the problem starts 4096 bytes into the span: a range that reaches it is refused
    assert call(0, 2048, 0) == L.ERR_INVALID and "writes into the exchanged range" in L.last_error()
    comm.world = 1
    assert call(0, 1024, 0) == L.ERR_INVALID and "rank/world" in L.last_error()


def test_row_wise_epilogue_entry_points_check_their_arguments_first():
    """llmt_b200_gemm_softmax_fwd/_bwd, lm_head_ce_fwd/_bwd, cross_entropy_bwd, rowdot: every
    refusal below happens on the host, before anything is planned, encoded or launched."""
    lib = L.lib()
    P, Q, K, V = 0x100000, 0x200000, 0x300000, 0x400000
    ws = 0x800000

    def sm_desc(**kw):
        d = _desc(m=128, n=128, k=64, batch=2, lda=64, ldb=64, ldc=128, stride_a=128 * 64, stride_b=128 * 64,
                  stride_c=128 * 128, dtype_c=L.BF16, workspace=ws, workspace_bytes=1 << 20)
        for k, v in kw.items():
            setattr(d, k, v)
        return d

    def fwd(d, causal=1):
        return lib.llmt_b200_gemm_softmax_fwd(ctypes.byref(d), ctypes.c_void_p(P), ctypes.c_void_p(Q), ctypes.c_void_p(K),
                                              causal, None, None)

    assert fwd(sm_desc(n=256, ldc=256, stride_b=256 * 64, stride_c=128 * 256)) == L.ERR_INVALID and "square scores" in L.last_error()
    assert fwd(sm_desc(beta=1.0)) == L.ERR_UNSUPPORTED and "beta must be 0" in L.last_error()
    assert fwd(sm_desc(dtype_ab=L.FP32, dtype_c=L.FP32)) == L.ERR_UNSUPPORTED and "bf16 operands only" in L.last_error()
    assert fwd(sm_desc(epilogue=L.EPI_GELU)) == L.ERR_UNSUPPORTED
    assert fwd(sm_desc(workspace_bytes=0)) == L.ERR_WORKSPACE and "llmt_b200_gemm_softmax_workspace_bytes" in L.last_error()
    assert lib.llmt_b200_gemm_softmax_workspace_bytes(ctypes.byref(sm_desc()), None, None) > 2 * 128 * 8

    def bwd(d, probs=V, rowdot=0x500000, ds=P):
        return lib.llmt_b200_gemm_softmax_bwd(ctypes.byref(d), ctypes.c_void_p(ds), ctypes.c_void_p(Q), ctypes.c_void_p(K),
                                              ctypes.c_void_p(probs), ctypes.c_void_p(rowdot), 1, None)

    assert bwd(sm_desc(), probs=None) == L.ERR_INVALID and "null probabilities" in L.last_error()
    assert bwd(sm_desc(), probs=P + 64) == L.ERR_INVALID and "must not overlap" in L.last_error()

    def ce_desc(**kw):
        d = _desc(m=128, n=1000, k=64, lda=64, ldb=64, ldc=1000, workspace=ws, workspace_bytes=1 << 22)
        for k, v in kw.items():
            setattr(d, k, v)
        return d

    T, M_, NLL, LOSS = 0x600000, 0x610000, 0x620000, 0x630000
    ce_fwd = lambda d, targets=T: lib.llmt_b200_lm_head_ce_fwd(ctypes.byref(d), None, ctypes.c_void_p(Q), ctypes.c_void_p(K),
                                                              ctypes.c_void_p(targets), ctypes.c_void_p(M_),
                                                              ctypes.c_void_p(NLL), ctypes.c_void_p(LOSS), None)
    assert ce_fwd(ce_desc(), targets=None) == L.ERR_INVALID
    assert ce_fwd(ce_desc(batch=0)) == L.ERR_INVALID and "empty problem" in L.last_error()
    assert ce_fwd(ce_desc(beta=1.0)) == L.ERR_INVALID and "beta needs the logits" in L.last_error()
    assert ce_fwd(ce_desc(workspace_bytes=16)) == L.ERR_WORKSPACE
    ce_bwd = lambda d, dl=P: lib.llmt_b200_lm_head_ce_bwd(ctypes.byref(d), ctypes.c_void_p(dl), ctypes.c_void_p(Q), ctypes.c_void_p(K),
                                                         ctypes.c_void_p(T), ctypes.c_void_p(M_), 1.0, 0, None)
    assert ce_bwd(ce_desc(), dl=None) == L.ERR_INVALID
    assert ce_bwd(ce_desc(beta=0.5)) == L.ERR_UNSUPPORTED
    assert ce_bwd(ce_desc(workspace_bytes=16)) == L.ERR_WORKSPACE

    assert lib.llmt_b200_cross_entropy_bwd(ctypes.c_void_p(P), ctypes.c_void_p(P), ctypes.c_void_p(T), ctypes.c_void_p(M_),
                                           1.0, 8, 100, 100, 104, None) == L.ERR_INVALID and "one pitch" in L.last_error()
    assert lib.llmt_b200_cross_entropy_bwd(ctypes.c_void_p(P + 16), ctypes.c_void_p(P), ctypes.c_void_p(T), ctypes.c_void_p(M_),
                                           1.0, 8, 100, 100, 100, None) == L.ERR_INVALID and "overlap" in L.last_error()
    assert lib.llmt_b200_rowdot(ctypes.c_void_p(P), ctypes.c_void_p(Q), ctypes.c_void_p(K), 8, 64, 32, 64, L.BF16, None) == L.ERR_INVALID
    assert lib.llmt_b200_rowdot(ctypes.c_void_p(P), ctypes.c_void_p(Q), ctypes.c_void_p(K), 8, 64, 64, 64, 7, None) == L.ERR_UNSUPPORTED
    assert lib.llmt_b200_rowdot(ctypes.c_void_p(P), ctypes.c_void_p(Q), ctypes.c_void_p(K), 0, 64, 64, 64, L.BF16, None) == L.OK


def test_aux_epilogues_are_never_split_along_k():
    # a row-wise epilogue sees whole reductions: the plan of such a problem has one split, forced or not
    d = _desc(m=256, n=256, k=8192, lda=8192, ldb=8192, ldc=256, dtype_c=L.BF16)
    assert "splits=1" not in L.plan(d)            # alone, this shape is split
    d.epilogue, d.aux = L.EPI_GELU_BWD, 0x700000
    assert "splits=1" in L.plan(d)
    d.plan_splits = 4
    assert "splits=1" in L.plan(d)
