"""The gradient all-reduce kernel (llmt_b200_grad_allreduce): every rank's partial sums of the
flat fp32 span are added in rank order and all ranks end with the same bits.

On one GPU the ranks are emulated inside one cooperative launch (every pointer local); with
two or more GPUs the real path runs as one process per GPU over peer-mapped memory."""
import os
import socket

import pytest
import torch

import llmt_b200 as L
from llmt_b200.dp import exchange_layout

pytestmark = pytest.mark.gpu


def _emulated(world, numel, dev):
    lay = exchange_layout(numel, world)
    bufs = [torch.zeros(lay["total"], dtype=torch.uint8, device=dev) for _ in range(world)]
    epochs = [torch.zeros(L.COMM_EPOCH_BYTES // 4, dtype=torch.int32, device=dev) for _ in range(world)]
    descs = []
    for r in range(world):
        d = L.CommDesc()
        d.rank, d.world, d.slot_elems = r, world, lay["slot_elems"]
        for p in range(world):
            d.grad[p] = bufs[p].data_ptr() + lay["grad_off"]
            d.stage[p] = bufs[p].data_ptr() + lay["stage_off"]
            d.flags[p] = bufs[p].data_ptr() + lay["flags_off"]
        d.epoch = epochs[r].data_ptr()
        descs.append(d)
    spans = [b[:numel * 4].view(torch.float32) for b in bufs]
    return descs, spans, (bufs, epochs)


def _rank_order_sum(parts):
    acc = parts[0].clone()
    for p in parts[1:]:
        acc += p
    return acc


@pytest.mark.parametrize("world,ctas,numel,offset,count", [
    (2, 1, 4096, 0, 4096),
    (2, 4, 1 << 20, 64, (1 << 20) - 128),
    (3, 4, 40000, 128, 4 * 1237),     # shards that do not divide evenly; the last one short
    (8, 4, 1 << 20, 0, 1 << 20),
    (8, 3, 4096, 0, 36),              # fewer float4s than ranks * ctas: empty shards and slices
    (5, 2, 7 * 64, 64, 64),
])
def test_emulated_ranks_sum_in_rank_order(world, ctas, numel, offset, count):
    dev = torch.device("cuda", 0)
    descs, spans, keep = _emulated(world, numel, dev)
    g = torch.Generator(device=dev).manual_seed(world * 1000 + ctas)
    for call in range(3):  # call counters advance: the same buffers serve call after call
        parts = [torch.randn(numel, device=dev, generator=g) * (1.0 + r) for r in range(world)]
        for s, p in zip(spans, parts):
            s.copy_(p)
        L.grad_allreduce_emulated(descs, offset, count, ctas)
        L.device_status()
        want = _rank_order_sum([p[offset:offset + count] for p in parts])
        for r in range(world):
            assert torch.equal(spans[r][offset:offset + count], want), (call, r)
            # outside the range every rank keeps its own values
            assert torch.equal(spans[r][:offset], parts[r][:offset])
            assert torch.equal(spans[r][offset + count:], parts[r][offset + count:])


def test_single_rank_and_empty_range_launch_nothing():
    dev = torch.device("cuda", 0)
    descs, spans, keep = _emulated(1, 256, dev)
    spans[0].fill_(3.0)
    n0 = L.launch_count()
    L.grad_allreduce(descs[0], 0, 256, 4)
    descs2, spans2, keep2 = _emulated(2, 256, dev)
    L.grad_allreduce_emulated(descs2, 0, 0, 4)
    assert L.launch_count() == n0
    assert float(spans[0].sum()) == 3.0 * 256


def test_rejects_bad_arguments():
    dev = torch.device("cuda", 0)
    descs, spans, keep = _emulated(2, 256, dev)
    for off, cnt, ctas, status in [(2, 8, 4, L.ERR_UNSUPPORTED), (0, 6, 4, L.ERR_UNSUPPORTED),
                                   (0, 8, 0, L.ERR_INVALID), (0, 8, L.COMM_MAX_CTAS + 1, L.ERR_INVALID),
                                   (0, 100000, 4, L.ERR_WORKSPACE)]:
        with pytest.raises(L.LlmtB200Error) as ei:
            L.grad_allreduce_emulated(descs, off, cnt, ctas)
        assert ei.value.status == status, (off, cnt, ctas)
    descs[1].rank = 0
    with pytest.raises(L.LlmtB200Error):
        L.grad_allreduce_emulated(descs, 0, 8, 4)


def test_a_peer_that_never_arrives_ends_the_wait_with_a_status_not_a_hang():
    """The plain (one rank per launch) kernel as rank 0 of a world of 2 whose 'peer' buffers are
    local and whose peer never runs: rank 1's flags are never raised.  With the wait limit
    lowered to 50 ms the kernel gives up, finishes, and the host reads ERR_DEVICE with
    DEV_WAIT_PEER; nothing faults, nothing waits for ever, and the context stays usable."""
    dev = torch.device("cuda", 0)
    descs, spans, keep = _emulated(2, 4096, dev)
    assert descs[0].grad_mc is None  # peer-copy form: no multicast object is involved
    L.set_wait_limit_ns(exchange_ns=50_000_000)
    try:
        L.grad_allreduce(descs[0], 0, 4096, 2)
        with pytest.raises(L.LlmtB200Error) as ei:
            L.device_status()
    finally:
        L.set_wait_limit_ns(exchange_ns=4_000_000_000)
    assert ei.value.status == L.ERR_DEVICE
    assert f"code {L.DEV_WAIT_PEER} " in str(ei.value)
    assert L.device_status() == (0, 0)  # reading the word cleared it
    # the same context afterwards: a complete exchange on fresh buffers, and an ordinary GEMM
    descs2, spans2, keep2 = _emulated(2, 4096, dev)
    parts = [torch.full((4096,), float(r + 1), device=dev) for r in range(2)]
    for s_, p_ in zip(spans2, parts):
        s_.copy_(p_)
    L.grad_allreduce_emulated(descs2, 0, 4096, 2)
    assert L.device_status() == (0, 0)
    assert torch.equal(spans2[0], parts[0] + parts[1]) and torch.equal(spans2[1], spans2[0])
    a = torch.ones(256, 64, device=dev, dtype=torch.bfloat16)
    c = torch.empty(256, 256, device=dev)
    L.gemm(c, a, torch.ones(256, 64, device=dev, dtype=torch.bfloat16), False, True)
    assert L.device_status() == (0, 0)
    assert torch.equal(c, torch.full_like(c, 64.0))


# ---- the real path: one process per GPU --------------------------------------------------

def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _peer_worker(rank, world, port, out_dir, multicast=False):
    import torch.distributed as dist
    from llmt_b200.dp import GradBucket, PeerExchange
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    msg = "ok"
    try:
        shapes = {"a.dW": (768, 2304), "a.dbias": (2304,), "b.dW": (100, 52), "b.dbias": (100,)}
        ex = PeerExchange(GradBucket.layout_numel(shapes), dev, ctas=4, multicast=multicast)
        if multicast and not ex.multicast:
            msg = "no multicast"
        bucket = GradBucket(shapes, dev, storage=ex.attach)
        g = torch.Generator(device=dev).manual_seed(7)  # same stream of numbers on every rank
        for call in range(3):
            parts = [torch.randn(bucket.flat.numel(), device=dev, generator=g) * (1.0 + r) for r in range(world)]
            bucket.flat.copy_(parts[rank])
            dist.barrier()
            off, cnt = bucket.span_of(["a.dW", "a.dbias"])
            ex.allreduce(off, cnt)
            off2, cnt2 = bucket.span_of(["b.dW", "b.dbias"])
            ex.allreduce(off2, cnt2)
            L.device_status()
            want = _rank_order_sum(parts)
            same = torch.equal(bucket.flat, want) if world == 2 or not ex.multicast else \
                torch.allclose(bucket.flat, want, rtol=1e-6, atol=1e-6)  # the switch's order of additions
            if not same:
                msg = f"call {call}: mismatch, max abs err {float((bucket.flat - want).abs().max())}"
                break
            # the same partial sums again: the exchange must reproduce its own bits
            first = bucket.flat.clone()
            bucket.flat.copy_(parts[rank])
            dist.barrier()
            ex.allreduce(off, cnt)
            ex.allreduce(off2, cnt2)
            L.device_status()
            if not torch.equal(bucket.flat, first):
                msg = f"call {call}: rerun differs"
                break
        gathered = [torch.empty_like(bucket.flat) for _ in range(world)]
        dist.all_gather(gathered, bucket.flat)
        if not all(torch.equal(gathered[0], t) for t in gathered):
            msg = "ranks disagree"
        dist.barrier()
    except Exception as exc:  # noqa: BLE001 - report instead of hanging the parent
        msg = f"exception: {exc!r}"
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(msg)
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_over_peer_memory(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_peer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_through_switch_multicast(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_peer_worker, args=(world, _free_port(), str(tmp_path), True), nprocs=world, join=True)
    texts = [(tmp_path / f"rank{r}.txt").read_text() for r in range(world)]
    if all(t == "no multicast" for t in texts):
        pytest.skip("the allocator offers no multicast mapping on this machine")
    assert texts == ["ok"] * world


def _ride_worker(rank, world, port, out_dir):
    """A range of the span rides inside a grouped GEMM launch (llmt_b200_gemm_grouped_exchange): the
    launch's own result and the exchanged range are both checked, three steps in a row and once
    more on the same inputs (bitwise)."""
    import torch.distributed as dist
    from llmt_b200.dp import GradBucket, PeerExchange
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    msg = "ok"
    try:
        shapes = {"a.dW": (768, 2304), "a.dbias": (2304,), "b.dW": (512, 384), "b.dbias": (512,)}
        ex = PeerExchange(GradBucket.layout_numel(shapes), dev, ctas=8, multicast=True)
        if not ex.multicast:
            msg = "no multicast"
        else:
            bucket = GradBucket(shapes, dev, storage=ex.attach)
            g = torch.Generator(device=dev).manual_seed(11)  # same stream of numbers on every rank
            bf = torch.bfloat16
            # the launch that carries slice a: dW and dbias of layer b (written into slice b) plus an unrelated product
            dy = [(torch.randn(1024, 512, device=dev, generator=g) * 0.1).to(bf) for _ in range(world)][rank]
            x = [(torch.randn(1024, 384, device=dev, generator=g)).to(bf) for _ in range(world)][rank]
            w = (torch.randn(512, 384, device=dev, generator=g) * 0.05).to(bf)
            dx = torch.empty(1024, 384, device=dev, dtype=bf)
            dw, db = bucket.view("b.dW"), bucket.view("b.dbias")
            probs = [(L.make_desc(dx, dy, w, False, False), dx, dy, w),
                     (L.make_desc(dw, dy, x, True, False, beta=1.0, dbias=db, dbias_beta=1.0), dw, dy, x)]
            grp = L.Group(probs)
            bufs = [torch.empty(max(b_, 256), dtype=torch.uint8, device=dev) for b_ in grp.workspace_bytes()]
            grp.set_workspaces(bufs)
            off_a, cnt_a = bucket.span_of(["a.dW", "a.dbias"])
            off_b, cnt_b = bucket.span_of(["b.dW", "b.dbias"])
            # a launch that writes the range it is asked to carry is refused
            try:
                grp.run_with_exchange(ex.desc, off_b, cnt_b, 0)
                msg = "a launch that writes the exchanged range was accepted"
            except L.LlmtB200Error as exc:
                if exc.status != L.ERR_INVALID:
                    msg = f"unexpected status {exc.status}"
            for call in range(3):
                if msg != "ok":
                    break
                parts = [torch.randn(bucket.flat.numel(), device=dev, generator=g) * (1.0 + r) for r in range(world)]

                def step():
                    bucket.flat.copy_(parts[rank])
                    torch.cuda.synchronize(); dist.barrier()
                    L.exchange_begin_step(ex.desc)
                    grp.run_with_exchange(ex.desc, off_a, cnt_a, 0)   # slice a rides, slice b is produced
                    ex.allreduce(off_b, cnt_b)                        # the last slice, and the step's closing rounds
                    torch.cuda.synchronize(); dist.barrier()
                    L.device_status()
                    return bucket.flat.clone()

                got = step()
                # reference for slice b: start + this rank's dW/dbias, summed over the ranks
                bucket.flat.copy_(parts[rank])
                grp.run()
                torch.cuda.synchronize()
                local_b = bucket.flat[off_b:off_b + cnt_b].clone()
                gathered = [torch.empty_like(local_b) for _ in range(world)]
                dist.all_gather(gathered, local_b)
                want_b = _rank_order_sum(gathered)
                want_a = _rank_order_sum([p_[off_a:off_a + cnt_a] for p_ in parts])
                ok_a = torch.equal(got[off_a:off_a + cnt_a], want_a) if world == 2 else \
                    torch.allclose(got[off_a:off_a + cnt_a], want_a, rtol=1e-6, atol=1e-6)
                ok_b = torch.equal(got[off_b:off_b + cnt_b], want_b) if world == 2 else \
                    torch.allclose(got[off_b:off_b + cnt_b], want_b, rtol=1e-6, atol=1e-6)
                if not (ok_a and ok_b):
                    msg = f"call {call}: mismatch (carried range ok={ok_a}, produced range ok={ok_b})"
                    break
                if not torch.equal(step(), got):
                    msg = f"call {call}: rerun differs"
                    break
            if msg == "ok":
                gathered = [torch.empty_like(bucket.flat) for _ in range(world)]
                dist.all_gather(gathered, bucket.flat)
                if not all(torch.equal(gathered[0], t) for t in gathered):
                    msg = "ranks disagree"
        dist.barrier()
    except Exception as exc:  # noqa: BLE001 - report instead of hanging the parent
        msg = f"exception: {exc!r}"
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(msg)
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_exchange_riding_inside_a_grouped_launch(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_ride_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    texts = [(tmp_path / f"rank{r}.txt").read_text() for r in range(world)]
    if all(t == "no multicast" for t in texts):
        pytest.skip("the allocator offers no multicast mapping on this machine")
    assert texts == ["ok"] * world


@pytest.mark.parametrize("offset,count", [(0, 4096), (1, 1031), (3, 5), (2, 0), (0, 7080960)])
def test_zero_grads_clears_exactly_the_span(offset, count):
    dev = torch.device("cuda", 0)
    buf = torch.ones(offset + count + 9, device=dev)
    n0 = L.launch_count()
    L.zero_grads(buf[offset:offset + count])
    torch.cuda.synchronize()
    assert L.launch_count() - n0 == (1 if count else 0)
    assert float(buf[offset:offset + count].abs().sum()) == 0.0
    assert float(buf[:offset].sum()) == offset and float(buf[offset + count:].sum()) == 9.0
    with pytest.raises(L.LlmtB200Error):
        L.zero_grads(torch.ones(8, device=dev, dtype=torch.bfloat16))
