"""The multi-GPU path on CPU: world_size-2 gloo ranks shard the token rows, form
local dW / dbias partial sums (with the fp64 oracle standing in for the GPU
kernel) and sum them with one all-reduce of the flat gradient span."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llmt_b200.dp import GradBucket, shard_rows


def test_shard_rows_partition_is_exact():
    for m in (0, 1, 7, 8192, 65536, 50257):
        for world in (1, 2, 3, 4, 8):
            edges = [shard_rows(m, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == m
            for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
                assert a1 == b0 and a1 >= a0
            sizes = [b - a for a, b in edges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_rows(8, 2, 2)


def test_grad_bucket_layout():
    b = GradBucket({"w": (10, 12), "b": (10,), "w2": (3, 5)}, "cpu")
    assert b.view("w").shape == (10, 12) and b.view("b").shape == (10,)
    offs = [b.offsets[n][0] for n in ("w", "b", "w2")]
    assert offs == sorted(offs) and all(o % GradBucket.ALIGN_ELEMS == 0 for o in offs)
    b.view("b").fill_(2.0)
    assert float(b.flat.sum()) == 20.0  # views alias the flat span; padding is zero
    b.zero_()
    assert float(b.flat.abs().sum()) == 0.0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle
    M, OUT, IN = 96, 10, 12
    rng = np.random.default_rng(0)  # same seed everywhere: every rank can form any shard
    x = oracle.round_bf16(rng.standard_normal((M, IN)))
    dy = oracle.round_bf16(rng.standard_normal((M, OUT)) * 0.01)
    lo, hi = shard_rows(M, rank, world)
    bucket = GradBucket({"dW": (OUT, IN), "dbias": (OUT,)}, "cpu")
    # two local accumulations (beta = 1) before the single reduction
    for _ in range(2):
        part = oracle.gemm(dy[lo:hi], x[lo:hi], trans_a=True, beta=1.0, c=bucket.view("dW").numpy())
        bucket.view("dW").copy_(torch.from_numpy(part.astype(np.float32)))
        db = oracle.rowsum(dy[lo:hi], trans_a=True, out=bucket.view("dbias").numpy(), out_beta=1.0)
        bucket.view("dbias").copy_(torch.from_numpy(db.astype(np.float32)))
    bucket.allreduce()
    full_dw = 2.0 * oracle.gemm(dy, x, trans_a=True)
    full_db = 2.0 * oracle.rowsum(dy, trans_a=True)
    ok = (oracle.rel_fro(bucket.view("dW").numpy(), full_dw) < 1e-6
          and oracle.rel_fro(bucket.view("dbias").numpy(), full_db) < 1e-6)
    # every rank holds the same bits after the reduction
    gathered = [torch.empty_like(bucket.flat) for _ in range(world)]
    dist.all_gather(gathered, bucket.flat)
    same = all(torch.equal(gathered[0], g) for g in gathered)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("ok" if (ok and same) else f"bad ok={ok} same={same}")
    dist.destroy_process_group()


def test_two_rank_sharded_dw_allreduce(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"
