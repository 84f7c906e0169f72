"""Data-parallel host logic for the GEMM path: token-row sharding and the one
exchange step (sum of the per-GPU dW / dbias partial sums).

llmt has no multi-GPU code; its designed seam for it is the flat gradient span
of ParamStore (llmt include/llmt/model/param_store.h:131-135,185: "future NCCL —
one transfer each instead of one per tensor"). GradBucket is that span: every
dW and dbias of a step lives in one contiguous fp32 buffer so ONE all-reduce
covers them. Forward and dX need no communication (rows are independent and the
weights are replicated); gradients accumulate locally with beta = 1 (llmt
param_store.h:142-148) and are reduced once per step, never twice.

One process per GPU; the collective is torch.distributed (NCCL over NVLink on
GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Dict, Sequence, Tuple


def shard_rows(m: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous row range [start, stop) of an [m, .] tensor owned by `rank`.
    The first m % world ranks get one extra row; the union over ranks is [0, m)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world {world}")
    base, extra = divmod(m, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


class GradBucket:
    """Flat fp32 gradient span with named views, 256-byte aligned slices (the
    padding stays zero so it is inert under the sum)."""

    ALIGN_ELEMS = 64  # 256 bytes of fp32

    def __init__(self, shapes: Dict[str, Sequence[int]], device):
        import torch
        self.offsets = {}
        off = 0
        for name, shape in shapes.items():
            n = 1
            for e in shape:
                n *= int(e)
            self.offsets[name] = (off, n, tuple(int(e) for e in shape))
            off += (n + self.ALIGN_ELEMS - 1) // self.ALIGN_ELEMS * self.ALIGN_ELEMS
        self.flat = torch.zeros(off, dtype=torch.float32, device=device)

    def view(self, name: str):
        off, n, shape = self.offsets[name]
        return self.flat[off:off + n].view(shape)

    def zero_(self):
        self.flat.zero_()

    def nbytes(self) -> int:
        return self.flat.numel() * 4

    def allreduce(self, group=None, async_op: bool = False):
        """Sums the span over all ranks in place. Call once per step, after the
        last local accumulation."""
        import torch.distributed as dist
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return None
        return dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
