"""Data-parallel host logic for the GEMM path: token-row sharding and the one
exchange step (sum of the per-GPU dW / dbias partial sums).

llmt has no multi-GPU code; its designed seam for it is the flat gradient span
of ParamStore (llmt include/llmt/model/param_store.h:131-135,185: "future NCCL —
one transfer each instead of one per tensor"). GradBucket is that span: every
dW and dbias of a step lives in one contiguous fp32 buffer so ONE all-reduce
covers them. Forward and dX need no communication (rows are independent and the
weights are replicated); gradients accumulate locally with beta = 1 (llmt
param_store.h:142-148) and are reduced once per step, never twice.

One process per GPU.  Two ways to sum the span: torch.distributed (NCCL on GPUs,
gloo in the CPU tests), or PeerExchange — the library's own all-reduce kernel over
NVLink peer memory, which runs on a few SMs beside the persistent GEMM kernels.
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

    def __init__(self, shapes: Dict[str, Sequence[int]], device, storage=None):
        """storage: optional callable numel -> zeroed fp32 tensor (e.g. PeerExchange.attach,
        which places the span in peer-mapped memory)."""
        import torch
        self.offsets = {}
        off = 0
        for name, shape in shapes.items():
            n = 1
            for e in shape:
                n *= int(e)
            self.offsets[name] = (off, n, tuple(int(e) for e in shape))
            off += (n + self.ALIGN_ELEMS - 1) // self.ALIGN_ELEMS * self.ALIGN_ELEMS
        self.flat = storage(off) if storage is not None else torch.zeros(off, dtype=torch.float32, device=device)
        if self.flat.numel() != off or self.flat.dtype != torch.float32:
            raise ValueError("storage() must return an fp32 tensor of the requested length")

    @staticmethod
    def layout_numel(shapes: Dict[str, Sequence[int]]) -> int:
        """Length of the flat span GradBucket(shapes) would allocate."""
        off = 0
        for shape in shapes.values():
            n = 1
            for e in shape:
                n *= int(e)
            off += (n + GradBucket.ALIGN_ELEMS - 1) // GradBucket.ALIGN_ELEMS * GradBucket.ALIGN_ELEMS
        return off

    def span_of(self, names: Sequence[str]) -> Tuple[int, int]:
        """(offset, count) of the smallest aligned range covering the named entries."""
        lo = min(self.offsets[n][0] for n in names)
        hi = max(self.offsets[n][0] + self.offsets[n][1] for n in names)
        hi = (hi + self.ALIGN_ELEMS - 1) // self.ALIGN_ELEMS * self.ALIGN_ELEMS
        return lo, hi - lo

    def view(self, name: str):
        off, n, shape = self.offsets[name]
        return self.flat[off:off + n].view(shape)

    def zero_(self):
        if self.flat.is_cuda:
            from . import zero_grads
            zero_grads(self.flat)
        else:
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


def exchange_layout(numel: int, world: int) -> Dict[str, int]:
    """Byte layout of one rank's peer-mapped allocation for PeerExchange: the span, then
    `world` staging slots (one shard each, rounded up to 256 bytes), then the flag words."""
    from . import COMM_FLAG_BYTES
    if numel % 4 != 0:
        raise ValueError("span length must be a multiple of 4 floats")
    shard = (numel // 4 + world - 1) // world * 4
    slot = (shard + 63) // 64 * 64
    grad_bytes = (numel * 4 + 255) // 256 * 256
    stage_bytes = world * slot * 4
    return {"slot_elems": slot, "grad_off": 0, "stage_off": grad_bytes,
            "flags_off": grad_bytes + stage_bytes, "total": grad_bytes + stage_bytes + COMM_FLAG_BYTES}


class PeerExchange:
    """The span in peer-mapped memory plus the library's all-reduce kernel over it.

    Usage: ex = PeerExchange(numel, device); bucket = GradBucket(shapes, device, storage=ex.attach);
    ex.allreduce(offset, count) on the stream that must see the sum (calls of one exchange
    must not overlap: keep them on one stream).  Every rank makes the same calls."""

    def __init__(self, numel: int, device, group=None, ctas: int = 8, multicast: bool = False):
        """multicast=False: plain peer loads and stores, no NVLink multicast object is bound to
        the span.  multicast=True: ask the allocator for an NVSwitch multicast mapping and, when
        it provides one, let the switch form and broadcast the sums (self.multicast tells)."""
        import os
        import torch
        import torch.distributed as dist
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "0" if multicast else "1"
        import torch.distributed._symmetric_memory as symm
        from . import CommDesc, COMM_EPOCH_BYTES
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.ctas, self.numel = int(ctas), int(numel)
        lay = exchange_layout(numel, self.world)
        self.buf = symm.empty(lay["total"], dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = torch.zeros(COMM_EPOCH_BYTES // 4, dtype=torch.int32, device=device)
        d = CommDesc()
        d.rank, d.world, d.slot_elems = self.rank, self.world, lay["slot_elems"]
        for r in range(self.world):
            d.grad[r] = ptrs[r] + lay["grad_off"]
            d.stage[r] = ptrs[r] + lay["stage_off"]
            d.flags[r] = ptrs[r] + lay["flags_off"]
        d.epoch = self.epoch.data_ptr()
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0) if multicast else 0
        self.multicast = mc != 0
        d.grad_mc = (mc + lay["grad_off"]) if mc else None
        self.desc = d
        self.flat = self.buf[:numel * 4].view(torch.float32)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # nobody raises a flag before every rank has zeroed its own

    def attach(self, numel: int):
        if numel != self.numel:
            raise ValueError(f"exchange was sized for {self.numel} floats, span has {numel}")
        return self.flat

    def allreduce(self, offset: int = 0, count: int = None, stream=None):
        from . import grad_allreduce
        grad_allreduce(self.desc, offset, self.numel if count is None else count, self.ctas, stream)
