"""Host logic of the multi-GPU path: one process per GPU, the batch (or Linear row) dimension is
sharded, forward and input-gradient need no exchange, weight and bias gradients are sums over the
batch and are all-reduced.  The reference has no multi-device code (its README states
single-device training only); this is the one exchange step the sharded path needs.

Works with any torch.distributed backend: NCCL on GPUs, gloo on CPU (which is how it is tested
without GPUs).
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced shard of ``total`` samples: returns (start, count).  The first
    ``total % world`` ranks get one extra sample; ranks beyond ``total`` get an empty shard."""
    if world <= 0 or not (0 <= rank < world) or total < 0:
        raise ValueError(f"bad shard request total={total} world={world} rank={rank}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


class GradientBucket:
    """Flat fp32 buffer the weight / bias gradients of several layers are packed into so that one
    all-reduce moves them all (collective cost on NVSwitch is latency-, not link-bound, so few
    large buckets beat many small ones)."""

    def __init__(self, shapes: Iterable[Tuple[int, ...]], device) -> None:
        self.shapes: List[Tuple[int, ...]] = [tuple(s) for s in shapes]
        self.offsets: List[int] = []
        n = 0
        for s in self.shapes:
            self.offsets.append(n)
            cnt = 1
            for d in s:
                cnt *= d
            n += (cnt + 63) // 64 * 64  # keep every view 256-byte aligned
        self.flat = torch.zeros(n, dtype=torch.float32, device=device)

    def view(self, i: int) -> torch.Tensor:
        cnt = 1
        for d in self.shapes[i]:
            cnt *= d
        return self.flat[self.offsets[i]:self.offsets[i] + cnt].view(self.shapes[i])

    def all_reduce(self, group: Optional[dist.ProcessGroup] = None, average: bool = False, async_op: bool = False):
        """Sums (or averages) the bucket over the ranks; a no-op without an initialised group."""
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return None
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        if average:
            if async_op:
                work.wait()
                work = None
            self.flat.div_(dist.get_world_size(group))
        return work
