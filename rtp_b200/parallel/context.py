"""Process-group context of a rotation ring.

The reference accepts ``group=`` in several constructors but its rotation primitives always use the
default group (rtp/module/collectives.py:84,204,223). Here every primitive takes the context, so a
sub-group ring works.
"""
import os
from dataclasses import dataclass
from typing import Optional

import torch.distributed as dist

_BACKEND = os.environ.get("RTP_BACKEND", "auto")  # auto | functional | fused


def set_backend(name: str):
    """Select how rotated layers execute: ``functional`` (torch.distributed send/recv + ATen; works on
    CPU/gloo and serves as oracle and NCCL baseline), ``fused`` (sm_100a kernels that push shards over
    NVLink from inside the GEMM), or ``auto`` (fused for bf16 CUDA tensors when available)."""
    global _BACKEND
    if name not in ("auto", "functional", "fused"):
        raise ValueError(name)
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


@dataclass(frozen=True)
class RingContext:
    group: Optional[object]
    rank: int
    world: int

    def __deepcopy__(self, memo):
        return self          # immutable; process groups cannot be copied or pickled

    def __reduce__(self):
        raise TypeError("a RingContext holds a process group and cannot be pickled")

    def global_rank(self, ring_rank: int) -> int:
        """Rank in the default group of ring member ``ring_rank`` (what isend/irecv expect)."""
        if self.group is None or not dist.is_initialized():
            return ring_rank
        return dist.get_global_rank(self.group, ring_rank) if self.group is not dist.group.WORLD else ring_rank

    @property
    def up(self) -> int:      # ring neighbour r+1
        return (self.rank + 1) % self.world

    @property
    def down(self) -> int:    # ring neighbour r-1
        return (self.rank - 1) % self.world


def get_context(group=None, world_size: Optional[int] = None, rank: Optional[int] = None) -> RingContext:
    """Context for ``group`` (default group when None). Without an initialised process group the ring
    has one member, which makes every rotated layer degenerate to its plain torch counterpart."""
    if dist.is_available() and dist.is_initialized():
        g = group if group is not None else dist.group.WORLD
        return RingContext(g, dist.get_rank(g), dist.get_world_size(g))
    if world_size not in (None, 1):
        raise RuntimeError("world_size > 1 requires an initialised torch.distributed process group")
    return RingContext(None, 0, 1)
