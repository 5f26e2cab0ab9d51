"""Flat-shard bookkeeping shared by every rotated module.

A rotated layer registers exactly one set of ordinary parameters (its own shard, e.g. ``linear.weight``
of shape ``[out/N, in]``), which keeps the per-rank ``state_dict`` identical to the reference's
(keys and shapes).  The parameters' storage is one contiguous flat buffer ``_full_param`` — the unit
that travels around the ring (the reference builds the same aliasing with ``set_full_param`` /
``allign_storage``, rtp/module/collectives.py:19-63, but needs N module replicas for it).

Moving the module (``.to()``, ``.cuda()``, ``.bfloat16()``) re-creates the flat buffer afterwards, so
dtype/device moves never break the aliasing.
"""
import copy
from typing import List

import torch
from torch import nn

from .context import RingContext, get_context
from .rotated import ShardLayout


class RotatedModule(nn.Module):
    """Base class: owns the flat shard buffer and the ring context."""

    inplace = False

    def _setup_ring(self, group=None, world_size=None, rank=None):
        self.ring: RingContext = get_context(group)
        if world_size is not None and world_size != self.ring.world:
            raise ValueError(f"world_size={world_size} does not match the process group ({self.ring.world})")
        if rank is not None and rank != self.ring.rank:
            raise ValueError(f"rank={rank} does not match the process group ({self.ring.rank})")
        self.world_size = self.ring.world
        self.rank = self.ring.rank
        self._displaced = False
        self._last_flat_grad = None

    @property
    def group(self):
        return self.ring.group

    # -- flat buffer ------------------------------------------------------------------------
    def shard_parameters(self) -> List[nn.Parameter]:
        """Parameters that make up the travelling shard, in flat-buffer order."""
        raise NotImplementedError

    def shard_names(self) -> List[str]:
        return [f"p{i}" for i in range(len(self.shard_parameters()))]

    def _flatten(self):
        params = self.shard_parameters()
        if not params:
            return
        dtype, device = params[0].dtype, params[0].device
        layout = ShardLayout([(n, p.shape) for n, p in zip(self.shard_names(), params)], dtype)
        flat = torch.zeros(layout.numel, dtype=dtype, device=device)
        with torch.no_grad():
            for v, p in zip(layout.views(flat), params):
                v.copy_(p.data)
                p.data = v
                p.rtp_sharded = True
        self._layout = layout
        self._full_param = flat
        if flat.is_cuda:
            from .engine import reserve_shard_bytes
            reserve_shard_bytes(layout.numel * flat.element_size())

    def _apply(self, fn, recurse=True):
        out = super()._apply(fn, recurse)
        if getattr(self, "_layout", None) is not None:
            self._flatten()
        return out

    def __deepcopy__(self, memo):
        # nn.Parameter.__deepcopy__ clones its data, which would detach the copies from the copied flat buffer
        new = self.__class__.__new__(self.__class__)
        memo[id(self)] = new
        for k, v in self.__dict__.items():
            new.__dict__[k] = copy.deepcopy(v, memo)
        if getattr(new, "_layout", None) is not None:
            new._flatten()
        return new

    @property
    def flat_param(self) -> torch.Tensor:
        return self._full_param

    def assert_home(self):
        if self._displaced:
            raise RuntimeError("in-place rotated layer is displaced: a forward in grad mode was not followed "
                               "by its backward; shards are not at their owners")
