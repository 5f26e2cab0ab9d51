"""Collective helpers with the reference's names (rtp/module/collectives.py).

Two families:
  * classic tensor-parallel regions (copy / gather / reduce / shift), each an ``autograd.Function`` whose
    backward is the transposed collective (reference lines 428-590);
  * flat-buffer helpers (``set_full_param``, ``allign_storage``, ``allign_grad``, ``zero_full_grads`` ...)
    that expose the rotation engine's bookkeeping under the reference's vocabulary.
All collectives honour an optional ``group``.
"""
from typing import Optional

import torch
import torch.distributed as dist

from ..parallel.context import get_context
from ..parallel.flat import RotatedModule
from ..parallel import ring as _ring


def _world(group=None):
    return get_context(group)


def _reduce(input_: torch.Tensor, group=None) -> torch.Tensor:
    ctx = _world(group)
    if ctx.world == 1:
        return input_
    dist.all_reduce(input_, group=ctx.group)
    return input_


def _split(input_: torch.Tensor, group=None, dim: int = -1) -> torch.Tensor:
    ctx = _world(group)
    if ctx.world == 1:
        return input_
    return torch.chunk(input_, ctx.world, dim=dim)[ctx.rank].contiguous()


def _gather(input_: torch.Tensor, group=None, dim: int = -1) -> torch.Tensor:
    ctx = _world(group)
    if ctx.world == 1:
        return input_
    parts = [torch.empty_like(input_) for _ in range(ctx.world)]
    parts[ctx.rank] = input_
    dist.all_gather(parts, input_.contiguous(), group=ctx.group)
    return torch.cat(parts, dim=dim).contiguous()


class _CopyToModelParallelRegion(torch.autograd.Function):
    """Identity forward, all-reduce backward."""

    @staticmethod
    def forward(ctx, input_, group=None):
        ctx.group = group
        return input_

    @staticmethod
    def backward(ctx, grad_output):
        return _reduce(grad_output.contiguous().clone(), ctx.group), None


class _ReduceFromModelParallelRegion(torch.autograd.Function):
    """All-reduce forward, identity backward."""

    @staticmethod
    def forward(ctx, input_, group=None):
        return _reduce(input_.clone(), group)

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output, None


class _GatherFromModelParallelRegion(torch.autograd.Function):
    """All-gather along the last dim forward, split backward."""

    @staticmethod
    def forward(ctx, input_, group=None):
        ctx.group = group
        return _gather(input_, group, dim=-1)

    @staticmethod
    def backward(ctx, grad_output):
        return _split(grad_output, ctx.group, dim=-1), None


class _GatherFromConvParallelRegion(torch.autograd.Function):
    """All-gather along the channel dim (1) forward, split backward."""

    @staticmethod
    def forward(ctx, input_, group=None):
        ctx.group = group
        return _gather(input_, group, dim=1)

    @staticmethod
    def backward(ctx, grad_output):
        return _split(grad_output, ctx.group, dim=1), None


class _ShiftToModelParallelRegion(torch.autograd.Function):
    """Ring shift forward (receive the neighbour's tensor), opposite shift backward."""

    @staticmethod
    def forward(ctx, input_, group=None):
        ctx.group = group
        rc = _world(group)
        out = torch.empty_like(input_)
        _ring.wait_all(_ring.shift_async(rc, input_.contiguous(), out, "up"))
        return out

    @staticmethod
    def backward(ctx, grad_output):
        rc = _world(ctx.group)
        out = torch.empty_like(grad_output)
        _ring.wait_all(_ring.shift_async(rc, grad_output.contiguous(), out, "down"))
        return out, None


def copy_to_model_parallel_region(input_: torch.Tensor, group=None) -> torch.Tensor:
    return _CopyToModelParallelRegion.apply(input_, group)


def gather_from_model_parallel_region(input_: torch.Tensor, group=None) -> torch.Tensor:
    return _GatherFromModelParallelRegion.apply(input_, group)


def gather_from_conv_parallel_region(input_: torch.Tensor, group=None) -> torch.Tensor:
    return _GatherFromConvParallelRegion.apply(input_, group)


def reduce_from_model_parallel_region(input_: torch.Tensor, group=None) -> torch.Tensor:
    return _ReduceFromModelParallelRegion.apply(input_, group)


def shift_to_model_parallel_region(input_: torch.Tensor, group=None) -> torch.Tensor:
    return _ShiftToModelParallelRegion.apply(input_, group)


# ---------------------------------------------------------------------------------------------------
# flat-buffer helpers under the reference's names
# ---------------------------------------------------------------------------------------------------
def _rotated(module) -> Optional[RotatedModule]:
    return module if isinstance(module, RotatedModule) else None


def set_full_param(module, device=None, dtype=None):
    """(Re)build the flat shard buffer of a rotated module; its parameters become views of it."""
    m = _rotated(module)
    if m is None:
        raise TypeError("set_full_param expects a rotated module")
    if device is not None or dtype is not None:
        m.to(device=device, dtype=dtype)
    else:
        m._flatten()
    return m._full_param


def set_full_param2(module, device, dtype, full_param):
    """Alias a rotated module onto an existing flat buffer of the same layout."""
    m = _rotated(module)
    with torch.no_grad():
        m._full_param.copy_(full_param.to(m._full_param.dtype))
    return m._full_param


def allign_storage(module):
    """Re-point the parameters at their slices of the flat buffer."""
    m = _rotated(module)
    for v, p in zip(m._layout.views(m._full_param), m.shard_parameters()):
        p.data = v


def allign_grad(module):
    """Expose the ring-reduced flat gradient of the last backward as views in ``param.grad``."""
    m = _rotated(module)
    if m._last_flat_grad is None:
        return
    for v, p in zip(m._layout.views(m._last_flat_grad), m.shard_parameters()):
        p.grad = v


def free_storage(module):
    """No-op: visitors live in engine-owned work buffers that are released after each call."""


def free_grad(module):
    m = _rotated(module)
    m._last_flat_grad = None
    for p in m.shard_parameters():
        p.grad = None


def zero_full_grads(module):
    """Drop the gradients of every rotated layer below ``module`` (the reference's version never finds its
    list-held replicas and does nothing)."""
    for m in module.modules():
        if isinstance(m, RotatedModule):
            free_grad(m)
