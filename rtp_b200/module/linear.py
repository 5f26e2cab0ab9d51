"""Rotated linear layers.

``ColumnParallelLinear`` shards the weight by output rows (``[out/N, in]``) and concatenates the N
column blocks; ``RowParallelLinear`` shards by input columns (``[out, in/N]``), splits the input on
its last dim and sums the N partial products.  API and sharding rules follow the reference
(rtp/module/linear.py:137-236 and :307-392; shard classes :32-135).  On bf16 CUDA tensors the layers
run the fused sm_100a rotation kernel; otherwise the functional ring.
"""
from typing import Callable, Optional

import torch
import torch.nn.functional as F
from torch import nn
from torch.nn import init

from ..parallel.flat import RotatedModule
from ..parallel.rotated import rotated_apply
from ..parallel import fused
from .utils import affine_weight, divide_and_check_no_remainder


class ModelParallelLinear(nn.Linear):
    """One output-row shard ``[out/N, in]`` of a linear layer (reference: rtp/module/linear.py:32-82)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 world_size: int = 1, rank: int = 0):
        self.world_size, self.rank = world_size, rank
        self.full_in_features, self.full_out_features = in_features, out_features
        self.output_size_per_partition = divide_and_check_no_remainder(out_features, world_size)
        super().__init__(in_features, self.output_size_per_partition, bias=bias, device=device, dtype=dtype)

    def affine_weight(self, linear_layer: Optional[nn.Linear]):
        if linear_layer is None:
            return
        affine_weight(self.weight, linear_layer.weight, self.output_size_per_partition, 0, self.world_size, self.rank)
        if self.bias is not None and linear_layer.bias is not None:
            affine_weight(self.bias, linear_layer.bias, self.output_size_per_partition, 0, self.world_size, self.rank)


class ModelParallelLinear2(nn.Linear):
    """One input-column shard ``[out, in/N]``; the bias has full length and holds ``b / N`` so that the N
    partial products add up to one bias (reference: rtp/module/linear.py:84-135)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 world_size: int = 1, rank: int = 0):
        self.world_size, self.rank = world_size, rank
        self.full_in_features, self.full_out_features = in_features, out_features
        self.input_size_per_partition = divide_and_check_no_remainder(in_features, world_size)
        super().__init__(self.input_size_per_partition, out_features, bias=bias, device=device, dtype=dtype)
        if self.bias is not None:
            with torch.no_grad():
                self.bias.div_(world_size)
            self.bias.rtp_sum_replicated = world_size

    def affine_weight(self, linear_layer: Optional[nn.Linear]):
        if linear_layer is None:
            return
        affine_weight(self.weight, linear_layer.weight, self.input_size_per_partition, 1, self.world_size, self.rank)
        if self.bias is not None and linear_layer.bias is not None:
            with torch.no_grad():
                self.bias.copy_(linear_layer.bias / self.world_size)


class _RotatedLinearBase(RotatedModule):
    row = False

    def __init__(self, in_features: int, out_features: int, bias: bool = True, gather_weight: bool = True,
                 init_method: Callable[[torch.Tensor], torch.Tensor] = init.xavier_normal_, stride: int = 1,
                 keep_master_weight_for_test: bool = False, device=None, dtype=None, group=None,
                 linear_layer: Optional[nn.Linear] = None, world_size: Optional[int] = None,
                 rank: Optional[int] = None, packed_parts: int = 1):
        super().__init__()
        self._setup_ring(group, world_size, rank)
        # packed_parts > 1: the full weight stacks `packed_parts` equally sized projections along the output dim
        # (e.g. q, k, v) and every shard holds its slice of EACH of them: rows [p0_r; p1_r; ...]
        self.packed_parts = packed_parts
        self.in_features, self.out_features = in_features, out_features
        self.gather_weight = gather_weight
        cls = ModelParallelLinear2 if self.row else ModelParallelLinear
        self.linear = cls(in_features, out_features, bias=bias, device=device, dtype=dtype,
                          world_size=self.world_size, rank=self.rank)
        if self.row:
            self.input_size_per_partition = self.linear.input_size_per_partition
        else:
            self.output_size_per_partition = self.linear.output_size_per_partition
        self.linear.affine_weight(linear_layer)
        self._flatten()

    def shard_parameters(self):
        return [p for p in (self.linear.weight, self.linear.bias) if p is not None]

    def shard_names(self):
        return ["weight", "bias"][: len(self.shard_parameters())]

    def shard_spec(self):
        """How each registered tensor relates to the unsharded layer (used by rtp_b200.checkpoint)."""
        if self.row:
            spec = {"linear.weight": ("split", 1)}
            if self.linear.bias is not None:
                spec["linear.bias"] = ("sum",)
        else:
            rule = ("split", 0) if self.packed_parts == 1 else ("packed", 0, self.packed_parts)
            spec = {"linear.weight": rule}
            if self.linear.bias is not None:
                spec["linear.bias"] = rule
        return spec

    @property
    def linears(self):
        """The reference exposes N aliased replicas; here there is one shard module."""
        return [self.linear] * self.world_size

    def forward(self, input_: torch.Tensor) -> torch.Tensor:  # type: ignore
        if fused.use_fused(input_, self._full_param) and \
                fused.linear_ok(self.row, self.in_features, self.out_features, self.world_size):
            return fused.linear(self, input_, row=self.row)
        has_bias = self.linear.bias is not None
        if self.row:
            ks = self.input_size_per_partition

            def fn(j, views, x):
                return F.linear(x[..., j * ks:(j + 1) * ks], views[0], views[1] if has_bias else None)
            combine = "sum"
        else:
            def fn(j, views, x):
                return F.linear(x, views[0], views[1] if has_bias else None)
            combine = "cat"
        return rotated_apply(self.ring, fn, self.shard_parameters(), self._full_param, self._layout, (input_,),
                             combine=combine, cat_dim=-1, inplace=self.inplace, owner=self)


class ColumnParallelLinear(_RotatedLinearBase):
    """Y = X W^T + b with W sharded by output rows; every rank gets the full Y for its own batch."""
    row = False


class RowParallelLinear(_RotatedLinearBase):
    """Y = sum_j X[..., j] W_j^T + b with W sharded by input columns."""
    row = True
