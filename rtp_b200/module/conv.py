"""Rotated Conv2d: output channels are sharded (``[Cout/N, Cin, kh, kw]``) and the N channel blocks are
concatenated on dim 1 (reference: rtp/module/conv.py:17-129)."""
from typing import Optional

import torch
from torch import nn

from ..parallel import fused
from ..parallel.flat import RotatedModule
from ..parallel.rotated import rotated_apply
from .utils import affine_weight, divide_and_check_no_remainder


class ModelParallelConv2d(nn.Conv2d):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode="zeros", device=None, dtype=None, world_size=1, rank=0):
        self.world_size, self.rank = world_size, rank
        self.full_out_channels = out_channels
        self.out_channels_per_partition = divide_and_check_no_remainder(out_channels, world_size)
        super().__init__(in_channels, self.out_channels_per_partition, kernel_size, stride, padding, dilation, groups,
                         bias, padding_mode, device, dtype)

    def affine_weight(self, Conv2d_layer: Optional[nn.Conv2d]):
        if Conv2d_layer is None:
            return
        affine_weight(self.weight, Conv2d_layer.weight, self.out_channels_per_partition, 0, self.world_size, self.rank)
        if self.bias is not None and Conv2d_layer.bias is not None:
            affine_weight(self.bias, Conv2d_layer.bias, self.out_channels_per_partition, 0, self.world_size, self.rank)


class ColumnParallelConv2d(RotatedModule):
    def __init__(self, in_channels, out_channels, kernel_size, stride=1, padding=0, dilation=1, groups=1, bias=True,
                 padding_mode="zeros", device=None, dtype=None, group=None, gather_output=True, Conv2d_layer=None,
                 world_size=None, rank=None):
        super().__init__()
        self._setup_ring(group, world_size, rank)
        self.in_channels, self.out_channels = in_channels, out_channels
        self.conv = ModelParallelConv2d(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                                        padding_mode, device, dtype, world_size=self.world_size, rank=self.rank)
        self.conv.affine_weight(Conv2d_layer)
        self._flatten()

    def shard_parameters(self):
        return [p for p in (self.conv.weight, self.conv.bias) if p is not None]

    def shard_names(self):
        return ["weight", "bias"][: len(self.shard_parameters())]

    def shard_spec(self):
        spec = {"conv.weight": ("split", 0)}
        if self.conv.bias is not None:
            spec["conv.bias"] = ("split", 0)
        return spec

    @property
    def convs(self):
        return [self.conv] * self.world_size

    def forward(self, input_: torch.Tensor) -> torch.Tensor:  # type: ignore
        conv = self.conv
        has_bias = conv.bias is not None
        if fused.use_fused(input_, self._full_param) and not (self.inplace and self.world_size > 1):
            from ..parallel import engine
            if engine.fused_conv_ok(conv, input_):
                return engine.fused_conv(self, conv, input_)

        def fn(j, views, x):
            # nn.Conv2d._conv_forward handles every padding_mode
            return conv._conv_forward(x, views[0], views[1] if has_bias else None)
        return rotated_apply(self.ring, fn, self.shard_parameters(), self._full_param, self._layout, (input_,),
                             combine="cat", cat_dim=1, inplace=self.inplace, owner=self)
