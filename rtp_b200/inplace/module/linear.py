"""In-place rotated linear (reference: rtp/inplace/module/linear.py:147-229) and the TP linear it ships with."""
from ...module.layers import ColumnParallelLinear  # noqa: F401  (classic TP, all-gather)
from ...module.linear import ColumnParallelLinear as _Col, RowParallelLinear as _Row
from ...module.linear import ModelParallelLinear  # noqa: F401


class WeightParallelLinear(_Col):
    """Column-rotated linear whose single flat buffer travels (blocking exchange, no receive slot)."""
    inplace = True

    def __init__(self, in_features, out_features, world_size=None, rank=None, bias=True, gather_output=True,
                 init_method=None, stride=1, keep_master_weight_for_test=False, device=None, dtype=None,
                 linear_layer=None, group=None):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype, group=group,
                         linear_layer=linear_layer, world_size=world_size, rank=rank)


class WeightParallelRowLinear(_Row):
    inplace = True

    def __init__(self, in_features, out_features, world_size=None, rank=None, bias=True, device=None, dtype=None,
                 linear_layer=None, group=None, **unused):
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype, group=group,
                         linear_layer=linear_layer, world_size=world_size, rank=rank)
