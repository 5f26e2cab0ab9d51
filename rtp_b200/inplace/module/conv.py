"""In-place rotated Conv2d (the reference has no in-place conv; provided for symmetry)."""
from ...module.conv import ColumnParallelConv2d as _Conv


class WeightParallelConv2d(_Conv):
    inplace = True
