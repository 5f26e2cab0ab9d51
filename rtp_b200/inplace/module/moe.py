"""In-place rotating experts (reference: rtp/inplace/module/moe.py)."""
from ...module.moe import MOELayer, _AllToAll, WeightMOELayer as _MOE  # noqa: F401


class WeightMOELayer(_MOE):
    inplace = True
