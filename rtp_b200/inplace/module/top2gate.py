"""In-place rotated top-2 gate (reference: rtp/inplace/module/top2gate.py)."""
from ...module.top2gate import (Top2Gate, gumbel_rsample, one_hot, top2gating, top2_routing,  # noqa: F401
                                WeightTop2Gate as _Gate)


class WeightTop2Gate(_Gate):
    inplace = True
