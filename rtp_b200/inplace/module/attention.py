"""In-place rotated attention (reference: rtp/inplace/module/attention.py:258-325) and the TP attention."""
from ...module.layers import ParallelMultiheadAttention  # noqa: F401  (classic TP, all-reduce)
from ...module.attention import ParallelMultiheadAttention as _MHA, SubParallelMultiheadAttention  # noqa: F401


class WeightParallelMultiheadAttention(_MHA):
    inplace = True
