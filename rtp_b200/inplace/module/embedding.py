"""In-place rotated embedding (reference: rtp/inplace/module/embedding.py:129-206) and the TP embedding."""
from ...module.layers import ParallelEmbedding  # noqa: F401  (classic TP, all-gather)
from ...module.embedding import ParallelEmbedding as _Emb, ModelParallelEmbedding  # noqa: F401


class WeightParallelEmbedding(_Emb):
    inplace = True
