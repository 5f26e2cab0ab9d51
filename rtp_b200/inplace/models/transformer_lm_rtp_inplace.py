"""The reference LM built from in-place rotated layers (reference:
rtp/inplace/models/transformer_lm_rtp_inplace.py); identical state_dict keys and shapes."""
from ...models import transformer_lm_rtp as _m
from ..module.attention import WeightParallelMultiheadAttention
from ..module.embedding import WeightParallelEmbedding
from ..module.linear import WeightParallelLinear
from ..module.moe import WeightMOELayer
from ..module.top2gate import WeightTop2Gate

PositionalEncodingLayer = _m.PositionalEncodingLayer
FeedForwardLayer_expert = _m.FeedForwardLayer_expert


class EmbeddingLayer(_m.EmbeddingLayer):
    emb_cls = WeightParallelEmbedding


class FeedForwardLayer(_m.FeedForwardLayer):
    lin_cls = WeightParallelLinear


class TransformerEncoderLayer(_m.TransformerEncoderLayer):
    mha_cls, ff_cls, gate_cls, moe_cls = (WeightParallelMultiheadAttention, FeedForwardLayer, WeightTop2Gate,
                                          WeightMOELayer)


class TransformerDecoderLayer(_m.TransformerDecoderLayer):
    mha_cls, ff_cls, gate_cls, moe_cls = (WeightParallelMultiheadAttention, FeedForwardLayer, WeightTop2Gate,
                                          WeightMOELayer)


class LinearLayer(_m.LinearLayer):
    lin_cls = WeightParallelLinear


class TransformerLM(_m.TransformerLM):
    emb_layer_cls, dec_layer_cls, head_cls = EmbeddingLayer, TransformerDecoderLayer, LinearLayer
