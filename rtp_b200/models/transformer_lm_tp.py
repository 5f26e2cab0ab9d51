"""The language model with classic tensor parallelism (all-gather / all-reduce of activations instead of rotating
weights): the TP baseline of the benchmarks (reference: rtp/models/transformer_lm_tp.py)."""
from . import transformer_lm_rtp as _m
from ..module import layers as TP

PositionalEncodingLayer = _m.PositionalEncodingLayer


class EmbeddingLayer(_m.EmbeddingLayer):
    emb_cls = TP.ParallelEmbedding


class FeedForwardLayer(_m.FeedForwardLayer):
    lin_cls = TP.ColumnParallelLinear


class TransformerDecoderLayer(_m.TransformerDecoderLayer):
    mha_cls, ff_cls = TP.ParallelMultiheadAttention, FeedForwardLayer


class LinearLayer(_m.LinearLayer):
    lin_cls = TP.ColumnParallelLinear


class TransformerLM(_m.TransformerLM):
    """Every rank must see the SAME batch (the activations are what is exchanged)."""
    emb_layer_cls, dec_layer_cls, head_cls = EmbeddingLayer, TransformerDecoderLayer, LinearLayer
