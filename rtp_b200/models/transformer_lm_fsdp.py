"""The same language model without any weight sharding (plain torch layers): the single-process oracle
and the model that the DP / FSDP baselines wrap (reference: rtp/models/transformer_lm_fsdp.py,
benchmarks/transformer_lm_dp.py)."""
import math

import torch
import torch.nn as nn

from .transformer_lm_rtp import FeedForwardLayer_expert, PositionalEncodingLayer
from ..module.moe import MOELayer
from ..module.top2gate import Top2Gate


class EmbeddingLayer(nn.Embedding):
    def __init__(self, ntoken, ninp, initrange):
        super().__init__(ntoken, ninp)
        self.ninp_sqrt = math.sqrt(ninp)
        with torch.no_grad():
            self.weight.uniform_(-initrange, initrange)

    def forward(self, src):
        return super().forward(src) * self.ninp_sqrt


class FeedForwardLayer(FeedForwardLayer_expert):
    pass


class TransformerEncoderLayer(nn.Module):
    def __init__(self, d_model, nhead, dim_feedforward=2048, dropout=0.1, activation=None, layer_norm_eps=1e-5,
                 norm_first=False, is_moe=False, num_local_experts=1, capacity_factor=1.0):
        super().__init__()
        activation = activation if activation is not None else nn.ReLU()
        self.self_attn = nn.MultiheadAttention(d_model, nhead, dropout=dropout)
        self.norm_first = norm_first
        self.norm1 = nn.LayerNorm(d_model, eps=layer_norm_eps)
        self.norm2 = nn.LayerNorm(d_model, eps=layer_norm_eps)
        self.dropout = nn.Dropout(dropout)
        self.is_moe = is_moe
        if is_moe:
            world = torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1
            self.gate = Top2Gate(d_model, num_local_experts * world, capacity_factor)
            experts = nn.ModuleList([FeedForwardLayer_expert(d_model, dim_feedforward, activation, dropout)
                                     for _ in range(num_local_experts)])
            self.moe_layer = MOELayer(self.gate, experts)
        else:
            self.ff_block = FeedForwardLayer(d_model, dim_feedforward, activation, dropout)

    def forward(self, src, src_mask=None, src_key_padding_mask=None):
        x = src
        if self.norm_first:
            x = x + self._sa_block(self.norm1(x), src_mask, src_key_padding_mask)
            x = x + self._ff_block(self.norm2(x))
        else:
            x = self.norm1(x + self._sa_block(x, src_mask, src_key_padding_mask))
            x = self.norm2(x + self._ff_block(x))
        return x

    def _sa_block(self, x, attn_mask, key_padding_mask):
        x = self.self_attn(x, x, x, attn_mask=attn_mask, key_padding_mask=key_padding_mask, need_weights=False)[0]
        return self.dropout(x)

    def _ff_block(self, x):
        return self.moe_layer(x) if self.is_moe else self.ff_block(x)


class TransformerDecoderLayer(TransformerEncoderLayer):
    def __init__(self, ninp, nhead, nhid, dropout, is_moe=False, num_local_experts=1, **kw):
        super().__init__(ninp, nhead, nhid, dropout, is_moe=is_moe, num_local_experts=num_local_experts, **kw)
        self.src_mask = None

    def forward(self, src):
        if self.src_mask is None or self.src_mask.size(0) != len(src) or self.src_mask.device != src.device \
                or self.src_mask.dtype != src.dtype:
            self.src_mask = torch.full((len(src), len(src)), float("-inf")).triu_(1).to(device=src.device,
                                                                                        dtype=src.dtype)
        return super().forward(src, self.src_mask)


class LinearLayer(nn.Linear):
    def __init__(self, ninp, ntoken, initrange):
        super().__init__(ninp, ntoken)
        with torch.no_grad():
            self.bias.zero_()
            self.weight.uniform_(-initrange, initrange)


class TransformerLM(nn.Sequential):
    def __init__(self, ntokens, ninp, nhead, nhid, dropout, initrange, ndecoder, is_moe=False, num_local_experts=1,
                 **layer_kw):
        layers = [EmbeddingLayer(ntokens, ninp, initrange), PositionalEncodingLayer(ninp, dropout)]
        for _ in range(ndecoder):
            layers.append(TransformerDecoderLayer(ninp, nhead, nhid, dropout, is_moe, num_local_experts, **layer_kw))
        layers.append(LinearLayer(ninp, ntokens, initrange))
        super().__init__(*layers)
