"""The reference language model built from rotated layers (reference: rtp/models/transformer_lm_rtp.py:19-242).

``nn.Sequential`` of: embedding * sqrt(ninp) -> sinusoidal positional encoding + dropout -> ``ndecoder``
post-LN decoder layers with a causal mask (rotated MHA, two column-rotated FFN linears or a rotating
MoE block) -> column-rotated LM head.  Activations are ``[seq, batch, dim]``.  state_dict keys and
shapes are those of the reference (``0.embedding.embedding.weight [V, D/N]``, ``{l}.self_attn.
MultiheadAttention.in_proj_weight [3D/N, D]``, ``{l}.ff_block.linear1.linear.weight [H/N, D]`` ...).

On bf16 CUDA tensors ``forward`` runs the fused sm_100a path (``rtp_b200.models.fused_lm``).
"""
import math

import torch
import torch.nn as nn

from ..module.attention import ParallelMultiheadAttention
from ..module.embedding import ParallelEmbedding
from ..module.linear import ColumnParallelLinear
from ..module.moe import WeightMOELayer
from ..module.top2gate import WeightTop2Gate

MHA = ParallelMultiheadAttention
EMB = ParallelEmbedding
LIN = ColumnParallelLinear
GATE = WeightTop2Gate
MOE = WeightMOELayer


class EmbeddingLayer(nn.Module):
    """Rotated embedding scaled by sqrt(ninp)."""

    emb_cls = EMB

    def __init__(self, ntoken, ninp, initrange, world_size, rank, device=None, dtype=None):
        super().__init__()
        self.embedding = self.emb_cls(ntoken, ninp, world_size=world_size, rank=rank, device=device, dtype=dtype)
        self.ninp_sqrt = math.sqrt(ninp)
        with torch.no_grad():
            self.embedding.embedding.weight.uniform_(-initrange, initrange)

    def forward(self, src):
        return self.embedding(src) * self.ninp_sqrt


class PositionalEncodingLayer(nn.Module):
    """Sinusoidal positional encoding (buffer ``pe [max_len, 1, d_model]``) followed by dropout."""

    def __init__(self, d_model, dropout=0.1, max_len=5000):
        super().__init__()
        self.dropout = nn.Dropout(p=dropout)
        pe = torch.zeros(max_len, d_model)
        position = torch.arange(0, max_len, dtype=torch.float).unsqueeze(1)
        div_term = torch.exp(torch.arange(0, d_model, 2).float() * (-math.log(10000.0) / d_model))
        pe[:, 0::2] = torch.sin(position * div_term)
        pe[:, 1::2] = torch.cos(position * div_term)
        self.register_buffer("pe", pe.unsqueeze(0).transpose(0, 1))

    def forward(self, x):
        return self.dropout(x + self.pe[: x.size(0), :])


class FeedForwardLayer_expert(nn.Module):
    """One whole (unsharded) expert FFN."""

    def __init__(self, d_model, dim_feedforward, activation, dropout):
        super().__init__()
        self.linear1 = nn.Linear(d_model, dim_feedforward)
        self.activation = activation
        self.dropout1 = nn.Dropout(dropout)
        self.linear2 = nn.Linear(dim_feedforward, d_model)
        self.dropout2 = nn.Dropout(dropout)

    def forward(self, x):
        return self.dropout2(self.linear2(self.dropout1(self.activation(self.linear1(x)))))


class FeedForwardLayer(nn.Module):
    """FFN of two column-rotated linears (the reference uses no row-parallel layer here)."""

    lin_cls = LIN

    def __init__(self, d_model, dim_feedforward, activation, dropout, world_size, rank, device=None, dtype=None):
        super().__init__()
        self.linear1 = self.lin_cls(d_model, dim_feedforward, device=device, dtype=dtype, world_size=world_size, rank=rank)
        self.activation = activation
        self.dropout1 = nn.Dropout(dropout)
        self.linear2 = self.lin_cls(dim_feedforward, d_model, device=device, dtype=dtype, world_size=world_size, rank=rank)
        self.dropout2 = nn.Dropout(dropout)

    def forward(self, x):
        return self.dropout2(self.linear2(self.dropout1(self.activation(self.linear1(x)))))


class TransformerEncoderLayer(nn.Module):
    """Self-attention + FFN (or MoE) block, post-LN by default, pre-LN with ``norm_first=True``."""

    mha_cls, ff_cls, gate_cls, moe_cls = MHA, FeedForwardLayer, GATE, MOE

    def __init__(self, d_model, nhead, dim_feedforward=2048, dropout=0.1, activation=None, layer_norm_eps=1e-5,
                 norm_first=False, is_moe=False, num_local_experts=1, world_size=1, rank=0, device=None, dtype=None,
                 capacity_factor=1.0):
        super().__init__()
        activation = activation if activation is not None else nn.ReLU()
        self.self_attn = self.mha_cls(d_model, nhead, dropout=dropout, world_size=world_size, rank=rank,
                                      device=device, dtype=dtype)
        self.norm_first = norm_first
        self.norm1 = nn.LayerNorm(d_model, eps=layer_norm_eps, device=device, dtype=dtype)
        self.norm2 = nn.LayerNorm(d_model, eps=layer_norm_eps, device=device, dtype=dtype)
        self.dropout = nn.Dropout(dropout)
        self.is_moe = is_moe
        if is_moe:
            n_global = num_local_experts * world_size
            self.gate = self.gate_cls(d_model, n_global, device=device, dtype=dtype, capacity_factor=capacity_factor)
            experts = nn.ModuleList([FeedForwardLayer_expert(d_model, dim_feedforward, activation, dropout)
                                     for _ in range(num_local_experts)])
            self.moe_layer = self.moe_cls(self.gate, experts, device=device, dtype=dtype)
        else:
            self.ff_block = self.ff_cls(d_model, dim_feedforward, activation, dropout, world_size=world_size,
                                        rank=rank, device=device, dtype=dtype)

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
    """Encoder layer with a cached causal (square subsequent) float mask."""

    def __init__(self, ninp, nhead, nhid, dropout, is_moe=False, num_local_experts=1, world_size=1, rank=0,
                 device=None, dtype=None, **kw):
        super().__init__(ninp, nhead, nhid, dropout, is_moe=is_moe, num_local_experts=num_local_experts,
                         world_size=world_size, rank=rank, device=device, dtype=dtype, **kw)
        self.src_mask = None

    def _generate_square_subsequent_mask(self, sz):
        return torch.full((sz, sz), float("-inf")).triu_(1)

    def forward(self, src):
        if self.src_mask is None or self.src_mask.size(0) != len(src) or self.src_mask.device != src.device \
                or self.src_mask.dtype != src.dtype:
            self.src_mask = self._generate_square_subsequent_mask(len(src)).to(device=src.device, dtype=src.dtype)
        return super().forward(src, self.src_mask)


class LinearLayer(nn.Module):
    """LM head: column-rotated over the vocabulary, bias zero, weight U(-initrange, initrange)."""

    lin_cls = LIN

    def __init__(self, ninp, ntoken, initrange, world_size, rank, device=None, dtype=None):
        super().__init__()
        self.linear = self.lin_cls(ninp, ntoken, device=device, dtype=dtype, world_size=world_size, rank=rank)
        with torch.no_grad():
            self.linear.linear.bias.zero_()
            self.linear.linear.weight.uniform_(-initrange, initrange)

    def forward(self, src):
        return self.linear(src)


class TransformerLM(nn.Sequential):
    """A GPT-2 style ``nn.Sequential`` language model with every weight matrix rotated."""

    emb_layer_cls, dec_layer_cls, head_cls = EmbeddingLayer, TransformerDecoderLayer, LinearLayer

    def __init__(self, ntokens, ninp, nhead, nhid, dropout, initrange, ndecoder, world_size=None, rank=None,
                 is_moe=False, num_local_experts=1, device=None, dtype=None, **layer_kw):
        from ..parallel.context import get_context
        ctx = get_context()
        world_size = ctx.world if world_size is None else world_size
        rank = ctx.rank if rank is None else rank
        layers = [self.emb_layer_cls(ntokens, ninp, initrange, world_size, rank, device=device, dtype=dtype),
                  PositionalEncodingLayer(ninp, dropout)]
        for _ in range(ndecoder):
            layers.append(self.dec_layer_cls(ninp, nhead, nhid, dropout, is_moe, num_local_experts,
                                             world_size=world_size, rank=rank, device=device, dtype=dtype, **layer_kw))
        layers.append(self.head_cls(ninp, ntokens, initrange, world_size, rank, device=device, dtype=dtype))
        super().__init__(*layers)
        if device is not None:
            self.to(device)
        self.config = dict(ntokens=ntokens, ninp=ninp, nhead=nhead, nhid=nhid, dropout=dropout, ndecoder=ndecoder,
                           is_moe=is_moe, num_local_experts=num_local_experts)
