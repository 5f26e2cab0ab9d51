"""MoE transformer LM: every FFN is replaced by ``E`` experts with top-2 softmax gating; the experts rotate around
the ring (``WeightMOELayer``) instead of exchanging tokens with all-to-alls.  Built on the GPT block layout
(pre-LN, GELU experts); ``capacity_factor`` scales the reference's capacity ``2S/E``."""
from dataclasses import dataclass

import torch
import torch.nn as nn

from ..module.attention import ParallelMultiheadAttention
from ..module.embedding import ParallelEmbedding
from ..module.linear import ColumnParallelLinear
from ..module.norm import LayerNorm
from ..ops import functional as FO
from ..module.moe import WeightMOELayer
from ..module.top2gate import WeightTop2Gate
from ..parallel.context import get_context


@dataclass
class MoEConfig:
    vocab_size: int = 32000
    d_model: int = 2048
    n_layers: int = 12
    n_heads: int = 16
    d_ff: int = 8192
    n_experts: int = 8
    capacity_factor: float = 1.25
    max_seq_len: int = 1024
    dropout: float = 0.0
    aux_loss_weight: float = 0.01
    init_std: float = 0.02


class Expert(nn.Module):
    def __init__(self, d_model, d_ff):
        super().__init__()
        self.linear1 = nn.Linear(d_model, d_ff)
        self.activation = nn.GELU()
        self.linear2 = nn.Linear(d_ff, d_model)

    def forward(self, x):
        return self.linear2(self.activation(self.linear1(x)))


class MoEBlock(nn.Module):
    def __init__(self, cfg: MoEConfig, device=None, dtype=None, group=None):
        super().__init__()
        ctx = get_context(group)
        if cfg.n_experts % ctx.world:
            raise ValueError("number of experts must be divisible by the ring size")
        self.ln1 = LayerNorm(cfg.d_model, device=device, dtype=dtype)
        self.attn = ParallelMultiheadAttention(cfg.d_model, cfg.n_heads, dropout=cfg.dropout, batch_first=True,
                                               device=device, dtype=dtype, group=group)
        self.ln2 = LayerNorm(cfg.d_model, device=device, dtype=dtype)
        self.gate = WeightTop2Gate(cfg.d_model, cfg.n_experts, device=device, dtype=dtype, group=group,
                                   capacity_factor=cfg.capacity_factor)
        experts = nn.ModuleList([Expert(cfg.d_model, cfg.d_ff) for _ in range(cfg.n_experts // ctx.world)])
        self.moe_layer = WeightMOELayer(self.gate, experts, group=group, device=device, dtype=dtype)

    def forward(self, x):
        h = self.ln1(x)
        x = x + self.attn(h, h, h, need_weights=False, is_causal=True)[0]
        x = x + self.moe_layer(self.ln2(x))
        return x


class MoELM(nn.Module):
    def __init__(self, cfg: MoEConfig, device=None, dtype=None, group=None):
        super().__init__()
        self.cfg = cfg
        self.tok = ParallelEmbedding(cfg.vocab_size, cfg.d_model, device=device, dtype=dtype, group=group)
        self.pos = nn.Parameter(torch.zeros(cfg.max_seq_len, cfg.d_model, device=device, dtype=dtype))
        self.blocks = nn.ModuleList([MoEBlock(cfg, device, dtype, group) for _ in range(cfg.n_layers)])
        self.ln_f = LayerNorm(cfg.d_model, device=device, dtype=dtype)
        self.head = ColumnParallelLinear(cfg.d_model, cfg.vocab_size, bias=False, device=device, dtype=dtype, group=group)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() > 1:
                    p.normal_(0.0, cfg.init_std)
            self.pos.normal_(0.0, cfg.init_std)

    def forward(self, ids, targets=None):
        B, S = ids.shape
        x = self.tok(ids) + self.pos[:S]
        for blk in self.blocks:
            x = blk(x)
        logits = self.head(self.ln_f(x))
        if targets is None:
            return logits
        ce = FO.cross_entropy(logits, targets)
        aux = sum(blk.moe_layer.l_aux for blk in self.blocks) / len(self.blocks)
        return ce + self.cfg.aux_loss_weight * aux.float()
