"""GPT-style decoder-only LM with rotated weights: pre-LN blocks, GELU FFN, learned positional embedding,
causal attention, LM head rotated over the vocabulary.

Every weight matrix is sharded 1/N and rotated: token embedding ``[V, D/N]`` (embedding-dim shards, as the
reference's ParallelEmbedding), attention = ``ParallelMultiheadAttention`` (head shards), FFN =
column-rotated ``D -> F`` followed by row-rotated ``F -> D``, head = column-rotated ``D -> V``.
Activations are ``[batch, seq, dim]``."""
from dataclasses import dataclass

import torch
import torch.nn as nn

from ..module.attention import ParallelMultiheadAttention
from ..module.embedding import ParallelEmbedding
from ..module.linear import ColumnParallelLinear, RowParallelLinear
from ..module.norm import LayerNorm
from ..ops import functional as FO


@dataclass
class GPTConfig:
    vocab_size: int = 50304
    d_model: int = 2048
    n_layers: int = 24
    n_heads: int = 16
    d_ff: int = 8192
    max_seq_len: int = 2048
    dropout: float = 0.0
    init_std: float = 0.02
    loss_chunk_rows: int = 0     # > 0: LM head + cross-entropy this many tokens at a time (no full logits)

    @staticmethod
    def gpt_1p3b():
        return GPTConfig()


class GPTBlock(nn.Module):
    def __init__(self, cfg: GPTConfig, device=None, dtype=None, group=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype, group=group)
        self.ln1 = LayerNorm(cfg.d_model, device=device, dtype=dtype)
        self.attn = ParallelMultiheadAttention(cfg.d_model, cfg.n_heads, dropout=cfg.dropout, batch_first=True, **kw)
        self.ln2 = LayerNorm(cfg.d_model, device=device, dtype=dtype)
        self.fc1 = ColumnParallelLinear(cfg.d_model, cfg.d_ff, **kw)
        self.fc2 = RowParallelLinear(cfg.d_ff, cfg.d_model, **kw)
        self.drop = nn.Dropout(cfg.dropout)

    def forward(self, x):
        h = self.ln1(x)
        x = x + self.drop(self.attn(h, h, h, need_weights=False, is_causal=True)[0])
        x = x + self.drop(self.fc2(FO.gelu(self.fc1(self.ln2(x)))))
        return x


class GPT(nn.Module):
    def __init__(self, cfg: GPTConfig, device=None, dtype=None, group=None):
        super().__init__()
        self.cfg = cfg
        self.tok = ParallelEmbedding(cfg.vocab_size, cfg.d_model, device=device, dtype=dtype, group=group)
        self.pos = nn.Parameter(torch.zeros(cfg.max_seq_len, cfg.d_model, device=device, dtype=dtype))
        self.drop = nn.Dropout(cfg.dropout)
        self.blocks = nn.ModuleList([GPTBlock(cfg, device, dtype, group) for _ in range(cfg.n_layers)])
        self.ln_f = LayerNorm(cfg.d_model, device=device, dtype=dtype)
        self.head = ColumnParallelLinear(cfg.d_model, cfg.vocab_size, bias=False, device=device, dtype=dtype, group=group)
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self):
        std = self.cfg.init_std
        for name, p in self.named_parameters():
            if p.dim() > 1:
                p.normal_(0.0, std)
            elif name.endswith("bias"):
                p.zero_()
        self.pos.normal_(0.0, std)

    def forward(self, ids, targets=None):
        B, S = ids.shape
        x = self.drop(self.tok(ids) + self.pos[:S])
        for blk in self.blocks:
            x = blk(x)
        if targets is not None and self.cfg.loss_chunk_rows > 0:
            # head and loss chunk by chunk: the [tokens, vocab] logits never exist as a whole
            return FO.chunked_head_loss(self.ln_f(x), targets, self.head, self.cfg.loss_chunk_rows)
        logits = self.head(self.ln_f(x))
        if targets is None:
            return logits
        return FO.cross_entropy(logits, targets)

    def num_parameters_global(self, world: int) -> int:
        n = 0
        for p in self.parameters():
            n += p.numel() * (world if getattr(p, "rtp_sharded", False) and not getattr(p, "rtp_sum_replicated", None) else 1)
        return n
