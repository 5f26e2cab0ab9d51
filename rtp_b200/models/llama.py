"""Llama-shaped decoder-only LM with rotated weights: RMSNorm, rotary position embedding, SwiGLU FFN, no biases.

Rotation plan per block: packed QKV projection = column-rotated ``D -> 3D`` whose shard rows are
``[q_r; k_r; v_r]`` (heads/N heads per shard), attention over all heads locally (each rank holds the full
projection of its own batch once the N column blocks are assembled), output projection = row-rotated ``D -> D``;
SwiGLU = column-rotated packed gate/up ``D -> 2F`` (shard rows ``[gate_r; up_r]``) and row-rotated ``F -> D``.
Embedding ``[V, D/N]`` and LM head ``[V/N, D]`` rotate as well.  Activations are ``[batch, seq, dim]``."""
from dataclasses import dataclass

import torch
import torch.nn as nn

from ..module.embedding import ParallelEmbedding
from ..module.linear import ColumnParallelLinear, RowParallelLinear
from ..parallel.context import get_context
from ..ops import functional as FO


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    d_model: int = 5120
    n_layers: int = 40
    n_heads: int = 40
    d_ff: int = 13824
    max_seq_len: int = 2048
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    init_std: float = 0.02
    loss_chunk_rows: int = 0     # > 0: LM head + cross-entropy this many tokens at a time (no full logits)

    @staticmethod
    def llama_13b():
        return LlamaConfig()


class RMSNorm(nn.Module):
    def __init__(self, dim, eps=1e-5, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        if FO.use_kernels(x):
            return FO.rms_norm(x, self.weight, self.eps)
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope_tables(seq_len, head_dim, theta, device, dtype=torch.float32):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    fr = torch.outer(t, inv)
    return fr.cos().to(dtype), fr.sin().to(dtype)


def apply_rope(x, cos, sin):
    """x: [B, S, H, hd]; rotates pairs (x[2i], x[2i+1])."""
    if FO.use_kernels(x) and x.shape[-1] % 16 == 0:
        from ..ops import kernels as K
        return K.rope(x, cos, sin, inner=1)
    x1, x2 = x[..., 0::2], x[..., 1::2]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    out = torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)
    return out.flatten(-2).to(x.dtype)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None, dtype=None, group=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype, group=group, bias=False)
        ctx = get_context(group)
        self.cfg, self.N = cfg, ctx.world
        self.norm1 = RMSNorm(cfg.d_model, cfg.norm_eps, device, dtype)
        self.qkv = ColumnParallelLinear(cfg.d_model, 3 * cfg.d_model, packed_parts=3, **kw)
        self.proj = RowParallelLinear(cfg.d_model, cfg.d_model, **kw)
        self.norm2 = RMSNorm(cfg.d_model, cfg.norm_eps, device, dtype)
        self.gate_up = ColumnParallelLinear(cfg.d_model, 2 * cfg.d_ff, packed_parts=2, **kw)
        self.down = RowParallelLinear(cfg.d_ff, cfg.d_model, **kw)

    def _split_packed(self, y, parts):
        """Column blocks of a rotated packed projection are grouped per shard: [p0_j | p1_j | ...] for j = 0..N-1."""
        B, S, W = y.shape
        y = y.view(B, S, self.N, parts, W // (self.N * parts))
        return [y[:, :, :, k].reshape(B, S, -1) for k in range(parts)]

    def forward(self, x, cos, sin):
        cfg = self.cfg
        B, S, D = x.shape
        hd = D // cfg.n_heads
        q, k, v = self._split_packed(self.qkv(self.norm1(x)), 3)
        q = apply_rope(q.view(B, S, cfg.n_heads, hd), cos, sin)
        k = apply_rope(k.view(B, S, cfg.n_heads, hd), cos, sin)
        v = v.view(B, S, cfg.n_heads, hd)
        a = FO.causal_attention(q, k, v)                         # [B, S, H, hd]
        x = x + self.proj(a.reshape(B, S, D))
        g, u = self._split_packed(self.gate_up(self.norm2(x)), 2)
        x = x + self.down(FO.swiglu(g, u))
        return x


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig, device=None, dtype=None, group=None):
        super().__init__()
        self.cfg = cfg
        self.tok = ParallelEmbedding(cfg.vocab_size, cfg.d_model, device=device, dtype=dtype, group=group)
        self.blocks = nn.ModuleList([LlamaBlock(cfg, device, dtype, group) for _ in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps, device, dtype)
        self.head = ColumnParallelLinear(cfg.d_model, cfg.vocab_size, bias=False, device=device, dtype=dtype, group=group)
        with torch.no_grad():
            for p in self.parameters():
                if p.dim() > 1:
                    p.normal_(0.0, cfg.init_std)

    def forward(self, ids, targets=None):
        B, S = ids.shape
        cos, sin = rope_tables(S, self.cfg.d_model // self.cfg.n_heads, self.cfg.rope_theta, ids.device)
        x = self.tok(ids)
        for blk in self.blocks:
            x = blk(x, cos, sin)
        if targets is not None and self.cfg.loss_chunk_rows > 0:
            # head and loss chunk by chunk: the [tokens, vocab] logits never exist as a whole
            return FO.chunked_head_loss(self.norm(x), targets, self.head, self.cfg.loss_chunk_rows)
        logits = self.head(self.norm(x))
        if targets is None:
            return logits
        return FO.cross_entropy(logits, targets)
