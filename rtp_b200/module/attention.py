"""Rotated multi-head attention: each shard holds ``heads/N`` heads — rows ``[q_r; k_r; v_r]`` of the packed
in-projection, the matching column block of the out-projection and ``out_proj.bias / N`` — and the N
partial outputs are summed (reference: rtp/module/attention.py:17-267)."""
from typing import Optional, Tuple

import torch
from torch import Tensor, nn
from torch.nn import Parameter

from ..parallel.flat import RotatedModule
from ..parallel.rotated import rotated_apply
from .functional import multi_head_attention_forward
from .utils import affine_weight, affine_weight_attention, divide_and_check_no_remainder, qkv_block_index


class SubParallelMultiheadAttention(nn.Module):
    """Parameters of one head-shard, named like ``nn.MultiheadAttention`` (in_proj_weight, in_proj_bias,
    out_proj.weight, out_proj.bias) so that state_dict keys match the reference."""

    def __init__(self, embed_dim, num_heads, world_size, rank, dropout=0., bias=True, add_bias_kv=False,
                 add_zero_attn=False, kdim=None, vdim=None, batch_first=False, device=None, dtype=None,
                 MultiheadAttention=None, empty_init=False):
        super().__init__()
        if embed_dim <= 0 or num_heads <= 0:
            raise ValueError(f"embed_dim and num_heads must be greater than 0, got {embed_dim} and {num_heads}")
        fk = {"device": device, "dtype": dtype}
        self.embed_dim = embed_dim
        self.kdim = kdim if kdim is not None else embed_dim
        self.vdim = vdim if vdim is not None else embed_dim
        self._qkv_same_embed_dim = self.kdim == embed_dim and self.vdim == embed_dim
        self.num_heads, self.dropout, self.batch_first = num_heads, dropout, batch_first
        self.head_dim = embed_dim // num_heads
        assert self.head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"
        self.world_size, self.rank = world_size, rank
        self.num_heads_per_partition = divide_and_check_no_remainder(num_heads, world_size)
        self.embed_dim_per_partition = divide_and_check_no_remainder(embed_dim, world_size)
        ep = self.embed_dim_per_partition
        if not self._qkv_same_embed_dim:
            self.q_proj_weight = Parameter(torch.empty((ep, embed_dim), **fk))
            self.k_proj_weight = Parameter(torch.empty((ep, self.kdim), **fk))
            self.v_proj_weight = Parameter(torch.empty((ep, self.vdim), **fk))
            self.register_parameter("in_proj_weight", None)
        else:
            self.in_proj_weight = Parameter(torch.empty((3 * ep, embed_dim), **fk))
            self.register_parameter("q_proj_weight", None)
            self.register_parameter("k_proj_weight", None)
            self.register_parameter("v_proj_weight", None)
        if bias:
            self.in_proj_bias = Parameter(torch.empty(3 * ep, **fk))
        else:
            self.register_parameter("in_proj_bias", None)
        self.out_proj = nn.Linear(ep, embed_dim, bias=bias, **fk)
        if add_bias_kv:
            self.bias_k = Parameter(torch.empty((1, 1, ep), **fk))
            self.bias_v = Parameter(torch.empty((1, 1, ep), **fk))
        else:
            self.bias_k = self.bias_v = None
        self.add_zero_attn = add_zero_attn
        self._reset_parameters()
        if bias:
            with torch.no_grad():
                self.out_proj.bias.div_(world_size)
            self.out_proj.bias.rtp_sum_replicated = world_size

    def _reset_parameters(self):
        # the reference leaves in_proj uninitialised (torch.empty); initialise like nn.MultiheadAttention
        for w in (self.in_proj_weight, self.q_proj_weight, self.k_proj_weight, self.v_proj_weight):
            if w is not None:
                nn.init.xavier_uniform_(w)
        if self.in_proj_bias is not None:
            nn.init.constant_(self.in_proj_bias, 0.)
            nn.init.constant_(self.out_proj.bias, 0.)
        if self.bias_k is not None:
            nn.init.xavier_normal_(self.bias_k)
            nn.init.xavier_normal_(self.bias_v)

    def affine_weight(self, mha: Optional[nn.MultiheadAttention]):
        if mha is None:
            return
        N, r, ep = self.world_size, self.rank, self.embed_dim_per_partition
        idx = qkv_block_index(r, N)
        if self._qkv_same_embed_dim:
            affine_weight_attention(self.in_proj_weight, mha.in_proj_weight, idx, ep, 0, N, r)
        else:
            affine_weight(self.q_proj_weight, mha.q_proj_weight, ep, 0, N, r)
            affine_weight(self.k_proj_weight, mha.k_proj_weight, ep, 0, N, r)
            affine_weight(self.v_proj_weight, mha.v_proj_weight, ep, 0, N, r)
        if self.in_proj_bias is not None and mha.in_proj_bias is not None:
            affine_weight_attention(self.in_proj_bias, mha.in_proj_bias, idx, ep, 0, N, r)
        affine_weight(self.out_proj.weight, mha.out_proj.weight, ep, 1, N, r)
        if self.out_proj.bias is not None and mha.out_proj.bias is not None:
            with torch.no_grad():
                self.out_proj.bias.copy_(mha.out_proj.bias / N)
        if self.bias_k is not None and mha.bias_k is not None:
            affine_weight(self.bias_k, mha.bias_k, ep, 2, N, r)
            affine_weight(self.bias_v, mha.bias_v, ep, 2, N, r)

    def param_list(self):
        names = ["in_proj_weight", "q_proj_weight", "k_proj_weight", "v_proj_weight", "in_proj_bias"]
        out = [(n, getattr(self, n)) for n in names if getattr(self, n) is not None]
        out.append(("out_proj.weight", self.out_proj.weight))
        if self.out_proj.bias is not None:
            out.append(("out_proj.bias", self.out_proj.bias))
        if self.bias_k is not None:
            out += [("bias_k", self.bias_k), ("bias_v", self.bias_v)]
        return out


class ParallelMultiheadAttention(RotatedModule):
    __constants__ = ["batch_first"]

    def __init__(self, embed_dim, num_heads, world_size=None, rank=None, dropout=0., bias=True, add_bias_kv=False,
                 add_zero_attn=False, kdim=None, vdim=None, batch_first=False, device=None, dtype=None,
                 MultiheadAttention_layer=None, group=None):
        super().__init__()
        self._setup_ring(group, world_size, rank)
        self.embed_dim, self.num_heads, self.dropout, self.batch_first = embed_dim, num_heads, dropout, batch_first
        self.MultiheadAttention = SubParallelMultiheadAttention(
            embed_dim, num_heads, self.world_size, self.rank, dropout, bias, add_bias_kv, add_zero_attn, kdim, vdim,
            batch_first, device, dtype)
        self.MultiheadAttention.affine_weight(MultiheadAttention_layer)
        self._names = [n for n, _ in self.MultiheadAttention.param_list()]
        self._flatten()

    def shard_parameters(self):
        return [p for _, p in self.MultiheadAttention.param_list()]

    def shard_names(self):
        return list(self._names)

    def shard_spec(self):
        kinds = {"in_proj_weight": ("qkv", 0), "in_proj_bias": ("qkv", 0), "q_proj_weight": ("split", 0),
                 "k_proj_weight": ("split", 0), "v_proj_weight": ("split", 0), "out_proj.weight": ("split", 1),
                 "out_proj.bias": ("sum",), "bias_k": ("split", 2), "bias_v": ("split", 2)}
        return {f"MultiheadAttention.{n}": kinds[n] for n in self._names}

    @property
    def layers(self):
        return [self.MultiheadAttention] * self.world_size

    def forward(self, query: Tensor, key: Tensor, value: Tensor, key_padding_mask: Optional[Tensor] = None,
                need_weights: bool = True, attn_mask: Optional[Tensor] = None, average_attn_weights: bool = True,
                is_causal: bool = False, test_tensor=None) -> Tuple[Tensor, Optional[Tensor]]:
        sub = self.MultiheadAttention
        batched = query.dim() == 3
        same_qkv = (key is value) and (query is key)
        if self._full_param.is_cuda:
            from ..parallel import engine
            if engine.mha_fused_ok(self, sub, query, key, value, key_padding_mask, need_weights, attn_mask, self.training):
                return engine.fused_mha(self, sub, query, is_causal=is_causal, attn_mask=attn_mask,
                                        key_padding_mask=key_padding_mask, need_weights=need_weights,
                                        average_attn_weights=average_attn_weights, training=self.training)
        if self.batch_first and batched:
            query, key, value = [t.transpose(1, 0) for t in (query, key, value)]
        names = self._names
        training = self.training
        N = self.world_size
        tensors = [query] if same_qkv else [query, key, value]
        n_in = len(tensors)
        masks = [key_padding_mask, attn_mask]

        def fn(j, views, *ins):
            p = dict(zip(names, views))
            if n_in == 1:
                q = k = v = ins[0]
            else:
                q, k, v = ins[:3]
            kpm, am = ins[n_in], ins[n_in + 1]
            out, w = multi_head_attention_forward(
                q, k, v, sub.embed_dim_per_partition, sub.num_heads_per_partition,
                p.get("in_proj_weight"), p.get("in_proj_bias"), p.get("bias_k"), p.get("bias_v"), sub.add_zero_attn,
                sub.dropout, p["out_proj.weight"], p.get("out_proj.bias"), training=training,
                key_padding_mask=kpm, need_weights=need_weights, attn_mask=am,
                use_separate_proj_weight=not sub._qkv_same_embed_dim, q_proj_weight=p.get("q_proj_weight"),
                k_proj_weight=p.get("k_proj_weight"), v_proj_weight=p.get("v_proj_weight"),
                average_attn_weights=average_attn_weights, is_causal=is_causal, E_div=N)
            return (out, w) if w is not None else out

        res = rotated_apply(self.ring, fn, self.shard_parameters(), self._full_param, self._layout,
                            (*tensors, *masks), combine="sum", inplace=self.inplace,
                            stochastic=training and sub.dropout > 0, owner=self)
        if isinstance(res, tuple):
            out, weights = res[0], res[1]
        else:
            out, weights = res, None
        if self.batch_first and batched:
            out = out.transpose(1, 0)
        return out, weights
