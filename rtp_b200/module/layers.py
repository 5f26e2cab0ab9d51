"""Classic (Megatron-style) tensor-parallel layers: the TP baseline of the benchmarks
(reference: rtp/module/layers.py).  Weights are sharded exactly like their rotated counterparts, but
instead of rotating weights the *activations* are all-gathered / all-reduced."""

from torch import nn

from ..parallel.context import get_context
from .attention import SubParallelMultiheadAttention
from .collectives import (copy_to_model_parallel_region, gather_from_conv_parallel_region,
                          gather_from_model_parallel_region, reduce_from_model_parallel_region)
from .conv import ModelParallelConv2d
from .embedding import ModelParallelEmbedding
from .functional import multi_head_attention_forward
from .linear import ModelParallelLinear


def _ctx(group, world_size, rank):
    ctx = get_context(group)
    if world_size is not None and world_size != ctx.world:
        raise ValueError("world_size does not match the process group")
    return ctx


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features, out_features, world_size=None, rank=None, bias=True, gather_output=True,
                 device=None, dtype=None, linear_layer=None, group=None, **unused):
        super().__init__()
        ctx = _ctx(group, world_size, rank)
        self.world_size, self.rank, self.ring = ctx.world, ctx.rank, ctx
        self.in_features, self.out_features, self.gather_output = in_features, out_features, gather_output
        self.linear = ModelParallelLinear(in_features, out_features, bias=bias, device=device, dtype=dtype,
                                          world_size=ctx.world, rank=ctx.rank)
        self.linear.affine_weight(linear_layer)

    def forward(self, input_):
        x = copy_to_model_parallel_region(input_, self.ring.group)
        out = self.linear(x)
        return gather_from_model_parallel_region(out, self.ring.group) if self.gather_output else out


class ParallelEmbedding(nn.Module):
    def __init__(self, num_embeddings, embedding_dim, world_size=None, rank=None, padding_idx=None, max_norm=None,
                 norm_type=2.0, scale_grad_by_freq=False, sparse=False, Embedding_layer=None, device=None, dtype=None,
                 group=None, gather_output=True, **unused):
        super().__init__()
        ctx = _ctx(group, world_size, rank)
        self.world_size, self.rank, self.ring, self.gather_output = ctx.world, ctx.rank, ctx, gather_output
        self.embedding = ModelParallelEmbedding(num_embeddings, embedding_dim, ctx.world, ctx.rank,
                                                padding_idx=padding_idx, max_norm=max_norm, norm_type=norm_type,
                                                scale_grad_by_freq=scale_grad_by_freq, sparse=sparse, device=device,
                                                dtype=dtype)
        self.embedding.affine_weight(Embedding_layer)

    def forward(self, input_):
        out = self.embedding(input_)
        return gather_from_model_parallel_region(out, self.ring.group) if self.gather_output else out


class ParallelMultiheadAttention(nn.Module):
    """Each rank computes its heads' partial output; partials are all-reduced."""

    def __init__(self, embed_dim, num_heads, world_size=None, rank=None, dropout=0., bias=True, add_bias_kv=False,
                 add_zero_attn=False, kdim=None, vdim=None, batch_first=False, device=None, dtype=None,
                 MultiheadAttention_layer=None, group=None):
        super().__init__()
        ctx = _ctx(group, world_size, rank)
        self.world_size, self.rank, self.ring, self.batch_first = ctx.world, ctx.rank, ctx, batch_first
        self.MultiheadAttention = SubParallelMultiheadAttention(embed_dim, num_heads, ctx.world, ctx.rank, dropout,
                                                                bias, add_bias_kv, add_zero_attn, kdim, vdim,
                                                                batch_first, device, dtype)
        self.MultiheadAttention.affine_weight(MultiheadAttention_layer)

    def forward(self, query, key, value, key_padding_mask=None, need_weights=True, attn_mask=None,
                average_attn_weights=True, is_causal=False):
        sub = self.MultiheadAttention
        batched = query.dim() == 3
        same = (key is value) and (query is key)
        if self.batch_first and batched:
            query, key, value = [t.transpose(1, 0) for t in (query, key, value)]
        q = copy_to_model_parallel_region(query, self.ring.group)
        k, v = (q, q) if same else (copy_to_model_parallel_region(key, self.ring.group),
                                    copy_to_model_parallel_region(value, self.ring.group))
        out, w = multi_head_attention_forward(
            q, k, v, sub.embed_dim_per_partition, sub.num_heads_per_partition, sub.in_proj_weight, sub.in_proj_bias,
            sub.bias_k, sub.bias_v, sub.add_zero_attn, sub.dropout, sub.out_proj.weight, sub.out_proj.bias,
            training=self.training, key_padding_mask=key_padding_mask, need_weights=need_weights, attn_mask=attn_mask,
            use_separate_proj_weight=not sub._qkv_same_embed_dim, q_proj_weight=sub.q_proj_weight,
            k_proj_weight=sub.k_proj_weight, v_proj_weight=sub.v_proj_weight,
            average_attn_weights=average_attn_weights, is_causal=is_causal, E_div=self.world_size)
        out = reduce_from_model_parallel_region(out, self.ring.group)
        if self.batch_first and batched:
            out = out.transpose(1, 0)
        return out, w


class ColumnParallelConv2d(nn.Module):
    def __init__(self, in_channels, out_channels, kernel_size, world_size=None, rank=None, stride=1, padding=0,
                 dilation=1, groups=1, bias=True, padding_mode="zeros", device=None, dtype=None, gather_output=True,
                 Conv2d_layer=None, group=None):
        super().__init__()
        ctx = _ctx(group, world_size, rank)
        self.world_size, self.rank, self.ring, self.gather_output = ctx.world, ctx.rank, ctx, gather_output
        self.conv = ModelParallelConv2d(in_channels, out_channels, kernel_size, stride, padding, dilation, groups,
                                        bias, padding_mode, device, dtype, world_size=ctx.world, rank=ctx.rank)
        self.conv.affine_weight(Conv2d_layer)

    def forward(self, input_):
        out = self.conv(copy_to_model_parallel_region(input_, self.ring.group))
        return gather_from_conv_parallel_region(out, self.ring.group) if self.gather_output else out
