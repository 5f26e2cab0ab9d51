"""Single head-shard multi-head attention used by the ``RotatedTensorParallel`` wrapper
(reference: rtp/attention.py:12-147): holds ``heads / N`` heads (``in_proj_weight [3E/N, E]``,
``out_proj [E, E/N]``) and returns this shard's partial output; the wrapper rotates the shard and sums
the partials."""
from typing import Optional, Tuple

from torch import Tensor

from .module.attention import SubParallelMultiheadAttention
from .module.functional import multi_head_attention_forward
from .parallel.context import get_context


class ParallelMultiheadAttention(SubParallelMultiheadAttention):
    def __init__(self, embed_dim, num_heads, dropout=0., bias=True, add_bias_kv=False, add_zero_attn=False,
                 kdim=None, vdim=None, batch_first=False, device=None, dtype=None, group=None):
        ctx = get_context(group)
        super().__init__(embed_dim, num_heads, ctx.world, ctx.rank, dropout, bias, add_bias_kv, add_zero_attn, kdim,
                         vdim, batch_first, device, dtype)
        self.ring = ctx

    def forward(self, query: Tensor, key: Tensor, value: Tensor, key_padding_mask: Optional[Tensor] = None,
                need_weights: bool = True, attn_mask: Optional[Tensor] = None, average_attn_weights: bool = True,
                is_causal: bool = False) -> Tuple[Tensor, Optional[Tensor]]:
        batched = query.dim() == 3
        if self.batch_first and batched:
            if key is value and query is key:
                query = key = value = query.transpose(1, 0)
            else:
                query, key, value = [t.transpose(1, 0) for t in (query, key, value)]
        out, w = multi_head_attention_forward(
            query, key, value, self.embed_dim_per_partition, self.num_heads_per_partition, self.in_proj_weight,
            self.in_proj_bias, self.bias_k, self.bias_v, self.add_zero_attn, self.dropout, self.out_proj.weight,
            self.out_proj.bias, training=self.training, key_padding_mask=key_padding_mask, need_weights=need_weights,
            attn_mask=attn_mask, use_separate_proj_weight=not self._qkv_same_embed_dim,
            q_proj_weight=self.q_proj_weight, k_proj_weight=self.k_proj_weight, v_proj_weight=self.v_proj_weight,
            average_attn_weights=average_attn_weights, is_causal=is_causal, E_div=self.world_size)
        if self.batch_first and batched:
            out = out.transpose(1, 0)
        return out, w
