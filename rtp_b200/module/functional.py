"""Multi-head attention forward for one head-shard.

Same role and argument list as the reference's vendored ``multi_head_attention_forward``
(rtp/module/functional.py:464-833): the projection weights passed in hold only ``E / E_div`` of the
embedding (``num_heads`` is the number of heads of this shard), the input still has the full embedding
width, and the result is this shard's *partial* output ``[L, B, E]`` — the N partials sum to the full
attention output.  Written from the math, not from torch's source; supports packed or separate
projections, bias_k/bias_v, add_zero_attn, key padding and additive/boolean masks, causal masking,
dropout on the attention probabilities and averaged/per-head attention weights.
"""
import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor


def _additive_mask(mask: Optional[Tensor], dtype) -> Optional[Tensor]:
    if mask is None:
        return None
    if mask.dtype == torch.bool:
        return torch.zeros(mask.shape, dtype=dtype, device=mask.device).masked_fill_(mask, float("-inf"))
    return mask.to(dtype)


def multi_head_attention_forward(
    query: Tensor, key: Tensor, value: Tensor, embed_dim_to_check: int, num_heads: int,
    in_proj_weight: Optional[Tensor], in_proj_bias: Optional[Tensor],
    bias_k: Optional[Tensor], bias_v: Optional[Tensor], add_zero_attn: bool, dropout_p: float,
    out_proj_weight: Tensor, out_proj_bias: Optional[Tensor], training: bool = True,
    key_padding_mask: Optional[Tensor] = None, need_weights: bool = True, attn_mask: Optional[Tensor] = None,
    use_separate_proj_weight: bool = False, q_proj_weight: Optional[Tensor] = None,
    k_proj_weight: Optional[Tensor] = None, v_proj_weight: Optional[Tensor] = None,
    static_k: Optional[Tensor] = None, static_v: Optional[Tensor] = None,
    average_attn_weights: bool = True, is_causal: bool = False, E_div: int = 1,
) -> Tuple[Tensor, Optional[Tensor]]:
    batched = query.dim() == 3
    if not batched:
        query, key, value = query.unsqueeze(1), key.unsqueeze(1), value.unsqueeze(1)
        if key_padding_mask is not None:
            key_padding_mask = key_padding_mask.unsqueeze(0)
    L, B, _ = query.shape
    S = key.shape[0]
    Es = embed_dim_to_check          # embedding width of this shard
    hd = Es // num_heads
    if hd * num_heads != Es:
        raise AssertionError("shard embedding width must be divisible by its number of heads")

    # ---- input projections with this shard's rows
    if use_separate_proj_weight:
        bq = bk = bv = None
        if in_proj_bias is not None:
            bq, bk, bv = in_proj_bias.chunk(3)
        q = F.linear(query, q_proj_weight, bq)
        k = F.linear(key, k_proj_weight, bk)
        v = F.linear(value, v_proj_weight, bv)
    else:
        wq, wk, wv = in_proj_weight.chunk(3)
        bq = bk = bv = None
        if in_proj_bias is not None:
            bq, bk, bv = in_proj_bias.chunk(3)
        if key is value and query is key:
            q, k, v = F.linear(query, in_proj_weight, in_proj_bias).chunk(3, dim=-1)
        else:
            q, k, v = F.linear(query, wq, bq), F.linear(key, wk, bk), F.linear(value, wv, bv)

    amask = _additive_mask(attn_mask, q.dtype)
    if is_causal and amask is None:
        amask = torch.full((L, S), float("-inf"), dtype=q.dtype, device=q.device).triu_(1)
    if amask is not None and amask.dim() == 2:
        amask = amask.unsqueeze(0)
    kpm = _additive_mask(key_padding_mask, q.dtype)

    if bias_k is not None and bias_v is not None:
        k = torch.cat([k, bias_k.expand(1, B, -1)], dim=0)
        v = torch.cat([v, bias_v.expand(1, B, -1)], dim=0)
        if amask is not None:
            amask = F.pad(amask, (0, 1))
        if kpm is not None:
            kpm = F.pad(kpm, (0, 1))

    q = q.reshape(L, B * num_heads, hd).transpose(0, 1)
    k = k.reshape(k.shape[0], B * num_heads, hd).transpose(0, 1) if static_k is None else static_k
    v = v.reshape(v.shape[0], B * num_heads, hd).transpose(0, 1) if static_v is None else static_v

    if add_zero_attn:
        k = torch.cat([k, k.new_zeros(k.shape[0], 1, hd)], dim=1)
        v = torch.cat([v, v.new_zeros(v.shape[0], 1, hd)], dim=1)
        if amask is not None:
            amask = F.pad(amask, (0, 1))
        if kpm is not None:
            kpm = F.pad(kpm, (0, 1))
    S2 = k.shape[1]

    if kpm is not None:
        kp = kpm.view(B, 1, 1, S2).expand(-1, num_heads, -1, -1).reshape(B * num_heads, 1, S2)
        amask = kp if amask is None else amask + kp
    if not training:
        dropout_p = 0.0

    if need_weights:
        scores = torch.bmm(q * (1.0 / math.sqrt(hd)), k.transpose(1, 2))
        if amask is not None:
            scores = scores + amask
        probs = torch.softmax(scores, dim=-1)
        if dropout_p > 0.0:
            probs = F.dropout(probs, p=dropout_p)
        ctxv = torch.bmm(probs, v)
        weights = probs.view(B, num_heads, L, S2)
        if average_attn_weights:
            weights = weights.mean(dim=1)
    else:
        m4 = None
        if amask is not None:
            # [B * heads, 1 or L, S] (key padding merged in) or [1, L, S]: both broadcast over the query axis
            m4 = amask.view(B, num_heads, amask.shape[1], S2) if amask.shape[0] == B * num_heads else amask.unsqueeze(0)
        ctxv = F.scaled_dot_product_attention(q.view(B, num_heads, L, hd), k.view(B, num_heads, S2, hd),
                                              v.view(B, num_heads, S2, hd), attn_mask=m4, dropout_p=dropout_p)
        ctxv = ctxv.reshape(B * num_heads, L, hd)
        weights = None

    ctxv = ctxv.transpose(0, 1).reshape(L * B, Es)
    out = F.linear(ctxv, out_proj_weight, out_proj_bias).view(L, B, -1)
    if not batched:
        out = out.squeeze(1)
        if weights is not None:
            weights = weights.squeeze(0)
    return out, weights
