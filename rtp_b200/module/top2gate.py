"""Top-2 gating (GShard) and its rotated variant whose gate weight ``[E/N, D]`` travels like a
column-parallel linear (reference: rtp/module/top2gate.py:25-220).

``top2gating`` reproduces the reference's slot assignment exactly (token-order cumsum, top-1 slots
before top-2 slots, capacity ``2S/E``); ``capacity_factor`` scales the capacity (1.0 = reference) and
``noise`` lets tests inject the Gumbel sample."""
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from ..parallel.context import get_backend
from ..parallel.flat import RotatedModule
from ..parallel.rotated import rotated_apply
from .utils import affine_weight, divide_and_check_no_remainder

gumbel_map: Dict[torch.device, Callable] = {}


def gumbel_rsample(shape: Tuple, device: torch.device) -> Tensor:
    g = gumbel_map.get(device)
    if g is None:
        one = torch.tensor(1.0, device=device)
        zero = torch.tensor(0.0, device=device)
        g = torch.distributions.gumbel.Gumbel(zero, one).rsample  # type: ignore
        gumbel_map[device] = g
    return g(shape)


def one_hot(tensor: torch.Tensor, num_classes: int) -> Tensor:
    assert num_classes > 0, "num_classes must be a positive integer"
    ret = torch.zeros(tensor.shape + (num_classes,), device=tensor.device, dtype=tensor.dtype)
    ret.scatter_(-1, tensor.unsqueeze(-1), 1)
    return ret


def top2_routing(logits: Tensor, capacity_factor: float = 1.0, noise: Optional[Tensor] = None):
    """Index form of top-2 gating: per token its two experts, slots, normalised gate values and validity.
    Returns (l_aux, idx[S,2], loc[S,2], gate[S,2], valid[S,2], capacity)."""
    S, E = logits.shape
    assert S % E == 0, "number of tokens must be a multiple of the number of experts"
    capacity = int(capacity_factor * 2 * S // E)
    if logits.is_cuda and E <= 64 and get_backend() != "functional":
        # fused kernels: softmax / top-1 / noisy top-2 per token, token-order slots in one block, no [S, E] one-hots
        if noise is None:
            noise = gumbel_rsample(logits.shape, device=logits.device)
        from ..ops import kernels as K
        l_aux, idx, loc, gate, valid = K.top2_gate(logits, capacity, noise)
        valid = valid.bool()
        idx = idx.long()
        mask1 = one_hot(idx[:, 0], E) * valid[:, :1]
        mask2 = one_hot(idx[:, 1], E) * valid[:, 1:]
        return l_aux, idx, loc.long(), gate, valid, capacity, mask1, mask2
    gates = F.softmax(logits, dim=1, dtype=torch.float)
    idx1 = torch.argmax(gates, dim=1)
    mask1 = one_hot(idx1, E)
    if noise is None:
        noise = gumbel_rsample(logits.shape, device=logits.device)
    noisy = (logits + noise).masked_fill(mask1.bool(), float("-inf"))
    idx2 = torch.argmax(noisy, dim=1)
    mask2 = one_hot(idx2, E)
    loc1 = torch.cumsum(mask1, dim=0) - 1
    loc2 = torch.cumsum(mask2, dim=0) - 1 + torch.sum(mask1, dim=0, keepdim=True)
    me = torch.mean(gates, dim=0)
    ce = torch.mean(mask1.float(), dim=0)
    l_aux = torch.mean(me * ce)
    mask1 = mask1 * torch.lt(loc1, capacity)
    mask2 = mask2 * torch.lt(loc2, capacity)
    loc1_s = torch.sum(loc1 * mask1, dim=1)
    loc2_s = torch.sum(loc2 * mask2, dim=1)
    g1 = (gates * mask1).sum(dim=1)
    g2 = (gates * mask2).sum(dim=1)
    denom = torch.clamp(g1 + g2, min=torch.finfo(g1.dtype).eps)
    g1, g2 = g1 / denom, g2 / denom
    valid = torch.stack([mask1.sum(1) > 0, mask2.sum(1) > 0], dim=1)
    return (l_aux, torch.stack([idx1, idx2], 1), torch.stack([loc1_s, loc2_s], 1).long(),
            torch.stack([g1, g2], 1), valid, capacity, mask1, mask2)


def top2gating(logits: Tensor, capacity_factor: float = 1.0, noise: Optional[Tensor] = None
               ) -> Tuple[Tensor, Tensor, Tensor]:
    """Returns ``(l_aux, combine_weights[S,E,C], dispatch_mask[S,E,C])`` like the reference."""
    l_aux, idx, loc, gate, valid, capacity, mask1, mask2 = top2_routing(logits, capacity_factor, noise)
    gates1 = gate[:, 0].unsqueeze(-1) * mask1
    gates2 = gate[:, 1].unsqueeze(-1) * mask2
    loc1_sc = one_hot(loc[:, 0], capacity)
    loc2_sc = one_hot(loc[:, 1], capacity)
    combine = gates1.unsqueeze(2) * loc1_sc.unsqueeze(1) + gates2.unsqueeze(2) * loc2_sc.unsqueeze(1)
    return l_aux.to(logits.dtype), combine.to(logits.dtype), combine.bool()


class Top2Gate(nn.Module):
    """Plain (replicated) gate: ``wg`` is a bias-free linear ``[E, D]``."""

    wg: nn.Linear

    def __init__(self, model_dim: int, num_experts: int, capacity_factor: float = 1.0) -> None:
        super().__init__()
        self.wg = nn.Linear(model_dim, num_experts, bias=False)
        self.capacity_factor = capacity_factor

    def forward(self, input: torch.Tensor) -> Tuple[Tensor, Tensor, Tensor]:  # type: ignore
        return top2gating(self.wg(input), self.capacity_factor)

    def route(self, input: torch.Tensor):
        """Index form of the gating decision (see ``top2_routing``): no [S, E, C] tensors are built."""
        return top2_routing(self.wg(input), self.capacity_factor)[:6]


class WeightTop2Gate(RotatedModule):
    """Gate whose weight rows (experts) are sharded ``[E/N, D]`` and rotate; logits of all experts are
    assembled on every rank for its own tokens."""

    def __init__(self, model_dim: int, num_experts: int, gate: Optional[Top2Gate] = None, device=None, dtype=None,
                 group=None, capacity_factor: float = 1.0) -> None:
        super().__init__()
        self._setup_ring(group)
        self.model_dim, self.num_experts = model_dim, num_experts
        self.capacity_factor = capacity_factor
        self.num_local_experts = divide_and_check_no_remainder(num_experts, self.world_size)
        self.wg = nn.Linear(model_dim, self.num_local_experts, bias=False, device=device, dtype=dtype)
        if gate is not None:
            self.affine_weight(self.wg, gate.wg)
        self._flatten()

    def affine_weight(self, wg, layer):
        affine_weight(wg.weight, layer.weight, self.num_local_experts, 0, self.world_size, self.rank)

    def shard_parameters(self):
        return [self.wg.weight]

    def shard_names(self):
        return ["weight"]

    def shard_spec(self):
        return {"wg.weight": ("split", 0)}

    def logits(self, input: torch.Tensor) -> torch.Tensor:
        def fn(j, views, x):
            return F.linear(x, views[0])
        return rotated_apply(self.ring, fn, self.shard_parameters(), self._full_param, self._layout, (input,),
                             combine="cat", cat_dim=-1, inplace=self.inplace, owner=self)

    def forward(self, input: torch.Tensor) -> Tuple[Tensor, Tensor, Tensor]:  # type: ignore
        return top2gating(self.logits(input), self.capacity_factor)

    def route(self, input: torch.Tensor):
        return top2_routing(self.logits(input), self.capacity_factor)[:6]
