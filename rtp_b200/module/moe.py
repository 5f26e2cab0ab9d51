"""Mixture-of-experts layers: the all-to-all GShard baseline (``MOELayer``) and the rotating-expert layer
(``WeightMOELayer``) in which expert weights travel around the ring and tokens never leave their GPU
(reference: rtp/module/moe.py:25-187)."""
from typing import Any, Optional, Union, cast

import torch
import torch.distributed as dist
from torch import Tensor, nn
from torch.nn import Module, ModuleList

from ..parallel.flat import RotatedModule
from ..parallel.rotated import rotated_apply
from ..parallel.context import get_context


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, group, input: Tensor) -> Tensor:  # type: ignore
        ctx.group = group
        input = input.contiguous()
        output = torch.empty_like(input)
        if dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_to_all_single(output, input, group=group)
        else:
            output.copy_(input)
        return output

    @staticmethod
    def backward(ctx: Any, *grad_output: Tensor):
        return (None, _AllToAll.apply(ctx.group, *grad_output))


def _dispatch(dispatch_mask: Tensor, x: Tensor) -> Tensor:
    return torch.einsum("sec,sm->ecm", dispatch_mask.to(x.dtype), x)


def _combine(combine_weights: Tensor, expert_output: Tensor) -> Tensor:
    return torch.einsum("sec,ecm->sm", combine_weights, expert_output)


class MOELayer(nn.Module):
    """Expert-parallel MoE with two all-to-alls per direction (GShard algorithm 2)."""

    def __init__(self, gate: Module, experts: Union[Module, ModuleList], group: Optional[Any] = None) -> None:
        super().__init__()
        self.gate = gate
        self.experts = cast(ModuleList, experts) if isinstance(experts, ModuleList) else ModuleList([experts])
        ctx = get_context(group)
        self.ring, self.world_size = ctx, ctx.world
        for expert in self.experts:
            for p in expert.parameters():
                p.expert = True  # type: ignore
        self.num_local_experts = len(self.experts)

    def forward(self, *input: Tensor, **kwargs: Any) -> Tensor:
        assert len(input) == 1, "only single input Tensor supported"
        assert len(input[0].shape) == 3, "input Tensor must have dimensions: (s)equence, (t)oken, (m)odel"
        d_model = input[0].shape[2]
        reshaped = input[0].reshape(-1, d_model)
        self.l_aux, combine_weights, dispatch_mask = self.gate(reshaped)
        dispatched = _dispatch(dispatch_mask, reshaped)
        dispatched = _AllToAll.apply(self.ring.group, dispatched)
        dispatched = dispatched.reshape(self.world_size, self.num_local_experts, -1, d_model)
        chunks = dispatched.chunk(self.num_local_experts, dim=1)
        outs = [expert(chunk) for chunk, expert in zip(chunks, self.experts)]
        expert_output = torch.cat(outs, dim=1)
        expert_output = _AllToAll.apply(self.ring.group, expert_output)
        expert_output = expert_output.reshape(self.world_size * self.num_local_experts, -1, d_model)
        combined = _combine(combine_weights, expert_output)
        return combined.reshape(input[0].shape)


class WeightMOELayer(RotatedModule):
    """Rotating experts: rank r owns ``num_local_experts`` whole experts (global ids ``r*L .. r*L+L-1``).
    The dispatched tensor ``[E, C, M]`` is chunked into N expert groups; at step i the visiting expert
    group ``(r+i) % N`` processes chunk ``(r+i) % N``."""

    def __init__(self, gate: Module, experts: Union[Module, ModuleList], group: Optional[Any] = None,
                 device=None, dtype=None, original_experts=None) -> None:
        super().__init__()
        self._setup_ring(group)
        self.gate = gate
        self.experts = cast(ModuleList, experts) if isinstance(experts, ModuleList) else ModuleList([experts])
        if device is not None or dtype is not None:
            self.experts.to(device=device, dtype=dtype)
        for expert in self.experts:
            for p in expert.parameters():
                p.expert = True  # type: ignore
        self.num_local_experts = len(self.experts)
        if original_experts is not None:
            with torch.no_grad():
                for p, q in zip(self.experts.parameters(), original_experts.parameters()):
                    p.copy_(q)
        self._pnames = [n for n, _ in self.experts.named_parameters()]
        self._flatten()

    def shard_parameters(self):
        return [p for _, p in self.experts.named_parameters()]

    def shard_names(self):
        return list(self._pnames)

    def shard_spec(self):
        return {f"experts.{n}": ("expert", self.num_local_experts) for n in self._pnames}

    def forward(self, *input: Tensor, **kwargs: Any) -> Tensor:
        assert len(input) == 1, "only single input Tensor supported"
        assert len(input[0].shape) == 3, "input Tensor must have dimensions: (s)equence, (t)oken, (m)odel"
        assert (input[0].shape[0] * input[0].shape[1]) % len(self.experts) == 0, \
            "number of tokens must be a multiple of the number of local experts"
        d_model = input[0].shape[2]
        reshaped = input[0].reshape(-1, d_model)
        self.l_aux, combine_weights, dispatch_mask = self.gate(reshaped)
        dispatched = _dispatch(dispatch_mask, reshaped)          # [E, C, M]
        N, L = self.world_size, self.num_local_experts
        experts, names = self.experts, self._pnames
        training = self.training

        def fn(j, views, disp):
            chunk = disp[j * L:(j + 1) * L]                       # the tokens routed to expert group j
            pmap = dict(zip(names, views))
            outs = []
            for e, expert in enumerate(experts):
                sub = {k[len(str(e)) + 1:]: v for k, v in pmap.items() if k.startswith(f"{e}.")}
                outs.append(torch.func.functional_call(expert, sub, (chunk[e:e + 1],)))
            return torch.cat(outs, dim=0)

        stochastic = training and any(isinstance(m, nn.Dropout) and m.p > 0 for m in experts.modules())
        expert_output = rotated_apply(self.ring, fn, self.shard_parameters(), self._full_param, self._layout,
                                      (dispatched,), combine="cat", cat_dim=0, inplace=self.inplace,
                                      stochastic=stochastic, owner=self)
        combined = _combine(combine_weights, expert_output)
        return combined.reshape(input[0].shape)
