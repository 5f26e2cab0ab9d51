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


_plain_guard_done = False
_capture_warned = False


def _guard_plain_launches(world: int, on_gpu: bool) -> None:
    """A training step with rotating experts on 8 GPUs ended twice with an illegal-instruction error when its kernels
    were queued back to back, and ran clean (4 and 8 GPUs) with a synchronise and a status read after every launch; the
    cause is not known.  Until it is, the first rotating-expert layer that runs on a ring of more than two GPUs turns
    that serialised mode on for the process (``RTP_MOE_PLAIN=1`` opts out).  Launches inside a CUDA-graph capture are
    not covered: serialised mode skips them."""
    global _plain_guard_done, _capture_warned
    if not on_gpu or world <= 2:
        return
    import os
    import warnings
    if (not _capture_warned and torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()
            and os.environ.get("RTP_MOE_PLAIN", "0") in ("", "0")):
        _capture_warned = True
        warnings.warn("rtp_b200: rotating experts on more than two GPUs are being captured into a CUDA graph; replayed "
                      "launches are queued back to back, which is the mode in which the open fault was seen",
                      stacklevel=3)
    if _plain_guard_done:
        return
    _plain_guard_done = True
    from ..parallel.context import get_backend
    if get_backend() == "functional" or os.environ.get("RTP_MOE_PLAIN", "0") not in ("", "0"):
        return
    from ..ops import _lib
    if not _lib.set_serialize(True):      # returns the previous setting
        warnings.warn("rtp_b200: rotating experts on more than two GPUs run with serialised launches (a synchronise "
                      "after every library launch); set RTP_MOE_PLAIN=1 to queue them back to back", stacklevel=3)


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


def dispatch_by_index(x: Tensor, idx: Tensor, loc: Tensor, valid: Tensor, num_experts: int, capacity: int) -> Tensor:
    """Index form of ``einsum("sec,sm->ecm", dispatch_mask, x)``: token s goes to slot ``loc[s, k]`` of expert
    ``idx[s, k]`` for each valid choice k.  O(S*M) instead of O(S*E*C*M)."""
    from ..ops import moe as MK
    if MK.use_kernels(x):
        return MK.dispatch(x, idx, loc, valid, num_experts, capacity)
    S, M = x.shape
    dummy = num_experts * capacity
    slot = torch.where(valid, idx * capacity + loc, torch.full_like(idx, dummy))
    out = x.new_zeros(dummy + 1, M)
    out = out.index_copy(0, slot.reshape(-1), x.repeat_interleave(2, dim=0))
    return out[:dummy].view(num_experts, capacity, M)


def combine_by_index(expert_output: Tensor, idx: Tensor, loc: Tensor, gate: Tensor, valid: Tensor) -> Tensor:
    """Index form of ``einsum("sec,ecm->sm", combine_weights, expert_output)``."""
    from ..ops import moe as MK
    if MK.use_kernels(expert_output):
        return MK.combine(expert_output, idx, loc, gate, valid)
    E, C, M = expert_output.shape
    flat = torch.cat([expert_output.reshape(E * C, M), expert_output.new_zeros(1, M)])
    slot = torch.where(valid, idx * C + loc, torch.full_like(idx, E * C))
    g = (gate * valid).to(expert_output.dtype)
    return (flat[slot] * g.unsqueeze(-1)).sum(dim=1)


def _route(gate_module, x):
    """(l_aux, dispatch fn, combine fn) from a gate: index form when the gate offers ``route``, else the dense
    [S, E, C] tensors of the reference."""
    if hasattr(gate_module, "route"):
        l_aux, idx, loc, g, valid, capacity = gate_module.route(x)
        E = getattr(gate_module, "num_experts", None) or gate_module.wg.out_features
        return (l_aux.to(x.dtype), lambda t: dispatch_by_index(t, idx, loc, valid, E, capacity),
                lambda eo: combine_by_index(eo, idx, loc, g, valid))
    l_aux, combine_weights, dispatch_mask = gate_module(x)
    return l_aux, (lambda t: _dispatch(dispatch_mask, t)), (lambda eo: _combine(combine_weights, eo))


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
        self.l_aux, dispatch, combine = _route(self.gate, reshaped)
        dispatched = dispatch(reshaped)
        dispatched = _AllToAll.apply(self.ring.group, dispatched)
        dispatched = dispatched.reshape(self.world_size, self.num_local_experts, -1, d_model)
        chunks = dispatched.chunk(self.num_local_experts, dim=1)
        outs = [expert(chunk) for chunk, expert in zip(chunks, self.experts)]
        expert_output = torch.cat(outs, dim=1)
        expert_output = _AllToAll.apply(self.ring.group, expert_output)
        expert_output = expert_output.reshape(self.world_size * self.num_local_experts, -1, d_model)
        combined = combine(expert_output)
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
        # flat order: all (weight, bias) blocks of linear1, then of linear2, then anything else, so that each linear
        # of all local experts is one contiguous range with a uniform stride
        names = [n for n, _ in self.experts.named_parameters()]

        def key(n):
            parts = n.split(".")
            layer = parts[1] if len(parts) > 2 else ""
            rank = {"linear1": 0, "linear2": 1}.get(layer, 2)
            return (rank, int(parts[0]) if parts[0].isdigit() else 0, 0 if n.endswith("weight") else 1, n)
        self._pnames = sorted(names, key=key)
        self._flatten()

    def shard_parameters(self):
        d = dict(self.experts.named_parameters())
        return [d[n] for n in self._pnames]

    def shard_names(self):
        return list(self._pnames)

    def shard_spec(self):
        return {f"experts.{n}": ("expert", self.num_local_experts) for n in self._pnames}

    def _fused_ok(self, dispatched):
        from ..parallel import fused
        if self.inplace and self.world_size > 1:
            return False          # memory-lean mode: the expert shard itself travels (rotated_apply + ring-shift kernel)
        ex = self.experts[0]
        if not (hasattr(ex, "linear1") and hasattr(ex, "linear2") and isinstance(ex.linear1, nn.Linear)
                and isinstance(ex.linear2, nn.Linear) and ex.linear1.bias is not None and ex.linear2.bias is not None):
            return False
        act = getattr(ex, "activation", None)
        if not (act is None or isinstance(act, (nn.GELU, nn.ReLU)) or act is torch.nn.functional.gelu):
            return False
        if self.training and any(isinstance(m, nn.Dropout) and m.p > 0 for m in ex.modules()):
            return False
        if self.num_local_experts * self.world_size > 8 or dispatched.shape[1] % 8:
            return False
        if set(n.split(".", 1)[1] for n in self._pnames) != {"linear1.weight", "linear1.bias", "linear2.weight", "linear2.bias"}:
            return False
        return fused.use_fused(dispatched, self._full_param)

    def forward(self, *input: Tensor, **kwargs: Any) -> Tensor:
        assert len(input) == 1, "only single input Tensor supported"
        assert len(input[0].shape) == 3, "input Tensor must have dimensions: (s)equence, (t)oken, (m)odel"
        assert (input[0].shape[0] * input[0].shape[1]) % len(self.experts) == 0, \
            "number of tokens must be a multiple of the number of local experts"
        d_model = input[0].shape[2]
        _guard_plain_launches(self.world_size, input[0].is_cuda)
        reshaped = input[0].reshape(-1, d_model)
        self.l_aux, dispatch, combine = _route(self.gate, reshaped)
        dispatched = dispatch(reshaped)                          # [E, C, M]
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
        if self._fused_ok(dispatched):
            from ..parallel.engine import fused_experts
            return combine(fused_experts(self, dispatched)).reshape(input[0].shape)
        expert_output = rotated_apply(self.ring, fn, self.shard_parameters(), self._full_param, self._layout,
                                      (dispatched,), combine="cat", cat_dim=0, inplace=self.inplace,
                                      stochastic=stochastic, owner=self)
        combined = combine(expert_output)
        return combined.reshape(input[0].shape)
