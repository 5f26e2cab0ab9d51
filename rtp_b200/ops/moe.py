"""MoE token dispatch / combine by index on the GPU: row scatter / gather kernels that replace the reference's dense
``einsum("sec,sm->ecm")`` / ``einsum("sec,ecm->sm")`` (O(S*E*C*M)) by O(S*M) copies (rtp/module/moe.py:148,174)."""
import torch

from ..parallel.context import get_backend
from . import kernels as K


def use_kernels(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and get_backend() != "functional"


def _slots(idx, loc, valid, capacity):
    return torch.where(valid, idx * capacity + loc, torch.full_like(idx, -1)).to(torch.int32).contiguous()


class _Dispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, slot, rows):
        ctx.save_for_backward(slot)
        return K.moe_scatter(x.contiguous(), slot, None, rows)

    @staticmethod
    def backward(ctx, g):
        (slot,) = ctx.saved_tensors
        return K.moe_gather(g.contiguous(), slot, None), None, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, eo, slot, gate):
        eo = eo.contiguous()
        gate = gate.float().contiguous()
        ctx.save_for_backward(eo, slot, gate)
        return K.moe_gather(eo, slot, gate)

    @staticmethod
    def backward(ctx, dy):
        eo, slot, gate = ctx.saved_tensors
        dy = dy.contiguous()
        d_eo = K.moe_scatter(dy, slot, gate, eo.shape[0])
        d_gate = K.moe_rowdot(dy, eo, slot)
        return d_eo, None, d_gate


def dispatch(x, idx, loc, valid, num_experts, capacity):
    slot = _slots(idx, loc, valid, capacity)
    out = _Dispatch.apply(x, slot, num_experts * capacity)
    return out.view(num_experts, capacity, x.shape[1])


def combine(expert_output, idx, loc, gate, valid):
    E, C, M = expert_output.shape
    slot = _slots(idx, loc, valid, C)
    g = (gate * valid).float()
    return _Combine.apply(expert_output.reshape(E * C, M), slot, g).to(expert_output.dtype)
