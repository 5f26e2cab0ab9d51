"""Adam / AdamW for rotated models.

Each rank optimises only the shards it owns (the registered parameters of rotated layers) plus its copy
of the replicated parameters.  Two things the reference leaves to chance are handled here:

* replicated parameters (LayerNorm, anything outside a rotated layer) receive only the gradient of the
  local batch; their gradients are summed over the ring before the update, so the replicas stay equal
  and the model matches a single-process run;
* biases of row-sharded projections are stored as ``b / N`` on every rank and every copy receives the
  full bias gradient; their update is scaled by ``1 / N`` so that the sum of the copies moves like one
  bias (the parameters carry ``rtp_sum_replicated = N``).

On bf16 CUDA parameters the update (with optional ``clip_grad_value_`` clamp) runs as one multi-tensor
sm_100a kernel over all tensors; elsewhere it is evaluated with torch ops.
"""
import math
from typing import Iterable, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..parallel.context import get_context


def _is_sharded(p) -> bool:
    return bool(getattr(p, "rtp_sharded", False)) or bool(getattr(p, "expert", False))


def sync_replicated_grads(params: Iterable[torch.Tensor], group=None):
    """Sum the gradients of replicated (non-rotated) parameters over the ring in one flat bucket."""
    ctx = get_context(group)
    if ctx.world == 1:
        return
    reps = [p for p in params if p.grad is not None and not _is_sharded(p)]
    if not reps:
        return
    flat = torch.cat([p.grad.reshape(-1) for p in reps])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=ctx.group)
    off = 0
    for p in reps:
        n = p.numel()
        p.grad.copy_(flat[off:off + n].view_as(p.grad))
        off += n


def clip_grad_value_(params: Iterable[torch.Tensor], clip_value: float):
    for p in params:
        if p.grad is not None:
            p.grad.clamp_(-clip_value, clip_value)


class ShardedAdam(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adamw=False,
                 clip_value: Optional[float] = None, group=None, state_dtype=None,
                 sync_replicated: bool = True):
        """``state_dtype``: dtype policy of the moments of bf16 / fp16 parameters: ``None`` / ``"fp32"`` (default),
        ``"mixed"`` (first moment bf16, second moment fp32) or ``"bf16"`` (both bf16, the layout ``torch.optim.Adam``
        gives bf16 parameters; its second moment cannot decay, see ``ops.kernels.adam_state_dtypes``).  Moments of
        fp32 / fp64 parameters always have the parameter's dtype."""
        if isinstance(params, nn.Module):
            params = params.parameters()
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.adamw = adamw
        self.clip_value = clip_value
        self.ring = get_context(group)
        self.state_dtype = state_dtype
        self.sync_replicated = sync_replicated
        self._plan = None
        self._plan_key = None
        self._step_dev = None
        self._step = 0

    def _all_params(self):
        for g in self.param_groups:
            for p in g["params"]:
                yield p

    @staticmethod
    def _lr_mult(p) -> float:
        n = getattr(p, "rtp_sum_replicated", None)
        return 1.0 / n if n else 1.0

    def _init_state(self, p):
        st = self.state[p]
        if not st:
            if p.dtype in (torch.bfloat16, torch.float16):
                from ..ops.kernels import adam_state_dtypes
                dt_m, dt_v = adam_state_dtypes(self.state_dtype)
            else:
                dt_m = dt_v = p.dtype
            st["exp_avg"] = torch.zeros_like(p, dtype=dt_m, memory_format=torch.preserve_format)
            st["exp_avg_sq"] = torch.zeros_like(p, dtype=dt_v, memory_format=torch.preserve_format)
        return st

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.sync_replicated:
            sync_replicated_grads(self._all_params(), self.ring.group)
        self._step += 1
        params = [p for p in self._all_params() if p.grad is not None]
        fusable = params and all(p.is_cuda and p.dtype == torch.bfloat16 and p.grad.dtype == torch.bfloat16
                                 and p.is_contiguous() and p.grad.is_contiguous() for p in params) \
            and len(self.param_groups) == 1
        if fusable:
            self._step_fused(params)
            from ..ops import rng
            rng.advance(params[0].device)       # the kernels' dropout masks change with every optimizer step
        else:
            self._step_torch(params)
        return loss

    def _step_torch(self, params):
        for g in self.param_groups:
            lr, (b1, b2), eps, wd = g["lr"], g["betas"], g["eps"], g["weight_decay"]
            bc1 = 1 - b1 ** self._step
            bc2 = 1 - b2 ** self._step
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self._init_state(p)
                grad = p.grad
                if self.clip_value is not None:
                    grad = grad.clamp(-self.clip_value, self.clip_value)
                mult = self._lr_mult(p)
                if wd:
                    if self.adamw:
                        p.mul_(1 - lr * mult * wd)
                    else:
                        grad = grad.add(p, alpha=wd)
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.mul_(b1).add_(grad.to(m.dtype), alpha=1 - b1)
                gv = grad.to(v.dtype)
                v.mul_(b2).addcmul_(gv, gv, value=1 - b2)
                denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
                upd = (m.to(denom.dtype) / denom).to(p.dtype)
                p.add_(upd, alpha=-(lr * mult) / bc1)

    def _step_fused(self, params):
        from ..ops import kernels as K
        key = tuple((p.data_ptr(), p.grad.data_ptr()) for p in params)
        if self._plan is None or key != self._plan_key:
            entries = []
            for p in params:
                st = self._init_state(p)
                entries.append((p, p.grad, st["exp_avg"], st["exp_avg_sq"], self._lr_mult(p)))
            self._plan = K.AdamPlan(entries, params[0].device)
            self._plan_key = key
        if self._step_dev is None:
            self._step_dev = torch.zeros(1, dtype=torch.int64, device=params[0].device)
            self._step_dev.fill_(self._step - 1)
        self._step_dev.add_(1)
        g = self.param_groups[0]
        self._plan.step(self._step_dev, g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"],
                        self.adamw, self.clip_value or 0.0)


class ShardedAdamW(ShardedAdam):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, **kw):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adamw=True, **kw)
