"""Functional rotation engine: one ``autograd.Function`` that rotates a flat weight shard around the
ring in forward and carries the shard's gradient home in backward.

Semantics follow the reference's out-of-place modules (rtp/module/linear.py:204-236 forward loop,
rtp/module/collectives.py:240-317 regions): at forward step ``i`` rank ``r`` computes with shard
``(r+i) % N`` while the next shard is already in flight; backward visits the shards in the reverse
order and adds its local weight gradient to the partial sum that travels with each shard, so the
gradient that reaches the owner is the sum over all ranks.

Differences by design:
  * the home shard never moves (visitors live in two work buffers), so forward-only passes and
    repeated forwards are safe;
  * no AccumulateGrad hooks: the reduce-and-forward of gradients happens inside ``backward``;
  * backward recomputes each step's local function instead of keeping N autograd graphs alive, so
    the activation memory of a rotated layer is that of its inputs only;
  * ``inplace=True`` rotates the single flat buffer itself through a small staging chunk and, in
    no-grad mode, performs the N-th restoring shift.
"""
from typing import Callable, List, Sequence, Tuple

import torch

from .context import RingContext
from . import ring


class ShardLayout:
    """Placement of a layer's shard tensors inside one flat buffer (each tensor 128-byte aligned)."""

    ALIGN_BYTES = 128

    def __init__(self, named_shapes: Sequence[Tuple[str, Sequence[int]]], dtype: torch.dtype):
        self.names = [n for n, _ in named_shapes]
        self.shapes = [tuple(s) for _, s in named_shapes]
        self.dtype = dtype
        esz = torch.empty((), dtype=dtype).element_size()
        align = max(1, self.ALIGN_BYTES // esz)
        self.offsets = []
        off = 0
        for s in self.shapes:
            self.offsets.append(off)
            n = 1
            for d in s:
                n *= d
            off += (n + align - 1) // align * align
        self.numel = off

    def views(self, flat: torch.Tensor) -> List[torch.Tensor]:
        out = []
        for off, shape in zip(self.offsets, self.shapes):
            n = 1
            for d in shape:
                n *= d
            out.append(flat[off:off + n].view(shape))
        return out

    def offset_of(self, name: str) -> int:
        return self.offsets[self.names.index(name)]


def _rng_snapshot(device):
    cpu = torch.get_rng_state()
    cuda = torch.cuda.get_rng_state(device) if device.type == "cuda" else None
    return cpu, cuda


def _rng_restore(snap, device):
    cpu, cuda = snap
    torch.set_rng_state(cpu)
    if cuda is not None:
        torch.cuda.set_rng_state(cuda, device)


class _Spec:
    """Non-tensor arguments of one rotated call."""

    def __init__(self, ctx, fn, layout, combine, cat_dim, inplace, stochastic, n_params, needs_bwd, owner):
        self.ctx: RingContext = ctx
        self.fn: Callable = fn
        self.layout: ShardLayout = layout
        self.combine = combine
        self.cat_dim = cat_dim
        self.inplace = inplace
        self.stochastic = stochastic
        self.n_params = n_params
        self.needs_bwd = needs_bwd
        self.owner = owner


def _call(spec, j, flat, inputs):
    out = spec.fn(j, spec.layout.views(flat), *inputs)
    if isinstance(out, tuple):
        return out[0], out[1:]
    return out, ()


class _RotatedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, spec: _Spec, flat: torch.Tensor, *tensors):
        rc, N, r = spec.ctx, spec.ctx.world, spec.ctx.rank
        inputs = tensors[spec.n_params:]
        outs = [None] * N
        aux = ()
        snaps = [None] * N
        dev = flat.device
        if spec.inplace:
            for i in range(N):
                j = (r + i) % N
                if spec.stochastic:
                    snaps[i] = _rng_snapshot(dev)
                outs[j], aux = _call(spec, j, flat, inputs)
                if i < N - 1:
                    ring.shift_inplace(rc, flat, "down")
            if N > 1:
                if spec.needs_bwd:
                    if spec.owner is not None:
                        spec.owner._displaced = True
                else:
                    ring.shift_inplace(rc, flat, "down")  # N-th shift: every shard is home again
        else:
            work = [None, None]
            cur = flat
            for i in range(N):
                j = (r + i) % N
                reqs = []
                if i < N - 1:
                    nxt = i & 1
                    if work[nxt] is None:
                        work[nxt] = torch.empty_like(flat)
                    reqs = ring.shift_async(rc, cur, work[nxt], "down")
                if spec.stochastic:
                    snaps[i] = _rng_snapshot(dev)
                outs[j], aux = _call(spec, j, cur, inputs)
                if i < N - 1:
                    ring.wait_all(reqs)
                    cur = work[i & 1]
        if spec.combine == "cat":
            ctx.split_sizes = [o.shape[spec.cat_dim] for o in outs]
            out = torch.cat(outs, dim=spec.cat_dim) if N > 1 else outs[0]
        else:
            out = outs[0]
            for o in outs[1:]:
                out = out + o
        ctx.spec = spec
        ctx.flat = flat
        ctx.snaps = snaps
        ctx.save_for_backward(*inputs)
        ctx.n_aux = len(aux)
        for a in aux:
            if isinstance(a, torch.Tensor):
                ctx.mark_non_differentiable(a)
        return (out, *aux)

    @staticmethod
    def backward(ctx, grad_out, *grad_aux):
        spec: _Spec = ctx.spec
        rc, N, r = spec.ctx, spec.ctx.world, spec.ctx.rank
        flat = ctx.flat
        inputs = ctx.saved_tensors
        layout = spec.layout
        dev = flat.device
        diff_in = [isinstance(t, torch.Tensor) and t.is_floating_point() and need
                   for t, need in zip(inputs, ctx.needs_input_grad[2 + spec.n_params:])]
        dins = [None] * len(inputs)
        if spec.combine == "cat":
            gparts = list(torch.split(grad_out, ctx.split_sizes, dim=spec.cat_dim))

        # weights: out-of-place = visitors stream through two work buffers, starting with a prologue hop
        work = [None, None]
        cur = flat
        wreqs = []
        if not spec.inplace and N > 1:
            work[0] = torch.empty_like(flat)
            ring.wait_all(ring.shift_async(rc, flat, work[0], "up"))
            cur = work[0]
        g_in = None
        g_reqs = []
        g_recv = None
        g_send = None
        keep_rng = _rng_snapshot(dev) if spec.stochastic else None
        for s in range(N):
            i = N - 1 - s
            j = (r + i) % N
            last = s == N - 1
            # prefetch the next visitor while this step computes
            if not spec.inplace and N > 1 and s < N - 2:
                nxt = (s + 1) & 1
                if work[nxt] is None:
                    work[nxt] = torch.empty_like(flat)
                wreqs = ring.shift_async(rc, cur, work[nxt], "up")
            src = flat if (last and not spec.inplace) else cur
            if spec.inplace:
                src = flat
            leaf = src.detach().requires_grad_(True)
            local_inputs = [t.detach().requires_grad_(True) if d else t for t, d in zip(inputs, diff_in)]
            if spec.stochastic:
                _rng_restore(ctx.snaps[i], dev)
            with torch.enable_grad():
                out_j, _ = _call(spec, j, leaf, local_inputs)
            g_j = gparts[j] if spec.combine == "cat" else grad_out
            wrt = [leaf] + [t for t, d in zip(local_inputs, diff_in) if d]
            grads = torch.autograd.grad(out_j, wrt, g_j, allow_unused=True)
            g_flat = grads[0] if grads[0] is not None else torch.zeros_like(flat)
            k = 1
            for idx, d in enumerate(diff_in):
                if d:
                    g = grads[k]
                    k += 1
                    if g is not None:
                        dins[idx] = g if dins[idx] is None else dins[idx] + g
            # travelling gradient: add the partial that arrived with this shard, pass the sum on
            if s > 0:
                ring.wait_all(g_reqs)
                g_flat = g_flat + g_recv
            if not last:
                g_send = g_flat.contiguous()
                g_recv = torch.empty_like(g_send)
                g_reqs = ring.shift_async(rc, g_send, g_recv, "up")
            else:
                g_in = g_flat
            # move the weights on
            if spec.inplace:
                if not last:
                    ring.shift_inplace(rc, flat, "up")
            elif N > 1 and s < N - 2:
                ring.wait_all(wreqs)
                cur = work[(s + 1) & 1]
        if spec.stochastic:
            _rng_restore(keep_rng, dev)
        if spec.inplace and spec.owner is not None:
            spec.owner._displaced = False
        if spec.owner is not None:
            spec.owner._last_flat_grad = g_in
        pgrads = [None] * spec.n_params
        need_p = ctx.needs_input_grad[2:2 + spec.n_params]
        for idx, v in enumerate(layout.views(g_in)):
            if need_p[idx]:
                pgrads[idx] = v
        return (None, None, *pgrads, *dins)


def rotated_apply(ctx: RingContext, fn: Callable, params: Sequence[torch.Tensor], flat: torch.Tensor,
                  layout: ShardLayout, inputs: Sequence, *, combine: str = "cat", cat_dim: int = -1,
                  inplace: bool = False, stochastic: bool = False, owner=None):
    """Run ``fn(j, shard_views, *inputs)`` for every shard ``j`` as it visits this rank and combine the
    partial outputs (``cat`` along ``cat_dim`` in shard order, or ``sum``).

    ``params`` are the module's registered parameters (views into ``flat`` in ``layout`` order); they are
    passed through autograd so that their ``.grad`` receives the ring-reduced gradient of the home shard.
    ``fn`` may return a tuple: the first element is combined, the rest (of the last step) is returned
    as non-differentiable auxiliary output.
    """
    if combine not in ("cat", "sum"):
        raise ValueError(combine)
    if inplace and owner is not None and getattr(owner, "_displaced", False):
        raise RuntimeError("in-place rotated layer called while its shards are displaced: the backward of the "
                           "previous grad-mode forward has not run yet (use the out-of-place layer for that)")
    needs_bwd = torch.is_grad_enabled() and (
        any(p.requires_grad for p in params)
        or any(isinstance(t, torch.Tensor) and t.requires_grad for t in inputs))
    spec = _Spec(ctx, fn, layout, combine, cat_dim, inplace, stochastic, len(params), needs_bwd, owner)
    out = _RotatedFn.apply(spec, flat, *params, *inputs)
    if len(out) == 1:
        return out[0]
    return out
