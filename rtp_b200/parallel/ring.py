"""Ring transport over torch.distributed (gloo on CPU, NCCL on GPU).

Counterpart of the reference's ``_left_shift_buffer`` / ``_right_shift_buffer``
(rtp/module/collectives.py:202-238): one isend + one irecv per hop, returned as requests so that the
hop overlaps with compute.  Direction ``down`` sends to rank r-1 and receives from r+1 (forward
rotation), ``up`` is the reverse (backward rotation).
"""
import torch
import torch.distributed as dist

from .context import RingContext


def shift_async(ctx: RingContext, send: torch.Tensor, recv: torch.Tensor, direction: str):
    """Start one ring hop. Returns a list of requests to wait on (empty for a 1-rank ring)."""
    if ctx.world == 1:
        recv.copy_(send)
        return []
    if direction == "down":
        dst, src = ctx.down, ctx.up
    elif direction == "up":
        dst, src = ctx.up, ctx.down
    else:
        raise ValueError(direction)
    ops = [dist.P2POp(dist.isend, send, ctx.global_rank(dst), group=ctx.group),
           dist.P2POp(dist.irecv, recv, ctx.global_rank(src), group=ctx.group)]
    return dist.batch_isend_irecv(ops)


def wait_all(reqs):
    for r in reqs:
        r.wait()


def shift_inplace(ctx: RingContext, buf: torch.Tensor, direction: str, chunk_elems: int = 1 << 20):
    """Blocking hop that replaces ``buf`` by the neighbour's buffer using only a small staging chunk.

    This is the memory-lean variant: no second full-size buffer exists at any time (the reference's
    in-place modules receive into a full temporary, rtp/inplace/module/collectives.py:84,187-198).
    """
    if ctx.world == 1:
        return
    if buf.is_cuda and buf.is_contiguous() and (buf.numel() * buf.element_size()) % 16 == 0 and buf.data_ptr() % 16 == 0:
        from .context import get_backend
        if get_backend() != "functional":
            # sm_100a ring-shift kernel: NVLink P2P stores through a peer-mapped staging area, no NCCL on the path
            from .engine import get_engine
            get_engine(ctx).shift_inplace(buf, direction)
            return
    flat = buf.view(-1)
    n = flat.numel()
    stage = torch.empty(min(chunk_elems, n), dtype=flat.dtype, device=flat.device)
    for lo in range(0, n, chunk_elems):
        hi = min(lo + chunk_elems, n)
        piece = flat[lo:hi]
        st = stage[: hi - lo]
        wait_all(shift_async(ctx, piece, st, direction))
        piece.copy_(st)


def all_reduce_sum(ctx: RingContext, t: torch.Tensor):
    if ctx.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=ctx.group)
    return t
