"""Fused rotation engine: peer-mapped workspace + launch of the sm_100a rotation kernels.

One engine exists per (process, ring).  It owns a ``cudaMalloc``'d workspace — a flag block, two banks of N-1 weight
slots (one slot per visiting shard; the second bank receives the next launch's shards while the current launch computes)
and N gradient slots (one per contributing rank) — whose CUDA-IPC handle is exchanged once over the ring's process
group; afterwards every kernel launch only passes raw pointers.  The kernels themselves push weight shards from their
owner's home buffer into the consumer's slot with NVLink P2P stores, store weight-gradient tiles straight into the
owner's gradient slots and synchronise through monotonically increasing counters (see csrc/gemm_kernel.cuh), so there
is no NCCL send/recv, no copy kernel and no host involvement between rotation steps.

The memory-lean in-place mode (``inplace=True`` layers) uses none of these slots: the layer's single flat buffer itself
travels, one hop per rotation step, through a small staging area (``csrc/ring_shift.cu``).
"""
import ctypes as C
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib, kernels as K
from .context import RingContext

_engines: Dict[object, "FusedEngine"] = {}
_reserved_bytes = 0
DEFAULT_TIMEOUT_NS = 2_000_000_000


def reserve_shard_bytes(nbytes: int):
    """Rotated modules announce their shard size at construction so that the workspace, which is
    allocated at the first fused call, can hold the largest one."""
    global _reserved_bytes
    _reserved_bytes = max(_reserved_bytes, int(nbytes))


def _round_up(x, a):
    return (x + a - 1) // a * a


class FusedEngine:
    def __init__(self, ctx: RingContext, slot_bytes: int, ctas: Optional[int] = None,
                 timeout_ns: int = DEFAULT_TIMEOUT_NS):
        self.ctx = ctx
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.ctas = ctas or _lib.lib().rtp_sm_count()
        self.timeout_ns = timeout_ns
        self.ws_local = None
        self.mapped = {}
        self._host_status = C.c_ulonglong(0)
        self._staging = None            # (local, {rank: mapped}) of the in-place ring shift, created on first use
        self.shift_lanes = 32
        self._allocate(slot_bytes)

    def _allocate(self, slot_bytes: int):
        """Create the local workspace and map every peer's (collective over the ring)."""
        L = _lib.lib()
        ctx = self.ctx
        self.slot_bytes = _round_up(max(slot_bytes, 256), 1 << 16)
        ws = C.c_void_p()
        _lib.check(L.rtp_ws_create_world(self.slot_bytes if ctx.world > 1 else 256, ctx.world, C.byref(ws)),
                   "rtp_ws_create_world")
        self.ws_local = ws.value
        self.mapped = {}
        ptrs = [None] * ctx.world
        ptrs[ctx.rank] = self.ws_local
        if ctx.world > 1:
            handle = (C.c_char * 64)()
            _lib.check(L.rtp_ws_ipc_get(self.ws_local, handle), "rtp_ws_ipc_get")
            gathered = [None] * ctx.world
            dist.all_gather_object(gathered, bytes(handle), group=ctx.group)
            for r, h in enumerate(gathered):
                if r == ctx.rank:
                    continue
                out = C.c_void_p()
                buf = C.create_string_buffer(h, 64)
                _lib.check(L.rtp_ws_ipc_open(buf, C.byref(out)), "rtp_ws_ipc_open")
                ptrs[r] = out.value
                self.mapped[r] = out.value
            dist.barrier(group=ctx.group)
        self.ring = _lib.Ring()
        self.ring.rank, self.ring.world = ctx.rank, ctx.world
        for r in range(ctx.world):
            self.ring.ws[r] = ptrs[r]
        self.ring.slot_bytes = self.slot_bytes
        self.ring.ctas = self.ctas
        self.ring.timeout_ns = self.timeout_ns

    def grow(self, slot_bytes: int):
        """Replace the workspace by a larger one. Collective: every rank of the ring must call it at the same
        point of the program (it does when the need arises from constructing the same model everywhere)."""
        L = _lib.lib()
        torch.cuda.synchronize()
        if self.ctx.world > 1:
            dist.barrier(group=self.ctx.group)          # nobody is still pushing into the old slots
        for ptr in self.mapped.values():
            L.rtp_ws_ipc_close(ptr)
        if self.ctx.world > 1:
            dist.barrier(group=self.ctx.group)
        L.rtp_ws_destroy(self.ws_local)
        self._allocate(slot_bytes)

    # -- in-place ring shift ----------------------------------------------------------------------
    def _ensure_staging(self):
        """Create this rank's staging area and map the neighbours' (collective over the ring, first use only)."""
        if self._staging is not None:
            return self._staging
        L = _lib.lib()
        ctx = self.ctx
        mine = C.c_void_p()
        if L.rtp_shift_staging_create(self.shift_lanes, C.byref(mine)) != 0:
            raise RuntimeError("staging: " + L.rtp_shift_last_error().decode())
        ptrs = {ctx.rank: mine.value}
        handle = (C.c_char * 64)()
        _lib.check(L.rtp_ws_ipc_get(mine.value, handle), "rtp_ws_ipc_get")
        gathered = [None] * ctx.world
        dist.all_gather_object(gathered, bytes(handle), group=ctx.group)
        for r in {ctx.up, ctx.down} - {ctx.rank}:
            out = C.c_void_p()
            buf = C.create_string_buffer(gathered[r], 64)
            _lib.check(L.rtp_ws_ipc_open(buf, C.byref(out)), "rtp_ws_ipc_open")
            ptrs[r] = out.value
        dist.barrier(group=ctx.group)
        self._staging = ptrs
        return ptrs

    def staging_bytes(self) -> int:
        return int(_lib.lib().rtp_shift_staging_bytes(self.shift_lanes)) if self._staging is not None else 0

    def shift_inplace(self, buf: torch.Tensor, direction: str):
        """Replace ``buf`` (the same number of bytes on every rank) by the ring neighbour's buffer: ``down`` sends to rank
        r-1 and receives from r+1 (forward rotation), ``up`` the reverse.  Only a small staging area is used."""
        ctx = self.ctx
        if ctx.world == 1:
            return
        ptrs = self._ensure_staging()
        dst, src = (ctx.down, ctx.up) if direction == "down" else (ctx.up, ctx.down)
        nbytes = buf.numel() * buf.element_size()
        one = C.c_void_p * 1
        status = _lib.status_word(buf.device)
        rc = _lib.lib().rtp_ring_shift(1, one(buf.data_ptr()), nbytes, one(ptrs[ctx.rank]), one(ptrs[dst]), one(ptrs[src]),
                                       0 if direction == "down" else 1, self.shift_lanes, one(status.data_ptr()),
                                       self.timeout_ns, _lib.stream_ptr())
        if rc != 0:
            raise RuntimeError("rtp_ring_shift: " + _lib.lib().rtp_shift_last_error().decode())

    def ones_row(self, n: int) -> torch.Tensor:
        """A row of at least ``n`` bf16 ones (the A operand of the bias-gradient GEMM phase); grown on demand, and never
        while a CUDA graph that captured the old row may still be replayed."""
        row = getattr(self, "_ones", None)
        if row is None or row.numel() < n:
            if row is not None and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("ones row would have to grow during graph capture")
            row = torch.ones(max(n, 32768), dtype=torch.bfloat16, device=self.device)
            self._old_ones = getattr(self, "_old_ones", []) + ([self._ones] if getattr(self, "_ones", None) is not None else [])
            self._ones = row
        return row

    def counters(self):
        """(arrive, done, uses) lists of this rank's slot counters (synchronises the stream)."""
        L = _lib.lib()
        n = int(L.rtp_ws_num_counters())
        buf = (C.c_ulonglong * (3 * n))()
        _lib.check(L.rtp_ws_counters(self.ws_local, buf, _lib.stream_ptr()), "rtp_ws_counters")
        vals = list(buf)
        return vals[:n], vals[n:2 * n], vals[2 * n:]

    def verify_epochs(self):
        """Race-detection aid, collective over the ring, to be called at a quiescent point (after a step, stream
        synchronised everywhere): every slot must have seen the same number of fills on every rank (``uses``), every
        fill must have arrived completely and been read completely (``arrive == done == uses * CTAs``).  A rank that
        skipped or repeated a launch, or a producer that signalled a slot it did not fill, shows up here as an
        ``EpochMismatch`` naming the counter, instead of as a wrong gradient later."""
        ctx = self.ctx
        torch.cuda.synchronize()
        if ctx.world > 1:
            dist.barrier(group=ctx.group)         # every rank's last launch (and its signals to us) is complete
        arrive, done, uses = self.counters()
        bad = [f"counter {c}: arrive {arrive[c]}, done {done[c]}, uses {uses[c]} x {self.ctas} CTAs"
               for c in range(len(uses)) if ctx.world > 1 and (arrive[c] != uses[c] * self.ctas or done[c] != uses[c] * self.ctas)]
        if ctx.world > 1:
            gathered = [None] * ctx.world
            dist.all_gather_object(gathered, uses, group=ctx.group)
            for r, u in enumerate(gathered):
                bad += [f"counter {c}: {uses[c]} fills on rank {ctx.rank}, {u[c]} on rank {r}"
                        for c in range(len(uses)) if u[c] != uses[c]]
        if bad:
            raise EpochMismatch("; ".join(bad[:8]))

    def check(self):
        """Read the workspace status word (synchronises the stream); raise if a bounded wait expired."""
        _lib.check(_lib.lib().rtp_ws_status(self.ws_local, C.byref(self._host_status), _lib.stream_ptr()),
                   "rtp_ws_status")
        v = self._host_status.value
        if v:
            _lib.check(_lib.lib().rtp_ws_reset(self.ws_local, _lib.stream_ptr()), "rtp_ws_reset")
            raise _lib.RotationTimeout(_lib.status_text(v))


class EpochMismatch(RuntimeError):
    """The slot counters of a ring disagree at a quiescent point: some rank ran a different sequence of fills."""


def get_engine(ctx: RingContext) -> FusedEngine:
    key = (id(ctx.group), ctx.rank, ctx.world, torch.cuda.current_device())
    eng = _engines.get(key)
    if eng is None:
        eng = FusedEngine(ctx, _reserved_bytes)
        _engines[key] = eng
        if check_all not in _lib._after_launch_hooks:
            _lib._after_launch_hooks.append(check_all)
    elif ctx.world > 1 and _reserved_bytes > eng.slot_bytes:
        eng.grow(_reserved_bytes)
    return eng


def workspace_bytes() -> int:
    """Device bytes held by the peer-mapped workspaces of this process (allocated with cudaMalloc, outside the
    PyTorch caching allocator, so memory statistics of torch do not include them)."""
    L = _lib.lib()
    L.rtp_ws_bytes_world.restype = C.c_ulonglong
    L.rtp_ws_bytes_world.argtypes = [C.c_ulonglong, C.c_int]
    total = 0
    for e in _engines.values():
        total += int(L.rtp_ws_bytes_world(e.slot_bytes if e.ctx.world > 1 else 256, e.ctx.world))
        total += e.staging_bytes()
    return total


def check_all():
    for e in _engines.values():
        e.check()


# --------------------------------------------------------------------------------------------------
# rotated linear on the fused kernels
# --------------------------------------------------------------------------------------------------
def _set_prefetch(op, bank, pushed, next_flat, next_kind):
    """Cross-launch prefetch fields of a linear op: read weight-slot bank ``bank`` (already filled by the previous launch
    if ``pushed``) and push ``next_flat``, the home shard of the next rotated linear on the stream, into the other bank."""
    op.bank, op.no_self_push = int(bank), int(bool(pushed))
    if next_flat is not None:
        op.next_home = next_flat.data_ptr()
        op.next_bytes = _round_up(next_flat.numel() * 2, 16)
        op.next_kind = int(next_kind)


def linear_fwd_raw(eng, flat, layout_info, x2d, row, in_f, out_f, act=0, drop_p=0.0, seed=0, offset=0, out=None,
                   step=None, bank=0, pushed=False, next_flat=None, next_kind=0):
    has_bias, bias_off, shard_bytes = layout_info
    M = x2d.shape[0]
    y = out if out is not None else torch.empty(M, out_f, dtype=torch.bfloat16, device=x2d.device)
    op = _lib.LinearFwd()
    op.mode, op.M, op.in_features, op.out_features = int(row), M, in_f, out_f
    op.home, op.bias_off, op.shard_bytes = flat.data_ptr(), bias_off, shard_bytes
    op.x, op.ldx = x2d.data_ptr(), x2d.stride(0)
    op.y, op.ldy = y.data_ptr(), y.stride(0)
    op.act, op.drop_p, op.seed, op.offset = act, drop_p, seed, offset
    op.step_ptr = step.data_ptr() if step is not None else None
    _set_prefetch(op, bank, pushed, next_flat, next_kind)
    _lib.check(_lib.lib().rtp_linear_fwd(C.byref(eng.ring), C.byref(op), _lib.stream_ptr()), "rtp_linear_fwd")
    return y


def linear_bwd_raw(eng, flat, layout_info, x2d, dy2d, row, in_f, out_f, need_dx=True, mask=None, mask_scale=1.0,
                   grad_out=None, dx_out=None, dx_accumulate=False, dbias_buf=None, bank=0, pushed=False, next_flat=None,
                   next_kind=1):
    has_bias, bias_off, shard_bytes = layout_info
    M = x2d.shape[0]
    gflat = grad_out if grad_out is not None else torch.empty_like(flat)
    dx = None
    if need_dx:
        dx = dx_out if dx_out is not None else torch.empty(M, in_f, dtype=torch.bfloat16, device=x2d.device)
    op = _lib.LinearBwd()
    op.mode, op.M, op.in_features, op.out_features = int(row), M, in_f, out_f
    op.home, op.bias_off, op.shard_bytes = flat.data_ptr(), bias_off, shard_bytes
    op.x, op.ldx = x2d.data_ptr(), x2d.stride(0)
    op.dy, op.ldy = dy2d.data_ptr(), dy2d.stride(0)
    if dx is not None:
        op.dx, op.lddx = dx.data_ptr(), dx.stride(0)
    op.grad_home = gflat.data_ptr()
    if has_bias:
        # On a 1-rank ring the bias gradient is one more GEMM phase of the launch (a row of ones times dy); elsewhere
        # the column sums of dy come from a kernel of their own.
        op.ones = eng.ones_row(M).data_ptr()
        if not _lib.lib().rtp_linear_bwd_folds_bias(C.byref(eng.ring), C.byref(op)):
            op.ones = None
            op.dbias_full = K.colsum(dy2d, dbias_buf).data_ptr()
    if mask is not None:
        op.mask, op.ldmask, op.mask_scale = mask.data_ptr(), mask.stride(0), mask_scale
    op.dx_accumulate = int(dx_accumulate)
    _set_prefetch(op, bank, pushed, next_flat, next_kind)
    _lib.check(_lib.lib().rtp_linear_bwd(C.byref(eng.ring), C.byref(op), _lib.stream_ptr()), "rtp_linear_bwd")
    return dx, gflat


class LinSpec:
    """One rotated linear inside a flat shard buffer: where weight and bias live, the full layer's sizes, and the
    placement (offset, numel, shape) of the registered parameters whose gradients the backward returns.  ``owner`` is
    the rotated module (it carries the ``_displaced`` flag of the in-place mode)."""

    __slots__ = ("ring", "flat", "has_bias", "bias_off", "shard_bytes", "row", "in_f", "out_f", "places", "owner",
                 "inplace", "grad_mode", "recompute")

    def __init__(self, ring, flat, has_bias, bias_off, row, in_f, out_f, places, owner=None, inplace=False):
        self.ring, self.flat, self.has_bias, self.bias_off = ring, flat, has_bias, bias_off
        self.shard_bytes = _round_up(flat.numel() * 2, 16)
        self.row, self.in_f, self.out_f, self.places, self.owner, self.inplace = row, in_f, out_f, places, owner, inplace
        # a spec is built per call, outside autograd.Function.forward (which always runs with grad mode off)
        self.grad_mode = torch.is_grad_enabled()
        # (kind, sources) when the input of this call can be rebuilt in backward instead of being kept (see
        # ops.functional.recompute), else None
        self.recompute = None

    @property
    def info(self):
        return (self.has_bias, self.bias_off, self.shard_bytes)

    @property
    def shard_dims(self):
        """(rows, columns) of one weight shard."""
        N = self.ring.world
        return (self.out_f, self.in_f // N) if self.row else (self.out_f // N, self.in_f)


def fused_linear_ok(row: bool, in_f: int, out_f: int, world: int) -> bool:
    """Every operand of the forward and backward programs must be a legal TMA operand: 16-byte aligned bases, row
    pitches and tile x-offsets, i.e. the full and the per-shard feature counts must be multiples of 8."""
    if in_f % 8 or out_f % 8:
        return False
    return (in_f // world) % 8 == 0 if row else (out_f // world) % 8 == 0


def _as_2d(x):
    x2d = x.reshape(-1, x.shape[-1])
    if x2d.stride(1) != 1 or (x2d.stride(0) * 2) % 16 or x2d.data_ptr() % 16:
        x2d = x2d.contiguous()
    return x2d


def _inplace_linear_fwd(eng, spec, x2d, needs_bwd):
    """Memory-lean forward: the flat buffer itself visits every rank (one in-place hop per step); each step is a plain
    GEMM of the local activations with whichever shard is here (reference: rtp/inplace/module/linear.py:210-229)."""
    from ..ops.gemm import gemm
    ctx = spec.ring
    N, r = ctx.world, ctx.rank
    Os, Ks = spec.shard_dims
    flat = spec.flat
    w = flat[:Os * Ks].view(Os, Ks)
    b = flat[spec.bias_off:spec.bias_off + Os] if spec.has_bias else None
    y = torch.empty(x2d.shape[0], spec.out_f, dtype=torch.bfloat16, device=x2d.device)
    for i in range(N):
        j = (r + i) % N
        if spec.row:
            gemm(x2d[:, j * Ks:(j + 1) * Ks], w, bias=b, c=y if i > 0 else None, out=y)
        else:
            gemm(x2d, w, bias=b, out=y[:, j * Os:(j + 1) * Os])
        if i < N - 1:
            eng.shift_inplace(flat, "down")
    if N > 1:
        if needs_bwd:
            if spec.owner is not None:
                spec.owner._displaced = True     # backward's N-1 reverse hops bring the shards home
        else:
            eng.shift_inplace(flat, "down")      # N-th hop: every shard is home again
    return y


def _inplace_linear_bwd(eng, spec, x2d, dy2d, need_dx):
    """Backward of the in-place mode: weights hop back ("up") and the travelling gradient buffer hops with them,
    picking up this rank's contribution at every stop (reference: rtp/inplace/module/collectives.py:75-105)."""
    from ..ops.gemm import gemm
    ctx = spec.ring
    N, r = ctx.world, ctx.rank
    Os, Ks = spec.shard_dims
    flat = spec.flat
    w = flat[:Os * Ks].view(Os, Ks)
    g = torch.zeros_like(flat)
    gw = g[:Os * Ks].view(Os, Ks)
    gb = g[spec.bias_off:spec.bias_off + Os] if spec.has_bias else None
    M = x2d.shape[0]
    dx = torch.empty(M, spec.in_f, dtype=torch.bfloat16, device=x2d.device) if need_dx else None
    for s in range(N):
        j = (r + N - 1 - s) % N
        if spec.row:
            dy_j, x_j = dy2d, x2d[:, j * Ks:(j + 1) * Ks]
        else:
            dy_j, x_j = dy2d[:, j * Os:(j + 1) * Os], x2d
        if need_dx:
            if spec.row:
                gemm(dy_j, w, b_mn=True, out=dx[:, j * Ks:(j + 1) * Ks])
            else:
                gemm(dy_j, w, b_mn=True, c=dx if s > 0 else None, out=dx)
        gemm(dy_j, x_j, a_mn=True, b_mn=True, c=gw, out=gw)
        if gb is not None:
            gb.add_(K.colsum(dy_j).to(gb.dtype))
        if s < N - 1:
            eng.shift_inplace(flat, "up")
            eng.shift_inplace(g, "up")
    if spec.owner is not None:
        spec.owner._displaced = False
    return dx, g


class _FusedSubLinearFn(torch.autograd.Function):
    """Rotated linear described by a :class:`LinSpec` (a whole module's shard or a sub-range of it)."""

    @staticmethod
    def forward(ctx, spec, x, *params):
        eng = get_engine(spec.ring)
        x2d = _as_2d(x)
        # whether a backward will follow: grad mode at call time (it is always off in here) and an input that wants a gradient
        needs_bwd = spec.grad_mode and any(ctx.needs_input_grad)
        if spec.inplace and spec.ring.world > 1:
            if spec.owner is not None and getattr(spec.owner, "_displaced", False):
                raise RuntimeError("in-place rotated layer called while its shards are displaced: the backward of the "
                                   "previous grad-mode forward has not run yet")
            y = _inplace_linear_fwd(eng, spec, x2d, needs_bwd)
        else:
            y = linear_fwd_raw(eng, spec.flat, spec.info, x2d, spec.row, spec.in_f, spec.out_f)
        ctx.spec, ctx.eng = spec, eng
        # an input that its producer can rebuild is not kept: its sources (which the producer's own backward keeps
        # anyway) are saved instead
        rc = getattr(spec, "recompute", None) if needs_bwd else None
        ctx.rc_kind = None
        if rc is not None:
            kind, srcs = rc
            ctx.rc_kind, ctx.rc_is_tensor = kind, [torch.is_tensor(a) for a in srcs]
            ctx.rc_consts = [a for a in srcs if not torch.is_tensor(a)]
            ctx.save_for_backward(*[a for a in srcs if torch.is_tensor(a)])
        else:
            ctx.save_for_backward(x2d)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], spec.out_f)

    @staticmethod
    def backward(ctx, dy):
        spec = ctx.spec
        if ctx.rc_kind is not None:
            from ..ops import functional as FO
            tensors, consts = list(ctx.saved_tensors), list(ctx.rc_consts)
            srcs = [tensors.pop(0) if is_t else consts.pop(0) for is_t in ctx.rc_is_tensor]
            x2d = _as_2d(FO.recompute(ctx.rc_kind, srcs))
        else:
            (x2d,) = ctx.saved_tensors
        dy2d = _as_2d(dy)
        if spec.inplace and spec.ring.world > 1:
            dx, gflat = _inplace_linear_bwd(ctx.eng, spec, x2d, dy2d, ctx.needs_input_grad[1])
        else:
            dx, gflat = linear_bwd_raw(ctx.eng, spec.flat, spec.info, x2d, dy2d, spec.row, spec.in_f, spec.out_f,
                                       need_dx=ctx.needs_input_grad[1])
        if spec.owner is not None:
            spec.owner._last_flat_grad = gflat
        grads = [gflat[off:off + n].view(shape) for off, n, shape in spec.places]
        return (None, dx.view(ctx.x_shape) if dx is not None else None, *grads)


def linear_spec(owner, row, in_f, out_f, weight, bias):
    """LinSpec of a rotated module whose flat shard is exactly [weight, bias]."""
    lay = owner._layout
    names = lay.names
    places = [(lay.offset_of(names[0]), weight.numel(), weight.shape)]
    has_bias = bias is not None
    if has_bias:
        places.append((lay.offset_of(names[1]), bias.numel(), bias.shape))
    return LinSpec(owner.ring, owner._full_param, has_bias, lay.offset_of(names[1]) if has_bias else -1, row, in_f, out_f,
                   places, owner=owner, inplace=bool(getattr(owner, "inplace", False)))


def fused_linear(module, x, row=False):
    lin = module.linear
    spec = linear_spec(module, row, module.in_features, module.out_features, lin.weight, lin.bias)
    params = [p for p in (lin.weight, lin.bias) if p is not None]
    spec.recompute = getattr(x, "_rtp_recompute", None)
    return _FusedSubLinearFn.apply(spec, x, *params)


# --------------------------------------------------------------------------------------------------
# rotated Conv2d: a column-parallel linear over the patch matrix
# --------------------------------------------------------------------------------------------------
class _FusedConvFn(torch.autograd.Function):
    """Rotated Conv2d on the rotation GEMM kernels (reference: rtp/module/conv.py:103-114; the flat shard
    [Cout/N, Cin*kh*kw] + bias is a linear shard as it is).  When the patch length is not a multiple of 8 (a TMA row
    pitch must be a multiple of 16 bytes) the patch matrix and a shadow copy of the weight shard are zero-padded to the
    next multiple of 8; the shadow is what rotates, and the gradient is cut back to the real columns."""

    @staticmethod
    def forward(ctx, owner, conv, x, *params):
        eng = get_engine(owner.ring)
        x = x.contiguous()
        N = owner.ring.world
        K_ = conv.in_channels * conv.kernel_size[0] * conv.kernel_size[1]
        Kp = _round_up(K_, 8)
        Os = conv.out_channels                      # the shard module holds Cout / N channels
        cols = K.im2col(x, conv.kernel_size, conv.stride, conv.padding, conv.dilation, Kp=Kp)
        has_bias = conv.bias is not None
        if Kp == K_:
            lay = owner._layout
            flat = owner._full_param
            bias_off = lay.offset_of(lay.names[1]) if has_bias else -1
        else:
            bias_off = _round_up(Os * Kp, 64)
            flat = torch.zeros(bias_off + (_round_up(Os, 64) if has_bias else 0), dtype=torch.bfloat16, device=x.device)
            flat[:Os * Kp].view(Os, Kp)[:, :K_].copy_(conv.weight.detach().reshape(Os, K_))
            if has_bias:
                flat[bias_off:bias_off + Os].copy_(conv.bias.detach())
            else:
                bias_off = -1
            reserve_shard_bytes(flat.numel() * 2)
            eng = get_engine(owner.ring)
        places = [(0, Os * Kp, (Os, Kp))] + ([(bias_off, Os, (Os,))] if has_bias else [])
        spec = LinSpec(owner.ring, flat, has_bias, bias_off, False, Kp, Os * N, places)
        y2d = linear_fwd_raw(eng, flat, spec.info, cols, False, Kp, Os * N)
        OH, OW = K.conv_out_size(x.shape[2], x.shape[3], conv.kernel_size, conv.stride, conv.padding, conv.dilation)
        ctx.owner, ctx.conv, ctx.spec, ctx.eng, ctx.K_, ctx.Kp = owner, conv, spec, eng, K_, Kp
        ctx.x_shape = x.shape
        ctx.save_for_backward(cols)
        return y2d.view(x.shape[0], OH, OW, Os * N).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        owner, conv, spec = ctx.owner, ctx.conv, ctx.spec
        (cols,) = ctx.saved_tensors
        Cout = spec.out_f
        dy2d = dy.permute(0, 2, 3, 1).reshape(-1, Cout)
        if not dy2d.is_contiguous():
            dy2d = dy2d.contiguous()
        dcols, gflat = linear_bwd_raw(ctx.eng, spec.flat, spec.info, cols, dy2d, False, ctx.Kp, Cout,
                                      need_dx=ctx.needs_input_grad[2])
        dx = None
        if dcols is not None:
            dx = K.col2im(dcols, ctx.x_shape, conv.kernel_size, conv.stride, conv.padding, conv.dilation)
        Os = Cout // owner.ring.world
        gw = gflat[:Os * ctx.Kp].view(Os, ctx.Kp)[:, :ctx.K_].reshape(conv.weight.shape)
        grads = [gw]
        if spec.has_bias:
            grads.append(gflat[spec.bias_off:spec.bias_off + Os])
        if ctx.Kp == ctx.K_:
            owner._last_flat_grad = gflat
        return (None, None, dx, *grads)


def fused_conv_ok(conv, x) -> bool:
    """Plain convolutions (groups 1, zero padding, numeric padding) whose shard has a multiple of 8 output channels."""
    return (conv.groups == 1 and conv.padding_mode == "zeros" and not isinstance(conv.padding, str) and x.dim() == 4
            and conv.out_channels % 8 == 0)


def fused_conv(owner, conv, x):
    params = [p for p in (conv.weight, conv.bias) if p is not None]
    return _FusedConvFn.apply(owner, conv, x, *params)


# --------------------------------------------------------------------------------------------------
# rotated embedding
# --------------------------------------------------------------------------------------------------
def embed_fwd_rot(eng, flat, V, Ds, ids, out, D, scale, pe, tokens_per_pos, drop_p, seed, offset, step):
    """Rotated embedding lookup (+ scale, positional encoding, dropout) in one launch of the rotation kernel."""
    op = _lib.EmbedFwd()
    op.home, op.shard_bytes = flat.data_ptr(), _round_up(flat.numel() * 2, 16)
    op.V, op.Ds, op.D = V, Ds, D
    op.ids, op.T = ids.data_ptr(), ids.numel()
    op.out, op.ld_out = out.data_ptr(), out.stride(0)
    op.scale = scale
    if pe is not None:
        op.pe, op.ld_pe = pe.data_ptr(), pe.stride(0)
    op.tokens_per_pos = tokens_per_pos
    op.drop_p, op.seed, op.offset = drop_p, seed, offset
    op.step_ptr = step.data_ptr() if step is not None else None
    _lib.check(_lib.lib().rtp_embed_fwd_rot(C.byref(eng.ring), C.byref(op), _lib.stream_ptr()), "rtp_embed_fwd_rot")
    return out


def reduce_scatter_cols(eng, src, out):
    """Ring reduce-scatter of the column blocks of ``src`` [rows, N*cols]; ``out`` [rows, cols] receives the
    sum over ranks of this rank's block."""
    op = _lib.ReduceScatter()
    op.src, op.ld = src.data_ptr(), src.stride(0)
    op.rows, op.cols = out.shape[0], out.shape[1]
    op.out = out.data_ptr()
    _lib.check(_lib.lib().rtp_reduce_scatter_cols(C.byref(eng.ring), C.byref(op), _lib.stream_ptr()),
               "rtp_reduce_scatter_cols")
    return out


def reduce_blocks(eng, blocks, out):
    """One-hop reduce-scatter: ``blocks`` [N, ...] holds this rank's contribution to every owner (block j for owner j,
    contiguous); each block travels straight to its owner and ``out`` receives the sum over ranks of block ``rank``."""
    op = _lib.ReduceBlocks()
    op.src, op.block_elems, op.out = blocks.data_ptr(), blocks[0].numel(), out.data_ptr()
    _lib.check(_lib.lib().rtp_reduce_blocks(C.byref(eng.ring), C.byref(op), _lib.stream_ptr()), "rtp_reduce_blocks")
    return out


def embed_bwd_rot(eng, trainer, st, dx0):
    """Embedding backward on a ring: local scatter-add into a block-major [N, V, D/N] buffer, then every block goes
    straight to the owner of that embedding-dim shard, who adds the N contributions (one hop instead of N-1)."""
    import math
    D, N = trainer.D, trainer.N
    V = trainer.emb.embedding.weight.shape[0]
    blocks = st["emb_dense"]
    blocks.zero_()
    K.embed_bwd_blocks(blocks, st["ids"].view(-1), dx0, scale=math.sqrt(D), drop_p=trainer.p_drop, seed=trainer.seed,
                       offset=1, step=trainer.rng_step)
    reduce_blocks(eng, blocks, trainer.emb._layout.views(trainer.emb_gflat)[0])


class _FusedEmbeddingFn(torch.autograd.Function):
    """``owner``: rotated module whose flat shard is the [V, D/N] table."""

    @staticmethod
    def forward(ctx, owner, D, ids, weight):
        eng = get_engine(owner.ring)
        V, Ds = weight.shape
        flat_ids = ids.reshape(-1).contiguous()
        out = torch.empty(flat_ids.numel(), D, dtype=weight.dtype, device=weight.device)
        if getattr(owner, "inplace", False) and owner.ring.world > 1:
            # memory-lean mode: the table shard itself travels; every stop gathers its column block
            N, r = owner.ring.world, owner.ring.rank
            flat = owner._full_param
            for i in range(N):
                j = (r + i) % N
                K.embed_fwd(flat[:V * Ds].view(V, Ds), flat_ids, out, j * Ds, D=D, scale=1.0)
                eng.shift_inplace(flat, "down")        # N hops in all: the shards end at home (tables need no weights
                #                                        in backward, so nothing stays displaced)
        else:
            embed_fwd_rot(eng, owner._full_param, V, Ds, flat_ids, out, D, 1.0, None, 1, 0.0, 0, 0, None)
        ctx.eng = eng
        ctx.save_for_backward(flat_ids)
        ctx.dims = (V, Ds, D)
        return out.view(*ids.shape, D)

    @staticmethod
    def backward(ctx, dy):
        (flat_ids,) = ctx.saved_tensors
        V, Ds, D = ctx.dims
        dy2 = dy.reshape(-1, D).contiguous()
        N = D // Ds
        blocks = torch.zeros(N, V, Ds, dtype=dy2.dtype, device=dy2.device)
        K.embed_bwd_blocks(blocks, flat_ids, dy2)
        if N == 1:
            return None, None, None, blocks[0]
        g = torch.empty(V, Ds, dtype=dy2.dtype, device=dy2.device)
        reduce_blocks(ctx.eng, blocks, g)
        return None, None, None, g


def fused_embedding(owner, ids, weight=None, D=None):
    weight = weight if weight is not None else owner.embedding.weight
    D = D if D is not None else owner.embedding_dim
    return _FusedEmbeddingFn.apply(owner, D, ids, weight)


# --------------------------------------------------------------------------------------------------
# rotated multi-head attention
# --------------------------------------------------------------------------------------------------
class _SmallAttnPackedFn(torch.autograd.Function):
    """Short-sequence attention (S <= 96, head_dim 64) on the packed projection [S*B, 3*D], tokens ordered s*B + b."""

    @staticmethod
    def forward(ctx, qkv, S, B, H, nshard, causal, drop_p, seed, offset, step=None):
        qkv = qkv.contiguous()
        out = K.attn_small_fwd(qkv, S, B, H, nshard=nshard, causal=causal, drop_p=drop_p, seed=seed, offset=offset,
                               step=step)
        ctx.save_for_backward(qkv)
        ctx.cfg = (S, B, H, nshard, causal, drop_p, seed, offset, step)
        return out

    @staticmethod
    def backward(ctx, dout):
        (qkv,) = ctx.saved_tensors
        S, B, H, nshard, causal, drop_p, seed, offset, step = ctx.cfg
        dqkv = K.attn_small_bwd(qkv, dout.contiguous(), S, B, H, nshard=nshard, causal=causal, drop_p=drop_p, seed=seed,
                                offset=offset, step=step)
        return (dqkv,) + (None,) * 9


_causal_mask_cache = {}


def _is_causal_mask(mask, L):
    """True if ``mask`` is exactly the square subsequent mask (0 on and below the diagonal, -inf / True above).  The
    comparison synchronises, so its result is cached per mask tensor."""
    key = (mask.data_ptr(), tuple(mask.shape), mask.dtype, mask._version)
    hit = _causal_mask_cache.get(key)
    if hit is None:
        if mask.dim() != 2 or tuple(mask.shape) != (L, L):
            hit = False
        else:
            causal = torch.full((L, L), float("-inf"), device=mask.device, dtype=torch.float32).triu_(1)
            hit = bool(torch.equal(mask, causal == float("-inf"))) if mask.dtype == torch.bool else \
                bool(torch.equal(mask.float(), causal))
        if len(_causal_mask_cache) > 64:
            _causal_mask_cache.clear()
        _causal_mask_cache[key] = hit
    return hit


def mha_fused_ok(owner, sub, query, key, value, key_padding_mask, need_weights, attn_mask, training) -> bool:
    """Fused sm_100a path: batched self-attention on bf16 CUDA tensors with a packed in-projection and biases, head_dim
    64 or 128, any 2-D additive / boolean mask, key-padding mask and probability dropout.  Attention weights can be
    returned except under training dropout (the reference returns the dropped probabilities there)."""
    from . import fused
    if not ((key is value) and (query is key) and query.dim() == 3):
        return False
    if not (sub._qkv_same_embed_dim and sub.in_proj_bias is not None and sub.bias_k is None and not sub.add_zero_attn):
        return False
    if need_weights and training and sub.dropout > 0:
        return False
    if not fused.use_fused(query, owner._full_param):
        return False
    if sub.head_dim not in (64, 128):
        return False
    N = owner.ring.world
    if not (fused_linear_ok(False, sub.embed_dim, 3 * sub.embed_dim, N) and fused_linear_ok(True, sub.embed_dim, sub.embed_dim, N)):
        return False
    if attn_mask is not None and attn_mask.dim() != 2:
        return False
    L = query.shape[1] if sub.batch_first else query.shape[0]
    if training and sub.dropout > 0 and L % 4:
        return False
    return True


def fused_mha(owner, sub, x, *, is_causal=False, attn_mask=None, key_padding_mask=None, need_weights=False,
              average_attn_weights=True, training=False):
    """Self-attention of a rotated MHA shard on the fused kernels: column-rotated packed QKV projection, local attention
    over all heads (flash kernels, or the short-sequence kernels), row-rotated output projection.  ``owner`` is the
    rotated module (flat shard [in_proj_weight, in_proj_bias, out_proj.weight, out_proj.bias]), ``sub`` the shard module.
    ``x``: [L, B, E] (or [B, L, E] when ``batch_first``).  Returns (output, weights or None)."""
    from ..ops.flash import flash_attention_packed, next_dropout_offset
    lay, flat = owner._layout, owner._full_param
    N, E, H = owner.ring.world, sub.embed_dim, sub.num_heads
    hd = E // H
    inplace = bool(getattr(owner, "inplace", False))
    o_inw, o_inb = lay.offset_of("in_proj_weight"), lay.offset_of("in_proj_bias")
    o_ow, o_ob = lay.offset_of("out_proj.weight"), lay.offset_of("out_proj.bias")
    bf = sub.batch_first
    B, L = (x.shape[0], x.shape[1]) if bf else (x.shape[1], x.shape[0])
    if inplace and N > 1:
        # the in-place mode moves the whole flat shard: both projections travel together, twice per direction
        spec_qkv = LinSpec(owner.ring, flat, True, o_inb, False, E, 3 * E,
                           [(o_inw, sub.in_proj_weight.numel(), sub.in_proj_weight.shape),
                            (o_inb, sub.in_proj_bias.numel(), sub.in_proj_bias.shape)], owner=owner, inplace=True)
        spec_out = None
    else:
        qkv_flat, out_flat = flat[o_inw:o_ow], flat[o_ow:]
        spec_qkv = LinSpec(owner.ring, qkv_flat, True, o_inb - o_inw, False, E, 3 * E,
                           [(0, sub.in_proj_weight.numel(), sub.in_proj_weight.shape),
                            (o_inb - o_inw, sub.in_proj_bias.numel(), sub.in_proj_bias.shape)])
        spec_out = LinSpec(owner.ring, out_flat, True, o_ob - o_ow, True, E, E,
                           [(0, sub.out_proj.weight.numel(), sub.out_proj.weight.shape),
                            (o_ob - o_ow, sub.out_proj.bias.numel(), sub.out_proj.bias.shape)])
    if spec_out is None:
        return _mha_inplace(owner, sub, x, is_causal, attn_mask, key_padding_mask, training), None
    spec_qkv.recompute = getattr(x, "_rtp_recompute", None)
    qkv = _FusedSubLinearFn.apply(spec_qkv, x, sub.in_proj_weight, sub.in_proj_bias)       # [.., 3E] grouped per shard
    qkv2d = qkv.reshape(-1, 3 * E)
    causal = bool(is_causal) and attn_mask is None
    if attn_mask is not None and _is_causal_mask(attn_mask, L):
        causal, attn_mask = True, None
    p = float(sub.dropout) if training else 0.0
    seed = torch.initial_seed() & 0x7FFFFFFFFFFFFFFF
    offset = next_dropout_offset() if p > 0 else 0
    step = None
    if p > 0:
        from ..ops import rng
        step = rng.step_tensor(x.device)       # fresh masks at every optimizer step, also under CUDA-graph replay
    if hd == 64 and L <= 96 and not bf and attn_mask is None and key_padding_mask is None:
        ctxv = _SmallAttnPackedFn.apply(qkv2d, L, B, H, N, causal, p, seed, offset, step)
    else:
        ctxv = flash_attention_packed(qkv2d, B, L, H, nshard=N, seq_first=not bf, causal=causal, attn_mask=attn_mask,
                                      key_padding_mask=key_padding_mask, dropout_p=p, seed=seed, offset=offset, step=step)
    out = _FusedSubLinearFn.apply(spec_out, ctxv.view(*x.shape[:2], E), sub.out_proj.weight, sub.out_proj.bias)
    weights = None
    if need_weights:
        weights = _last_shard_weights(qkv2d.detach(), B, L, H, hd, N, owner.ring.rank, bf, causal, attn_mask,
                                      key_padding_mask, average_attn_weights)
    return out, weights


def _last_shard_weights(qkv2d, B, L, H, hd, N, rank, batch_first, causal, attn_mask, key_padding_mask, average):
    """Attention probabilities of the heads of the shard that visits last, as the reference returns them
    (rtp/module/attention.py:227-267): [B, L, S] averaged over those heads, or [B, H/N, L, S]."""
    j = (rank + N - 1) % N
    hps = H // N
    E3 = 3 * hps * hd
    blk = qkv2d[:, j * E3:(j + 1) * E3].float()
    t = blk.view(B, L, 3, hps, hd) if batch_first else blk.view(L, B, 3, hps, hd).transpose(0, 1)
    q, k = t[:, :, 0].permute(0, 2, 1, 3), t[:, :, 1].permute(0, 2, 1, 3)           # [B, hps, L, hd]
    s = torch.matmul(q, k.transpose(-1, -2)) * hd ** -0.5
    if causal:
        s = s + torch.full((L, L), float("-inf"), device=s.device).triu_(1)
    if attn_mask is not None:
        s = s.masked_fill(attn_mask, float("-inf")) if attn_mask.dtype == torch.bool else s + attn_mask.float()
    if key_padding_mask is not None:
        s = s.masked_fill(key_padding_mask.bool()[:, None, None, :], float("-inf"))
    w = torch.softmax(s, dim=-1)
    return (w.mean(dim=1) if average else w).to(torch.bfloat16)


class _LocalLinearFn(torch.autograd.Function):
    """y = x w^T + b on the tcgen05 GEMM kernel, single GPU (the building block of the in-place mode, where the shard
    that is currently here is an ordinary local weight)."""

    @staticmethod
    def forward(ctx, x, w, b):
        from ..ops.gemm import gemm
        x2d = _as_2d(x)
        w2 = w if (w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0) else w.contiguous()
        y = gemm(x2d, w2, bias=b.contiguous() if b is not None else None)
        ctx.save_for_backward(x2d, w2)
        ctx.has_bias, ctx.x_shape = b is not None, x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from ..ops.gemm import gemm
        x2d, w2 = ctx.saved_tensors
        dy2d = _as_2d(dy)
        dx = gemm(dy2d, w2, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = gemm(dy2d, x2d, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        db = K.colsum(dy2d).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[2] else None
        return dx, dw, db


def local_linear(x, w, b=None):
    return _LocalLinearFn.apply(x, w, b)


def _mha_inplace(owner, sub, x, is_causal, attn_mask, key_padding_mask, training):
    """In-place mode of the rotated attention: the single flat shard (both projections) travels through the staging
    ring; every stop computes the partial output of the visiting heads with the library's GEMM and attention kernels
    (reference: rtp/inplace/module/attention.py:258-325)."""
    from ..ops.flash import flash_attention_packed, next_dropout_offset
    from .rotated import rotated_apply
    N, E, H = owner.ring.world, sub.embed_dim, sub.num_heads
    hps = H // N
    bf = sub.batch_first
    B, L = (x.shape[0], x.shape[1]) if bf else (x.shape[1], x.shape[0])
    causal = bool(is_causal) and attn_mask is None
    if attn_mask is not None and _is_causal_mask(attn_mask, L):
        causal, attn_mask = True, None
    p = float(sub.dropout) if training else 0.0
    seed = torch.initial_seed() & 0x7FFFFFFFFFFFFFFF
    base = next_dropout_offset() if p > 0 else 0
    for _ in range(N - 1 if p > 0 else 0):
        next_dropout_offset()                       # one offset per visiting shard
    step = None
    if p > 0:
        from ..ops import rng
        step = rng.step_tensor(x.device)
    names = owner._layout.names

    def fn(j, views, xin):
        prm = dict(zip(names, views))
        qkv = local_linear(xin, prm["in_proj_weight"], prm["in_proj_bias"])            # [.., 3E/N] = [q_j | k_j | v_j]
        ctxv = flash_attention_packed(qkv.reshape(-1, 3 * E // N), B, L, hps, nshard=1, seq_first=not bf, causal=causal,
                                      attn_mask=attn_mask, key_padding_mask=key_padding_mask, dropout_p=p, seed=seed,
                                      offset=base + j, step=step)
        return local_linear(ctxv.view(*xin.shape[:2], E // N), prm["out_proj.weight"], prm["out_proj.bias"])

    return rotated_apply(owner.ring, fn, owner.shard_parameters(), owner._full_param, owner._layout, (x,), combine="sum",
                         inplace=True, stochastic=False, owner=owner)


# --------------------------------------------------------------------------------------------------
# rotating experts (one linear of every expert per launch)
# --------------------------------------------------------------------------------------------------
class _FusedExpertLinearFn(torch.autograd.Function):
    """x: [E_total, cap, in] (dispatched tokens, expert-major) -> [E_total, cap, out].  ``spec`` = (ring, flat range,
    n_local, in_f, out_f, expert_stride, bias_off, places) with places = [(offset, numel, shape)] of the given
    parameters inside the flat range (order: e0.weight, e0.bias, e1.weight, ...)."""

    @staticmethod
    def forward(ctx, spec, x, *params):
        ring, flat, L, in_f, out_f, stride, bias_off, places = spec
        eng = get_engine(ring)
        E, cap, _ = x.shape
        x2 = x.reshape(E * cap, in_f).contiguous()
        y = torch.empty(E * cap, out_f, dtype=torch.bfloat16, device=x.device)
        op = _lib.ExpertFwd()
        op.cap, op.n_local, op.in_features, op.out_features = cap, L, in_f, out_f
        op.home, op.expert_stride, op.bias_off = flat.data_ptr(), stride, bias_off
        op.shard_bytes = _round_up(flat.numel() * 2, 16)
        op.x, op.ldx, op.y, op.ldy, op.act = x2.data_ptr(), in_f, y.data_ptr(), out_f, 0
        _lib.check(_lib.lib().rtp_expert_fwd(C.byref(eng.ring), C.byref(op), _lib.stream_ptr()), "rtp_expert_fwd")
        ctx.spec, ctx.eng = spec, eng
        ctx.save_for_backward(x2)
        ctx.dims = (E, cap)
        return y.view(E, cap, out_f)

    @staticmethod
    def backward(ctx, dy):
        ring, flat, L, in_f, out_f, stride, bias_off, places = ctx.spec
        (x2,) = ctx.saved_tensors
        E, cap = ctx.dims
        dy2 = dy.reshape(E * cap, out_f).contiguous()
        need_dx = ctx.needs_input_grad[1]
        dx = torch.empty(E * cap, in_f, dtype=torch.bfloat16, device=dy.device) if need_dx else None
        gflat = torch.empty_like(flat)
        dbias = None
        if bias_off >= 0:
            dbias = torch.empty(E, out_f, dtype=torch.float32, device=dy.device)
            for g in range(E):
                K.colsum(dy2[g * cap:(g + 1) * cap], dbias[g])
        op = _lib.ExpertBwd()
        op.cap, op.n_local, op.in_features, op.out_features = cap, L, in_f, out_f
        op.home, op.expert_stride, op.bias_off = flat.data_ptr(), stride, bias_off
        op.shard_bytes = _round_up(flat.numel() * 2, 16)
        op.x, op.ldx, op.dy, op.ldy = x2.data_ptr(), in_f, dy2.data_ptr(), out_f
        if dx is not None:
            op.dx, op.lddx = dx.data_ptr(), in_f
        op.grad_home = gflat.data_ptr()
        op.dbias_full = dbias.data_ptr() if dbias is not None else None
        _lib.check(_lib.lib().rtp_expert_bwd(C.byref(ctx.eng.ring), C.byref(op), _lib.stream_ptr()), "rtp_expert_bwd")
        grads = [gflat[off:off + n].view(shape) for off, n, shape in places]
        return (None, dx.view(E, cap, in_f) if dx is not None else None, *grads)


def fused_experts(module, dispatched):
    """Both linears of every (rotating) expert on the fused kernels; the activation in between is an elementwise
    kernel.  ``module`` is a ``WeightMOELayer`` whose experts expose ``linear1`` / ``linear2`` / ``activation``."""
    from ..ops import functional as FO
    lay, flat = module._layout, module._full_param
    L = module.num_local_experts
    experts = list(module.experts)

    def spec_for(layer):
        w0 = getattr(experts[0], layer).weight
        out_f, in_f = w0.shape
        off0 = lay.offset_of(f"0.{layer}.weight")
        stride = (lay.offset_of(f"1.{layer}.weight") - off0) if L > 1 else 0
        bias_off = lay.offset_of(f"0.{layer}.bias") - off0
        end = lay.offset_of(f"{L - 1}.{layer}.bias") + ((out_f + 63) // 64) * 64
        rng = flat[off0:end]
        places, params = [], []
        for e in range(L):
            for nm in ("weight", "bias"):
                p = getattr(getattr(experts[e], layer), nm)
                places.append((lay.offset_of(f"{e}.{layer}.{nm}") - off0, p.numel(), p.shape))
                params.append(p)
        return (module.ring, rng, L, in_f, out_f, stride, bias_off, places), params

    s1, p1 = spec_for("linear1")
    s2, p2 = spec_for("linear2")
    h = _FusedExpertLinearFn.apply(s1, dispatched, *p1)
    act = experts[0].activation if hasattr(experts[0], "activation") else None
    if act is None or isinstance(act, torch.nn.GELU) or act is torch.nn.functional.gelu:
        h = FO.gelu(h)
    else:
        h = torch.relu(h)
    return _FusedExpertLinearFn.apply(s2, h, *p2)
