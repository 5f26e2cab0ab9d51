"""Fused rotation engine: peer-mapped workspace + launch of the sm_100a rotation kernels.

One engine exists per (process, ring).  It owns a ``cudaMalloc``'d workspace — flag block, two weight
slots and two travelling-gradient slots — whose CUDA-IPC handle is exchanged once over the ring's
process group; afterwards every kernel launch only passes raw pointers.  The kernels themselves push
weight shards from their owner's home buffer into the consumer's slot with NVLink P2P stores and
synchronise through monotonically increasing counters (see csrc/gemm_kernel.cuh), so there is no NCCL
send/recv, no copy kernel and no host involvement between rotation steps.
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

    def check(self):
        """Read the workspace status word (synchronises the stream); raise if a bounded wait expired."""
        _lib.check(_lib.lib().rtp_ws_status(self.ws_local, C.byref(self._host_status), _lib.stream_ptr()),
                   "rtp_ws_status")
        v = self._host_status.value
        if v:
            _lib.check(_lib.lib().rtp_ws_reset(self.ws_local, _lib.stream_ptr()), "rtp_ws_reset")
            raise _lib.RotationTimeout(_lib.STATUS_NAMES.get(v, f"status {v}"))


def get_engine(ctx: RingContext) -> FusedEngine:
    key = (id(ctx.group), ctx.rank, ctx.world, torch.cuda.current_device())
    eng = _engines.get(key)
    if eng is None:
        eng = FusedEngine(ctx, _reserved_bytes)
        _engines[key] = eng
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
    return total


def check_all():
    for e in _engines.values():
        e.check()


# --------------------------------------------------------------------------------------------------
# rotated linear on the fused kernels
# --------------------------------------------------------------------------------------------------
def _linear_desc(module, row):
    lay = module._layout
    has_bias = module.linear.bias is not None
    bias_off = lay.offset_of("bias") if has_bias else -1
    shard_bytes = _round_up(lay.numel * 2, 16)
    return has_bias, bias_off, shard_bytes


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
    dbias = K.colsum(dy2d, dbias_buf) if has_bias else None
    op = _lib.LinearBwd()
    op.mode, op.M, op.in_features, op.out_features = int(row), M, in_f, out_f
    op.home, op.bias_off, op.shard_bytes = flat.data_ptr(), bias_off, shard_bytes
    op.x, op.ldx = x2d.data_ptr(), x2d.stride(0)
    op.dy, op.ldy = dy2d.data_ptr(), dy2d.stride(0)
    if dx is not None:
        op.dx, op.lddx = dx.data_ptr(), dx.stride(0)
    op.grad_home = gflat.data_ptr()
    op.dbias_full = dbias.data_ptr() if dbias is not None else None
    if mask is not None:
        op.mask, op.ldmask, op.mask_scale = mask.data_ptr(), mask.stride(0), mask_scale
    op.dx_accumulate = int(dx_accumulate)
    _set_prefetch(op, bank, pushed, next_flat, next_kind)
    _lib.check(_lib.lib().rtp_linear_bwd(C.byref(eng.ring), C.byref(op), _lib.stream_ptr()), "rtp_linear_bwd")
    return dx, gflat


class _FusedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, module, row, x, *params):
        eng = get_engine(module.ring)
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.stride(1) != 1 or (x2d.stride(0) * 2) % 16:
            x2d = x2d.contiguous()
        info = _linear_desc(module, row)
        y = linear_fwd_raw(eng, module._full_param, info, x2d, row, module.in_features, module.out_features)
        ctx.module, ctx.row, ctx.info, ctx.eng = module, row, info, eng
        ctx.save_for_backward(x2d)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], module.out_features)

    @staticmethod
    def backward(ctx, dy):
        module = ctx.module
        (x2d,) = ctx.saved_tensors
        dy2d = dy.reshape(-1, dy.shape[-1])
        if not dy2d.is_contiguous():
            dy2d = dy2d.contiguous()
        dx, gflat = linear_bwd_raw(ctx.eng, module._full_param, ctx.info, x2d, dy2d, ctx.row, module.in_features,
                                   module.out_features, need_dx=ctx.needs_input_grad[2])
        module._last_flat_grad = gflat
        views = module._layout.views(gflat)
        return (None, None, dx.view(ctx.x_shape) if dx is not None else None, *views)


class _FusedConvFn(torch.autograd.Function):
    """Rotated Conv2d on the rotation GEMM kernels: a column-parallel linear over the patch matrix of the input
    (reference: rtp/module/conv.py:103-114; the flat shard [Cout/N, Cin*kh*kw] + bias is a linear shard as it is)."""

    @staticmethod
    def forward(ctx, module, x, *params):
        eng = get_engine(module.ring)
        conv = module.conv
        x = x.contiguous()
        K_ = conv.in_channels * conv.kernel_size[0] * conv.kernel_size[1]
        cols = K.im2col(x, conv.kernel_size, conv.stride, conv.padding, conv.dilation)
        lay = module._layout
        has_bias = conv.bias is not None
        info = (has_bias, lay.offset_of("bias") if has_bias else -1, _round_up(lay.numel * 2, 16))
        y2d = linear_fwd_raw(eng, module._full_param, info, cols, False, K_, module.out_channels)
        OH, OW = K.conv_out_size(x.shape[2], x.shape[3], conv.kernel_size, conv.stride, conv.padding, conv.dilation)
        ctx.module, ctx.info, ctx.eng, ctx.K_ = module, info, eng, K_
        ctx.x_shape = x.shape
        ctx.save_for_backward(cols)
        return y2d.view(x.shape[0], OH, OW, module.out_channels).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        module, conv = ctx.module, ctx.module.conv
        (cols,) = ctx.saved_tensors
        dy2d = dy.permute(0, 2, 3, 1).reshape(-1, module.out_channels)
        if not dy2d.is_contiguous():
            dy2d = dy2d.contiguous()
        dcols, gflat = linear_bwd_raw(ctx.eng, module._full_param, ctx.info, cols, dy2d, False, ctx.K_,
                                      module.out_channels, need_dx=ctx.needs_input_grad[1])
        module._last_flat_grad = gflat
        dx = None
        if dcols is not None:
            dx = K.col2im(dcols, ctx.x_shape, conv.kernel_size, conv.stride, conv.padding, conv.dilation)
        return (None, dx, *module._layout.views(gflat))


def fused_conv_ok(module, x) -> bool:
    """The patch matrix must be a legal TMA operand (row pitch a multiple of 16 bytes) and the convolution plain."""
    conv = module.conv
    K_ = conv.in_channels * conv.kernel_size[0] * conv.kernel_size[1]
    return (K_ % 8 == 0 and conv.groups == 1 and conv.padding_mode == "zeros" and not isinstance(conv.padding, str)
            and x.dim() == 4)


def fused_conv(module, x):
    return _FusedConvFn.apply(module, x, *module.shard_parameters())


def fused_linear(module, x, row=False):
    return _FusedLinearFn.apply(module, row, x, *module.shard_parameters())


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


def embed_bwd_rot(eng, trainer, st, dx0):
    """Embedding backward on a ring: dense local scatter-add into a [V, D] buffer, then a ring reduce-scatter
    over the embedding-dim blocks delivers each owner the summed gradient of its [V, D/N] shard."""
    import math
    D = trainer.D
    V = trainer.emb.embedding.weight.shape[0]
    dense = st.get("emb_dense")
    if dense is None:
        dense = torch.empty(V, D, dtype=torch.bfloat16, device=dx0.device)
        st["emb_dense"] = dense
    dense.zero_()
    K.embed_bwd(dense, st["ids"].view(-1), dx0, 0, D=D, scale=math.sqrt(D), drop_p=trainer.p_drop,
                seed=trainer.seed, offset=1, step=trainer.rng_step)
    reduce_scatter_cols(eng, dense, trainer.emb._layout.views(trainer.emb_gflat)[0])


# --------------------------------------------------------------------------------------------------
# generic autograd pieces for the module path
# --------------------------------------------------------------------------------------------------
class _FusedSubLinearFn(torch.autograd.Function):
    """Rotated linear on a (sub-)range of a module's flat shard: ``spec`` = (ring, flat, info, row, in_f, out_f,
    [(offset, numel, shape), ...]) lists where the given parameters live inside ``flat``."""

    @staticmethod
    def forward(ctx, spec, x, *params):
        ring, flat, info, row, in_f, out_f, places = spec
        eng = get_engine(ring)
        x2d = x.reshape(-1, x.shape[-1])
        if x2d.stride(1) != 1 or (x2d.stride(0) * 2) % 16 or x2d.data_ptr() % 16:
            x2d = x2d.contiguous()
        y = linear_fwd_raw(eng, flat, info, x2d, row, in_f, out_f)
        ctx.spec, ctx.eng = spec, eng
        ctx.save_for_backward(x2d)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], out_f)

    @staticmethod
    def backward(ctx, dy):
        ring, flat, info, row, in_f, out_f, places = ctx.spec
        (x2d,) = ctx.saved_tensors
        dy2d = dy.reshape(-1, dy.shape[-1])
        if not dy2d.is_contiguous():
            dy2d = dy2d.contiguous()
        dx, gflat = linear_bwd_raw(ctx.eng, flat, info, x2d, dy2d, row, in_f, out_f, need_dx=ctx.needs_input_grad[1])
        grads = [gflat[off:off + n].view(shape) for off, n, shape in places]
        return (None, dx.view(ctx.x_shape) if dx is not None else None, *grads)


def fused_mha(module, x, causal: bool):
    """Self-attention of a ``ParallelMultiheadAttention`` on the fused kernels: column-rotated packed QKV projection,
    local attention over all heads, row-rotated output projection.  ``x``: [L, B, E] (or [B, L, E] when batch_first)."""
    from ..ops import functional as FO
    from ..ops.flash import flash_attention, flash_attention_available
    from ..ops import kernels as KK
    sub = module.MultiheadAttention
    lay, flat = module._layout, module._full_param
    N, E, H = module.world_size, module.embed_dim, module.num_heads
    hd = E // H
    o_inw, o_inb = lay.offset_of("in_proj_weight"), lay.offset_of("in_proj_bias")
    o_ow, o_ob = lay.offset_of("out_proj.weight"), lay.offset_of("out_proj.bias")
    qkv_flat, out_flat = flat[o_inw:o_ow], flat[o_ow:]
    spec_qkv = (module.ring, qkv_flat, (True, o_inb - o_inw, _round_up(qkv_flat.numel() * 2, 16)), False, E, 3 * E,
                [(0, sub.in_proj_weight.numel(), sub.in_proj_weight.shape),
                 (o_inb - o_inw, sub.in_proj_bias.numel(), sub.in_proj_bias.shape)])
    spec_out = (module.ring, out_flat, (True, o_ob - o_ow, _round_up(out_flat.numel() * 2, 16)), True, E, E,
                [(0, sub.out_proj.weight.numel(), sub.out_proj.weight.shape),
                 (o_ob - o_ow, sub.out_proj.bias.numel(), sub.out_proj.bias.shape)])
    bf = module.batch_first
    if bf:
        B, L = x.shape[0], x.shape[1]
    else:
        L, B = x.shape[0], x.shape[1]
    qkv = _FusedSubLinearFn.apply(spec_qkv, x, sub.in_proj_weight, sub.in_proj_bias)       # [.., 3E] grouped per shard
    packed = qkv.reshape(*x.shape[:2], N, 3, H // N, hd)
    q, k, v = [packed[:, :, :, i].reshape(*x.shape[:2], H, hd) for i in range(3)]
    if not bf:
        q, k, v = [t.transpose(0, 1) for t in (q, k, v)]                                    # [B, L, H, hd]
    ctxv = FO.causal_attention(q, k, v)                                                       # [B, L, H, hd]
    if not bf:
        ctxv = ctxv.transpose(0, 1)
    ctxv = ctxv.reshape(*x.shape[:2], E)
    return _FusedSubLinearFn.apply(spec_out, ctxv, sub.out_proj.weight, sub.out_proj.bias)


class _FusedEmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, module, ids, weight):
        eng = get_engine(module.ring)
        V, Ds = weight.shape
        D = module.embedding_dim
        flat_ids = ids.reshape(-1).contiguous()
        out = torch.empty(flat_ids.numel(), D, dtype=weight.dtype, device=weight.device)
        embed_fwd_rot(eng, module._full_param, V, Ds, flat_ids, out, D, 1.0, None, 1, 0.0, 0, 0, None)
        ctx.module, ctx.eng = module, eng
        ctx.save_for_backward(flat_ids)
        ctx.dims = (V, Ds, D)
        return out.view(*ids.shape, D)

    @staticmethod
    def backward(ctx, dy):
        (flat_ids,) = ctx.saved_tensors
        V, Ds, D = ctx.dims
        dy2 = dy.reshape(-1, D).contiguous()
        dense = torch.zeros(V, D, dtype=dy2.dtype, device=dy2.device)
        K.embed_bwd(dense, flat_ids, dy2, 0, D=D, scale=1.0)
        g = torch.empty(V, Ds, dtype=dy2.dtype, device=dy2.device)
        reduce_scatter_cols(ctx.eng, dense, g)
        return None, None, g


def fused_embedding(module, ids):
    return _FusedEmbeddingFn.apply(module, ids, module.embedding.weight)


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
