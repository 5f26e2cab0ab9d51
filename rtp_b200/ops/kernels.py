"""ctypes front-ends of the memory-bound sm_100a kernels (norms, cross-entropy, embedding, short-sequence
attention, column sums, Adam). Raw functions on contiguous bf16 CUDA tensors; autograd wrappers live in
``rtp_b200.ops.functional``."""
import ctypes as C

import torch

from . import _lib

_declared = False


class AdamTensor(C.Structure):
    _fields_ = [("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
                ("n", C.c_longlong), ("lr_mult", C.c_float), ("state_fp32", C.c_int)]


def _L():
    global _declared
    L = _lib.lib()
    if not _declared:
        vp, ll, i, f, ull = C.c_void_p, C.c_longlong, C.c_int, C.c_float, C.c_ulonglong
        L.rtp_kernels_last_error.restype = C.c_char_p
        L.rtp_norm_fwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, f, i, f, ull, ull, vp, vp]
        L.rtp_norm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, f, ull, ull, vp, vp, vp]
        L.rtp_cross_entropy.argtypes = [vp, ll, vp, vp, i, i, f, ll, i, vp]
        L.rtp_embed_fwd.argtypes = [vp, vp, vp, ll, i, vp, ll, i, i, i, i, f, f, ull, ull, vp, vp]
        L.rtp_embed_bwd.argtypes = [vp, vp, vp, ll, i, i, i, i, f, f, ull, ull, vp, vp]
        L.rtp_attn_small_fwd.argtypes = [vp, vp, i, i, i, i, i, f, f, ull, ull, vp, vp]
        L.rtp_attn_small_bwd.argtypes = [vp, vp, vp, i, i, i, i, i, f, f, ull, ull, vp, vp]
        L.rtp_set_attn_tc.argtypes = [i]
        L.rtp_set_attn_tc.restype = None
        L.rtp_attn_tc_error.restype = i
        L.rtp_colsum.argtypes = [vp, ll, i, i, vp, vp]
        L.rtp_gate_last_error.restype = C.c_char_p
        L.rtp_top2_gate_fwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, vp]
        L.rtp_top2_gate_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, vp]
        L.rtp_rope.argtypes = [vp, vp, vp, vp, ll, i, i, i, i, i, vp]
        L.rtp_im2col_last_error.restype = C.c_char_p
        L.rtp_im2col.argtypes = [vp, vp] + [i] * 13 + [vp]
        L.rtp_col2im.argtypes = [vp, vp] + [i] * 13 + [vp]
        L.rtp_adam.argtypes = [vp, vp, i, i, vp, f, f, f, f, f, i, f, f, vp, vp]
        L.rtp_add.argtypes = [vp, vp, vp, ll, vp]
        L.rtp_moe_scatter.argtypes = [vp, vp, vp, vp, i, i, ll, vp]
        L.rtp_moe_gather.argtypes = [vp, vp, vp, vp, i, i, vp]
        L.rtp_moe_rowdot.argtypes = [vp, vp, vp, vp, i, i, vp]
        L.rtp_gelu_fwd.argtypes = [vp, vp, ll, vp]
        L.rtp_gelu_bwd.argtypes = [vp, vp, vp, ll, vp]
        L.rtp_swiglu_fwd.argtypes = [vp, vp, ll, vp, ll, i, vp]
        L.rtp_swiglu_bwd.argtypes = [vp, vp, ll, vp, vp, vp, ll, ll, i, vp]
        L.rtp_causal_softmax.argtypes = [vp, ll, i, f, vp]
        L.rtp_causal_softmax_bwd.argtypes = [vp, vp, ll, i, f, vp]
        L.rtp_cast_f32_bf16.argtypes = [vp, vp, ll, f, vp]
        L.rtp_sum_f32.argtypes = [vp, vp, i, f, vp]
        _declared = True
    return L


def _check(rc, what):
    _lib.launches += 1
    if rc != 0:
        msg = _L().rtp_kernels_last_error()
        raise RuntimeError(f"{what} failed: {msg.decode() if msg else rc}")


def _p(t):
    return None if t is None else t.data_ptr()


def norm_fwd(x, sub, gamma, beta, *, eps=1e-5, rms=False, drop_p=0.0, seed=0, offset=0, save_h=True, step=None,
             out=None, h_out=None, mean_out=None, rstd_out=None):
    """h = x + dropout(sub); y = LayerNorm/RMSNorm(h). Returns (y, h, mean, rstd)."""
    M, D = x.shape
    y = out if out is not None else torch.empty_like(x)
    h = h_out if h_out is not None else (torch.empty_like(x) if save_h else None)
    mean = None if rms else (mean_out if mean_out is not None else torch.empty(M, dtype=torch.float32, device=x.device))
    rstd = rstd_out if rstd_out is not None else torch.empty(M, dtype=torch.float32, device=x.device)
    _check(_L().rtp_norm_fwd(_p(x), _p(sub), _p(gamma), _p(beta), _p(h), _p(y), _p(mean), _p(rstd), M, D, eps,
                             int(rms), float(drop_p), seed, offset, _p(step), _lib.stream_ptr()), "norm_fwd")
    return y, h, mean, rstd


def norm_bwd(dy, h, gamma, mean, rstd, *, rms=False, has_beta=True, drop_p=0.0, seed=0, offset=0, want_dsub=True,
             dres=None, step=None, dgamma=None, dbeta=None, dx=None, dsub=None):
    """Returns (dx, dsub, dgamma_fp32, dbeta_fp32)."""
    M, D = dy.shape
    dx = dx if dx is not None else torch.empty_like(dy)
    if dsub is None and want_dsub:
        dsub = torch.empty_like(dy)
    if dgamma is None:  # caller-provided buffers are accumulated into (they must be zeroed by the caller)
        dgamma = torch.zeros(D, dtype=torch.float32, device=dy.device)
    if dbeta is None and has_beta:
        dbeta = torch.zeros(D, dtype=torch.float32, device=dy.device)
    _check(_L().rtp_norm_bwd(_p(dy), _p(h), _p(gamma), _p(mean), _p(rstd), _p(dx), _p(dsub), _p(dgamma), _p(dbeta),
                             M, D, int(rms), float(drop_p), seed, offset, _p(dres), _p(step), _lib.stream_ptr()),
           "norm_bwd")
    return dx, dsub, dgamma, dbeta


def cross_entropy_(logits, target, *, grad_scale=1.0, ignore_index=-100, write_grad=True):
    """Per-row loss (fp32 [M]); overwrites ``logits`` with ``grad_scale * (softmax - onehot)``."""
    M, V = logits.shape
    loss = torch.empty(M, dtype=torch.float32, device=logits.device)
    _check(_L().rtp_cross_entropy(_p(logits), logits.stride(0), _p(target), _p(loss), M, V, float(grad_scale),
                                  int(ignore_index), int(write_grad), _lib.stream_ptr()), "cross_entropy")
    return loss


def cross_entropy_into(logits, target, loss, *, grad_scale=1.0, ignore_index=-100, write_grad=True):
    """Same as :func:`cross_entropy_` but writes the per-row loss into a caller-provided fp32 buffer."""
    M, V = logits.shape
    _check(_L().rtp_cross_entropy(_p(logits), logits.stride(0), _p(target), _p(loss), M, V, float(grad_scale),
                                  int(ignore_index), int(write_grad), _lib.stream_ptr()), "cross_entropy")
    return loss


def cross_entropy_to(logits, target, grad=None, *, grad_scale=1.0, ignore_index=-100):
    """Per-row loss (fp32 [M]) of bf16 ``logits`` [M, V], which are NOT modified; when ``grad`` (bf16 [M, V]) is given it
    receives ``grad_scale * (softmax - onehot)``."""
    M, V = logits.shape
    loss = torch.empty(M, dtype=torch.float32, device=logits.device)
    L = _L()
    L.rtp_cross_entropy_to.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float,
                                       C.c_longlong, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p]
    _check(L.rtp_cross_entropy_to(_p(logits), logits.stride(0), _p(target), _p(loss), M, V, float(grad_scale),
                                  int(ignore_index), int(grad is not None), _p(grad),
                                  grad.stride(0) if grad is not None else 0, _lib.stream_ptr()), "cross_entropy")
    return loss


def embed_fwd(table, ids, out, col_off, *, D, scale=1.0, pe=None, tokens_per_pos=1, drop_p=0.0, seed=0, offset=0,
              step=None):
    T = ids.numel()
    Ds = table.shape[1]
    _check(_L().rtp_embed_fwd(_p(table), _p(ids), _p(pe), pe.stride(0) if pe is not None else 0, tokens_per_pos,
                              _p(out), out.stride(0), col_off, T, Ds, D, float(scale), float(drop_p), seed, offset,
                              _p(step), _lib.stream_ptr()), "embed_fwd")
    return out


def embed_bwd(gtable, ids, dy, col_off, *, D, scale=1.0, drop_p=0.0, seed=0, offset=0, step=None):
    T = ids.numel()
    Ds = gtable.shape[1]
    _check(_L().rtp_embed_bwd(_p(gtable), _p(ids), _p(dy), dy.stride(0), col_off, T, Ds, D, float(scale),
                              float(drop_p), seed, offset, _p(step), _lib.stream_ptr()), "embed_bwd")
    return gtable


def embed_bwd_blocks(gblocks, ids, dy, *, scale=1.0, drop_p=0.0, seed=0, offset=0, step=None):
    """Scatter-add of ``dy`` [T, D] into a zeroed block-major gradient ``gblocks`` [N, V, D / N]: block j is the
    contiguous [V, D / N] contribution to the owner of embedding-dim shard j."""
    N, V, Ds = gblocks.shape
    D = N * Ds
    T = ids.numel()
    L = _L()
    L.rtp_embed_bwd_blocks.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.c_float, C.c_float, C.c_ulonglong, C.c_ulonglong, C.c_void_p, C.c_int, C.c_int,
                                       C.c_void_p]
    _check(L.rtp_embed_bwd_blocks(_p(gblocks), _p(ids), _p(dy), dy.stride(0), 0, T, D, D, float(scale), float(drop_p), seed,
                                  offset, _p(step), Ds, V, _lib.stream_ptr()), "embed_bwd_blocks")
    return gblocks


def attn_small_fwd(qkv, S, B, heads, *, nshard=1, causal=True, drop_p=0.0, seed=0, offset=0, sm_scale=None, step=None,
                   out=None):
    D = heads * 64
    if out is None:
        out = torch.empty(S * B, D, dtype=qkv.dtype, device=qkv.device)
    sc = sm_scale if sm_scale is not None else 64 ** -0.5
    _check(_L().rtp_attn_small_fwd(_p(qkv), _p(out), S, B, heads, nshard, int(causal), sc, float(drop_p), seed, offset,
                                   _p(step), _lib.stream_ptr()), "attn_small_fwd")
    return out


def attn_small_bwd(qkv, dout, S, B, heads, *, nshard=1, causal=True, drop_p=0.0, seed=0, offset=0, sm_scale=None,
                   step=None, out=None):
    dqkv = out if out is not None else torch.empty_like(qkv)
    sc = sm_scale if sm_scale is not None else 64 ** -0.5
    _check(_L().rtp_attn_small_bwd(_p(qkv), _p(dout), _p(dqkv), S, B, heads, nshard, int(causal), sc, float(drop_p),
                                   seed, offset, _p(step), _lib.stream_ptr()), "attn_small_bwd")
    return dqkv


def set_attn_tc(on):
    """Route S = 32 / 64 attention to the tcgen05 kernels (default) or to the scalar kernels (A/B comparison)."""
    _L().rtp_set_attn_tc(int(bool(on)))


def attn_tc_error():
    """1 if a bounded wait inside a tcgen05 attention kernel ran out since the last call (synchronises)."""
    return int(_L().rtp_attn_tc_error())


def colsum(x, out=None):
    M, N = x.shape
    if out is None:
        out = torch.empty(N, dtype=torch.float32, device=x.device)
    _check(_L().rtp_colsum(_p(x), x.stride(0), M, N, _p(out), _lib.stream_ptr()), "colsum")
    return out


def causal_softmax_(scores, S, scale):
    """In-place causal softmax of a stack of [S, S] bf16 score matrices (any garbage above the diagonal is zeroed)."""
    rows = scores.numel() // S
    _check(_L().rtp_causal_softmax(_p(scores), rows, S, float(scale), _lib.stream_ptr()), "causal_softmax")
    return scores


def causal_softmax_bwd_(p, dp, S, scale):
    """dp <- scale * p * (dp - rowsum(p * dp)), zero above the diagonal."""
    rows = p.numel() // S
    _check(_L().rtp_causal_softmax_bwd(_p(p), _p(dp), rows, S, float(scale), _lib.stream_ptr()), "causal_softmax_bwd")
    return dp


def gelu_fwd(x):
    y = torch.empty_like(x)
    _check(_L().rtp_gelu_fwd(_p(x), _p(y), x.numel(), _lib.stream_ptr()), "gelu_fwd")
    return y


def gelu_bwd(x, dy):
    dx = torch.empty_like(x)
    _check(_L().rtp_gelu_bwd(_p(x), _p(dy), _p(dx), x.numel(), _lib.stream_ptr()), "gelu_bwd")
    return dx


def swiglu_fwd(g, u):
    """g, u: [rows, cols] views with a common row pitch (e.g. the two halves of a packed projection)."""
    rows, cols = g.shape
    y = torch.empty(rows, cols, dtype=g.dtype, device=g.device)
    _check(_L().rtp_swiglu_fwd(_p(g), _p(u), g.stride(0), _p(y), rows, cols, _lib.stream_ptr()), "swiglu_fwd")
    return y


def swiglu_bwd(g, u, dy):
    rows, cols = g.shape
    dg, du = torch.empty(rows, cols, dtype=g.dtype, device=g.device), torch.empty(rows, cols, dtype=g.dtype, device=g.device)
    _check(_L().rtp_swiglu_bwd(_p(g), _p(u), g.stride(0), _p(dy), _p(dg), _p(du), cols, rows, cols, _lib.stream_ptr()),
           "swiglu_bwd")
    return dg, du


def moe_scatter(src, slot, scale, dst_rows):
    """dst[slot[s, k]] = scale[s, k] * src[s] (rows without a token stay zero). slot: int32 [S, 2], -1 = dropped."""
    S, M = src.shape
    dst = torch.empty(dst_rows, M, dtype=src.dtype, device=src.device)
    _check(_L().rtp_moe_scatter(_p(src), _p(slot), _p(scale), _p(dst), S, M, dst_rows, _lib.stream_ptr()), "moe_scatter")
    return dst


def moe_gather(src, slot, scale):
    """dst[s] = sum_k scale[s, k] * src[slot[s, k]]."""
    S, M = slot.shape[0], src.shape[1]
    dst = torch.empty(S, M, dtype=src.dtype, device=src.device)
    _check(_L().rtp_moe_gather(_p(src), _p(slot), _p(scale), _p(dst), S, M, _lib.stream_ptr()), "moe_gather")
    return dst


def moe_rowdot(a, b, slot):
    S, M = a.shape
    out = torch.empty(S, 2, dtype=torch.float32, device=a.device)
    _check(_L().rtp_moe_rowdot(_p(a), _p(b), _p(slot), _p(out), S, M, _lib.stream_ptr()), "moe_rowdot")
    return out


def add(a, b, out=None):
    if out is None:
        out = torch.empty_like(a)
    _check(_L().rtp_add(_p(a), _p(b), _p(out), a.numel(), _lib.stream_ptr()), "add")
    return out


def cast_f32_bf16(src, dst, scale=1.0):
    _check(_L().rtp_cast_f32_bf16(_p(src), _p(dst), src.numel(), float(scale), _lib.stream_ptr()), "cast")
    return dst


def sum_f32(src, out, scale=1.0):
    _check(_L().rtp_sum_f32(_p(src), _p(out), src.numel(), float(scale), _lib.stream_ptr()), "sum")
    return out


def adam_state_dtypes(state_dtype):
    """(dtype of exp_avg, dtype of exp_avg_sq) for a state policy: ``"fp32"`` / ``torch.float32`` (default of the
    optimizers), ``"mixed"`` (first moment bf16, second moment fp32) or ``"bf16"`` / ``torch.bfloat16``.

    A bf16 second moment cannot follow beta2 = 0.999: its 0.1 % decay per step is below half a bf16 ulp (0.2-0.4 %),
    so the stored value rounds back and never shrinks.  The first moment decays by 10 % per step and is safe in bf16."""
    if state_dtype in (None, "fp32", torch.float32):
        return torch.float32, torch.float32
    if state_dtype == "mixed":
        return torch.bfloat16, torch.float32
    if state_dtype in ("bf16", torch.bfloat16):
        return torch.bfloat16, torch.bfloat16
    raise ValueError(f"unknown Adam state dtype {state_dtype!r}")


class AdamPlan:
    """Device-resident descriptor table for the multi-tensor Adam kernel (built once, reused every step)."""

    BLOCK_ELEMS = 4096     # kAdamGroups * 2048 of the kernel

    def __init__(self, entries, device):
        # entries: list of (p, g, m, v, lr_mult)
        arr = (AdamTensor * len(entries))()
        starts = []
        total = 0
        self.keep = entries
        for k, (p, g, m, v, lr_mult) in enumerate(entries):
            arr[k].p, arr[k].g, arr[k].m, arr[k].v = p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr()
            # kernel codes: 0 = both moments bf16, 1 = both fp32, 2 = first moment bf16 + second moment fp32
            if m.dtype == torch.float32 and v.dtype == torch.float32:
                code = 1
            elif m.dtype == torch.bfloat16 and v.dtype == torch.float32:
                code = 2
            elif m.dtype == torch.bfloat16 and v.dtype == torch.bfloat16:
                code = 0
            else:
                raise ValueError(f"unsupported Adam state dtypes {m.dtype} / {v.dtype}")
            arr[k].n, arr[k].lr_mult, arr[k].state_fp32 = p.numel(), float(lr_mult), code
            starts.append(total)
            total += (p.numel() + self.BLOCK_ELEMS - 1) // self.BLOCK_ELEMS
        raw = bytes(arr)
        self.table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        self.starts = torch.tensor(starts, dtype=torch.int32, device=device)
        self.n = len(entries)
        self.total_blocks = total
        # tensor index of every block: one load instead of a binary search at the start of each (short-lived) block
        counts = torch.tensor(starts[1:] + [total], dtype=torch.int64) - torch.tensor(starts, dtype=torch.int64)
        self.block_tensor = torch.repeat_interleave(torch.arange(len(entries), dtype=torch.int32), counts).to(device)

    def step(self, step_dev, lr, beta1, beta2, eps, weight_decay=0.0, adamw=False, clip_value=0.0, grad_scale=1.0):
        _check(_L().rtp_adam(_p(self.table), _p(self.starts), self.n, self.total_blocks, _p(step_dev), lr, beta1,
                             beta2, eps, weight_decay, int(adamw), clip_value, grad_scale, _p(self.block_tensor),
                             _lib.stream_ptr()), "adam")


def _gate_check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: {_L().rtp_gate_last_error().decode()}")


class _Top2Gate(torch.autograd.Function):
    """Fused top-2 routing on [S, E] logits (reference: rtp/module/top2gate.py:43-105), index form."""

    @staticmethod
    def forward(ctx, logits, noise, capacity):
        S, E = logits.shape
        lg = logits.detach().float().contiguous()
        nz = noise.detach().float().contiguous() if noise is not None else None
        dev = lg.device
        gates = torch.empty(S, E, dtype=torch.float32, device=dev)
        idx = torch.empty(S, 2, dtype=torch.int32, device=dev)
        loc = torch.empty(S, 2, dtype=torch.int32, device=dev)
        gate_w = torch.empty(S, 2, dtype=torch.float32, device=dev)
        valid = torch.empty(S, 2, dtype=torch.uint8, device=dev)
        me_sum = torch.empty(E, dtype=torch.float32, device=dev)
        ce = torch.empty(E, dtype=torch.float32, device=dev)
        l_aux = torch.empty((), dtype=torch.float32, device=dev)
        _gate_check(_L().rtp_top2_gate_fwd(_p(lg), _p(nz), _p(gates), _p(idx), _p(loc), _p(gate_w), _p(valid), _p(me_sum),
                                           _p(ce), _p(l_aux), S, E, int(capacity), _lib.stream_ptr()), "top2_gate_fwd")
        ctx.save_for_backward(gates, idx, valid, ce)
        ctx.in_dtype = logits.dtype
        ctx.mark_non_differentiable(idx, loc, valid)
        return l_aux, idx, loc, gate_w, valid

    @staticmethod
    def backward(ctx, d_l_aux, _di, _dl, d_gate_w, _dv):
        gates, idx, valid, ce = ctx.saved_tensors
        S, E = gates.shape
        dlogits = torch.empty_like(gates)
        dg = d_gate_w.float().contiguous() if d_gate_w is not None else torch.zeros(S, 2, device=gates.device)
        dl = d_l_aux.float().contiguous() if d_l_aux is not None else None
        _gate_check(_L().rtp_top2_gate_bwd(_p(gates), _p(idx), _p(valid), _p(ce), _p(dg), _p(dl), _p(dlogits), S, E,
                                           _lib.stream_ptr()), "top2_gate_bwd")
        return dlogits.to(ctx.in_dtype), None, None


def top2_gate(logits, capacity, noise=None):
    """Returns (l_aux, idx[S,2] int32, loc[S,2] int32, gate[S,2] fp32, valid[S,2] uint8); differentiable in `logits`
    through `gate` and `l_aux`.  `noise` is added to the logits for the second choice (None: no noise)."""
    return _Top2Gate.apply(logits, noise, capacity)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, inner):
        x = x.contiguous()
        H, hd = x.shape[-2], x.shape[-1]
        T = x.numel() // (H * hd)
        y = torch.empty_like(x)
        cos = cos.float().contiguous()
        sin = sin.float().contiguous()
        _gate_check(_L().rtp_rope(_p(x), _p(y), _p(cos), _p(sin), T, H, hd, cos.shape[0], int(inner), 0,
                                  _lib.stream_ptr()), "rope")
        ctx.save_for_backward(cos, sin)
        ctx.inner = int(inner)
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        dy = dy.contiguous()
        H, hd = dy.shape[-2], dy.shape[-1]
        T = dy.numel() // (H * hd)
        dx = torch.empty_like(dy)
        _gate_check(_L().rtp_rope(_p(dy), _p(dx), _p(cos), _p(sin), T, H, hd, cos.shape[0], ctx.inner, 1,
                                  _lib.stream_ptr()), "rope backward")
        return dx, None, None, None


def rope(x, cos, sin, inner=1):
    """Rotary position embedding of bf16 `x` [..., H, hd] whose flattened leading dims are tokens; token t sits at
    position (t // inner) % S, with cos / sin of shape [S, hd / 2] (pairs (x[2i], x[2i+1]) rotate together)."""
    return _Rope.apply(x, cos, sin, inner)


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def conv_out_size(H, W, kernel, stride, padding, dilation):
    (KH, KW), (sh, sw), (ph, pw), (dh, dw) = _pair(kernel), _pair(stride), _pair(padding), _pair(dilation)
    return (H + 2 * ph - dh * (KH - 1) - 1) // sh + 1, (W + 2 * pw - dw * (KW - 1) - 1) // sw + 1


def im2col(x, kernel, stride=1, padding=0, dilation=1, Kp=None):
    """Patch matrix [B*OH*OW, Kp] of a contiguous NCHW bf16 tensor; column (c, kh, kw), zero padded up to Kp."""
    B, Cc, H, W = x.shape
    (KH, KW), (sh, sw), (ph, pw), (dh, dw) = _pair(kernel), _pair(stride), _pair(padding), _pair(dilation)
    OH, OW = conv_out_size(H, W, kernel, stride, padding, dilation)
    Kp = Kp or Cc * KH * KW
    cols = torch.empty(B * OH * OW, Kp, dtype=x.dtype, device=x.device)
    rc = _L().rtp_im2col(_p(x), _p(cols), B, Cc, H, W, KH, KW, sh, sw, ph, pw, dh, dw, Kp, _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError("im2col: " + _L().rtp_im2col_last_error().decode())
    return cols


def col2im(dcols, x_shape, kernel, stride=1, padding=0, dilation=1):
    """Adjoint of im2col: gradient with respect to the NCHW input."""
    B, Cc, H, W = x_shape
    (KH, KW), (sh, sw), (ph, pw), (dh, dw) = _pair(kernel), _pair(stride), _pair(padding), _pair(dilation)
    dx = torch.empty(B, Cc, H, W, dtype=dcols.dtype, device=dcols.device)
    rc = _L().rtp_col2im(_p(dcols), _p(dx), B, Cc, H, W, KH, KW, sh, sw, ph, pw, dh, dw, dcols.shape[1],
                         _lib.stream_ptr())
    if rc != 0:
        raise RuntimeError("col2im: " + _L().rtp_im2col_last_error().decode())
    return dx
