"""Autograd front-ends of the sm_100a kernels for models written against the module API.

``use_kernels(x)`` is true for bf16 CUDA tensors unless the functional backend was requested; every function
below has a plain PyTorch evaluation for CPU / fp32 tensors so that the same model code runs on gloo."""
import torch
import torch.nn.functional as F

from ..parallel.context import get_backend


def use_kernels(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and get_backend() != "functional"


# ---------------------------------------------------------------------------------------------------------------------
# Recomputed activations.  The output of a cheap elementwise / normalisation op is usually consumed by a rotated linear,
# which would save it for its weight gradient although the op's own backward already keeps the op's INPUT.  Such outputs
# are tagged with how to rebuild them; a fused linear that receives a tagged tensor saves the (already saved) sources
# instead and rebuilds its input in backward, so the output lives only between the two forward launches.  For a GPT
# block this removes the [tokens, 4 d_model] GELU output and both LayerNorm outputs from the saved set (6 of 17
# d_model-sized rows per token and layer) for one extra elementwise pass each in backward.
# ---------------------------------------------------------------------------------------------------------------------
_RECOMPUTE = True


def set_activation_recompute(on: bool) -> bool:
    """Turns the tagging on or off (default on); returns the previous setting."""
    global _RECOMPUTE
    old, _RECOMPUTE = _RECOMPUTE, bool(on)
    return old


def _tag(out: torch.Tensor, kind: str, *srcs):
    if _RECOMPUTE and torch.is_grad_enabled():
        out._rtp_recompute = (kind, srcs)
    return out


def recompute_tag(x: torch.Tensor):
    """The (kind, sources) tag of a tensor produced by one of the ops below, or None."""
    return getattr(x, "_rtp_recompute", None)


def recompute(kind: str, srcs):
    """Rebuilds a tagged tensor from its sources."""
    from . import kernels as K
    if kind == "gelu":
        return K.gelu_fwd(srcs[0])
    if kind == "swiglu":
        g, u = srcs
        return K.swiglu_fwd(g.reshape(-1, g.shape[-1]), u.reshape(-1, u.shape[-1])).view(g.shape)
    if kind == "norm":
        x, weight, bias, eps, rms = srcs
        y = K.norm_fwd(x.reshape(-1, x.shape[-1]), None, weight, bias, eps=eps, rms=rms, save_h=False)[0]
        return y.view(x.shape)
    raise ValueError(f"unknown recompute kind {kind!r}")


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        from . import kernels as K
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y, h, mean, rstd = K.norm_fwd(x2, None, weight, bias, eps=eps, rms=rms, save_h=False)
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.rms, ctx.has_bias, ctx.shape = rms, bias is not None, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        from . import kernels as K
        x2, weight, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx, _, dg, db = K.norm_bwd(dy2, x2, weight, mean, rstd, rms=ctx.rms, has_beta=ctx.has_bias, want_dsub=False)
        return dx.view(ctx.shape), dg.to(weight.dtype), (db.to(weight.dtype) if ctx.has_bias else None), None, None


def layer_norm(x, weight, bias, eps=1e-5):
    if use_kernels(x) and x.shape[-1] % 8 == 0:
        y = _NormFn.apply(x, weight, bias, eps, False)
        return _tag(y, "norm", x, weight, bias, eps, False) if x.is_contiguous() else y
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def rms_norm(x, weight, eps=1e-5):
    if use_kernels(x) and x.shape[-1] % 8 == 0:
        y = _NormFn.apply(x, weight, None, eps, True)
        return _tag(y, "norm", x, weight, None, eps, True) if x.is_contiguous() else y
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


class _CrossEntropyFn(torch.autograd.Function):
    """Mean token cross-entropy of bf16 logits.  The input is never modified: the softmax gradient, produced in the same
    pass over the logits, goes to a buffer of its own, and only when the logits need a gradient."""

    @staticmethod
    def forward(ctx, logits, target, ignore_index):
        from . import kernels as K
        lg = logits.reshape(-1, logits.shape[-1])
        if lg.stride(1) != 1 or lg.stride(0) % 8:
            lg = lg.contiguous()
        t = target.reshape(-1)
        n = (t != ignore_index).sum().clamp(min=1)
        grad = torch.empty(lg.shape, dtype=lg.dtype, device=lg.device) if ctx.needs_input_grad[0] else None
        rows = K.cross_entropy_to(lg, t, grad, grad_scale=1.0, ignore_index=ignore_index)
        ctx.save_for_backward(grad, n)
        ctx.shape = logits.shape
        return rows.sum() / n

    @staticmethod
    def backward(ctx, g):
        grad, n = ctx.saved_tensors
        return grad.mul_((g / n).to(grad.dtype)).view(ctx.shape), None, None


def cross_entropy(logits, target, ignore_index=-100):
    """Mean token cross-entropy; the softmax gradient is produced in the same pass over the logits."""
    if use_kernels(logits) and logits.shape[-1] % 8 == 0:
        return _CrossEntropyFn.apply(logits, target, ignore_index)
    return F.cross_entropy(logits.reshape(-1, logits.shape[-1]).float(), target.reshape(-1), ignore_index=ignore_index)


class _SmallAttnFn(torch.autograd.Function):
    """q, k, v: [B, S, H, 64] -> [B, S, H, 64]; runs the short-sequence kernel on a packed [S*B, 3*H*64] buffer."""

    @staticmethod
    def forward(ctx, q, k, v):
        from . import kernels as K
        B, S, H, hd = q.shape
        packed = torch.cat([t.permute(1, 0, 2, 3).reshape(S * B, H * hd) for t in (q, k, v)], dim=1).contiguous()
        out = K.attn_small_fwd(packed, S, B, H, nshard=1, causal=True)
        ctx.save_for_backward(packed)
        ctx.dims = (B, S, H, hd)
        return out.view(S, B, H, hd).permute(1, 0, 2, 3)

    @staticmethod
    def backward(ctx, do):
        from . import kernels as K
        (packed,) = ctx.saved_tensors
        B, S, H, hd = ctx.dims
        do2 = do.permute(1, 0, 2, 3).reshape(S * B, H * hd).contiguous()
        dqkv = K.attn_small_bwd(packed, do2, S, B, H, nshard=1, causal=True)
        D = H * hd
        parts = [dqkv[:, i * D:(i + 1) * D].view(S, B, H, hd).permute(1, 0, 2, 3) for i in range(3)]
        return tuple(parts)


def causal_attention(q, k, v):
    """Causal self-attention on [B, S, H, hd] tensors (views are fine: the flash kernels take strides)."""
    B, S, H, hd = q.shape
    if use_kernels(q) and hd == 64 and S <= 96:
        return _SmallAttnFn.apply(q, k, v)
    if use_kernels(q) and hd in (64, 128):
        from .flash import flash_attention
        return flash_attention(q, k, v, causal=True)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
    return o.transpose(1, 2)


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        from . import kernels as K
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        return K.gelu_fwd(xc)

    @staticmethod
    def backward(ctx, dy):
        from . import kernels as K
        (x,) = ctx.saved_tensors
        return K.gelu_bwd(x, dy.contiguous())


def gelu(x):
    if use_kernels(x) and x.numel() % 8 == 0:
        y = _GeluFn.apply(x)
        return _tag(y, "gelu", x) if x.is_contiguous() else y
    return F.gelu(x)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        from . import kernels as K
        shape = g.shape
        g2, u2 = g.reshape(-1, shape[-1]).contiguous(), u.reshape(-1, shape[-1]).contiguous()
        ctx.save_for_backward(g2, u2)
        ctx.shape = shape
        return K.swiglu_fwd(g2, u2).view(shape)

    @staticmethod
    def backward(ctx, dy):
        from . import kernels as K
        g2, u2 = ctx.saved_tensors
        dg, du = K.swiglu_bwd(g2, u2, dy.reshape(-1, ctx.shape[-1]).contiguous())
        return dg.view(ctx.shape), du.view(ctx.shape)


def swiglu(g, u):
    """silu(g) * u."""
    if use_kernels(g) and g.shape[-1] % 8 == 0:
        # halves of a packed projection arrive as strided views: the contiguous copies made here are the tensors the
        # kernel's backward keeps, and the ones a following linear rebuilds its input from
        g, u = g.contiguous(), u.contiguous()
        return _tag(_SwigluFn.apply(g, u), "swiglu", g, u)
    return F.silu(g) * u


# ---------------------------------------------------------------------------------------------------------------------
# LM head + cross-entropy without the [tokens, vocab] logits
# ---------------------------------------------------------------------------------------------------------------------
class _ChunkedHeadLossFn(torch.autograd.Function):
    """Mean token cross-entropy of ``head(hidden)``, evaluated ``chunk_rows`` tokens at a time.  Forward AND backward of the
    head run chunk by chunk inside ``forward`` (the loss is the last op of a language model, so nothing is lost by doing
    the head's backward early): only one chunk of logits and of their gradient exists at any time — 0.4 GB instead of
    2 x 1.6 GB for 16 384 tokens of a 50 304-word vocabulary at 4 096 rows per chunk.  ``backward`` scales the stashed
    gradients by the incoming one.  The reference computes the full logits and hands them to ``nn.CrossEntropyLoss``
    (benchmarks/rtp_benchmark.py:182, rtp/models/transformer_lm_rtp.py:218-228).

    A rotated head pushes its shards once per chunk and direction; with N ranks that is 2 (N-1)/N of the head's bytes per
    chunk over NVLink, small against a chunk's GEMMs."""

    @staticmethod
    def forward(ctx, hidden, target, head, chunk_rows, ignore_index, *params):
        h2d = hidden.reshape(-1, hidden.shape[-1])
        t1d = target.reshape(-1)
        M = h2d.shape[0]
        n_valid = (t1d != ignore_index).sum().clamp(min=1)
        dx = torch.empty_like(h2d)
        gsum = [None] * len(params)
        total = torch.zeros((), dtype=torch.float32, device=h2d.device)
        for r0 in range(0, M, chunk_rows):
            r1 = min(r0 + chunk_rows, M)
            with torch.enable_grad():
                hc = h2d[r0:r1].detach().requires_grad_(True)
                logits = head(hc)
                # sum over the chunk's tokens; the division by the global count happens once, below
                tc = t1d[r0:r1]
                if use_kernels(logits) and logits.shape[-1] % 8 == 0:
                    loss_c = cross_entropy(logits, tc, ignore_index) * (tc != ignore_index).sum().clamp(min=1)
                else:
                    loss_c = F.cross_entropy(logits.float(), tc, ignore_index=ignore_index, reduction="sum")
                grads = torch.autograd.grad(loss_c, [hc] + list(params), allow_unused=True)
            total += loss_c.detach().float()
            dx[r0:r1] = grads[0]
            for k, g in enumerate(grads[1:]):
                if g is None:
                    continue
                gsum[k] = g.detach().float() if gsum[k] is None else gsum[k].add_(g)     # fp32 across the chunks
            del logits, loss_c, grads, hc
        inv = 1.0 / n_valid.to(torch.float32)
        ctx.save_for_backward(dx, inv, *[g if g is not None else torch.zeros(0, device=h2d.device) for g in gsum])
        ctx.has = [g is not None for g in gsum]
        ctx.dtypes = [p.dtype for p in params]
        ctx.shape = hidden.shape
        return total * inv

    @staticmethod
    def backward(ctx, gout):
        dx, inv, *gs = ctx.saved_tensors
        scale = (gout.to(torch.float32) * inv)
        dh = (dx.float() * scale).to(dx.dtype).view(ctx.shape)
        gp = [(g * scale).to(dt) if has else None for g, has, dt in zip(gs, ctx.has, ctx.dtypes)]
        return (dh, None, None, None, None, *gp)


def chunked_head_loss(hidden, target, head, chunk_rows: int = 4096, ignore_index: int = -100):
    """``cross_entropy(head(hidden), target)`` without ever holding more than ``chunk_rows`` rows of logits (see
    :class:`_ChunkedHeadLossFn`).  ``head`` is any module (a rotated ``ColumnParallelLinear`` included); its parameters
    receive their gradients through autograd as usual."""
    params = [p for p in head.parameters() if p.requires_grad]
    return _ChunkedHeadLossFn.apply(hidden, target, head, int(chunk_rows), ignore_index, *params)
