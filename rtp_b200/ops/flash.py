"""Flash attention on the tcgen05 kernels of ``csrc/flash_attn.cu``.

``softmax(scale * Q K^T + mask) V`` with online softmax: nothing of size S x S is written to global memory, forward
keeps one fp32 log-sum-exp per query row and backward recomputes the probabilities.  Causal or full attention,
optional additive ``[Sq, Sk]`` mask, optional key-padding mask, optional dropout on the probabilities (regenerated in
backward from a counter-based generator), any sequence length, ``head_dim`` 64 or 128, bf16 CUDA.

Two front-ends:

* :func:`flash_attention` takes ``[B, S, H, hd]`` views (any batch / sequence / head strides, unit stride on ``hd``);
* :func:`flash_attention_packed` takes the packed projection ``[tokens, 3 * D]`` of a rotated MHA directly — the q / k /
  v blocks of every head-shard side by side, tokens ordered ``[B, S]`` or ``[S, B]`` — and writes ``[tokens, D]``, so that
  no head transpose or q/k/v split is ever materialised (forward or backward).

Replaces the attention inside the reference's vendored ``multi_head_attention_forward``
(rtp/module/functional.py:785-792, :825).
"""
import ctypes as C
import itertools

import torch

from . import _lib

_offsets = itertools.count(1 << 20)


def flash_attention_available(seq_len: int, head_dim: int) -> bool:
    return head_dim in (64, 128) and seq_len >= 1


def next_dropout_offset() -> int:
    """A fresh offset of the counter-based dropout generator for one attention call of the module path."""
    return next(_offsets)


def _ref4(t):
    """FlashRef of a [B, S, H, hd] view."""
    B, S, H, hd = t.shape
    if t.stride(3) != 1:
        raise ValueError("head_dim must have unit stride")
    r = _lib.FlashRef()
    r.ptr, r.sb, r.ss = t.data_ptr(), t.stride(0), t.stride(1)
    r.col_base, r.hpg, r.gstride, r.hstride = 0, H, 0, t.stride(2)
    r.width = (H - 1) * t.stride(2) + hd
    return r


def _ref_packed(buf, which, B, S, H, hd, nshard, seq_first, row_width):
    """FlashRef of block ``which`` (0 q, 1 k, 2 v; -1: a plain [tokens, D] buffer) of a [tokens, row_width] buffer."""
    D = H * hd
    r = _lib.FlashRef()
    r.ptr = buf.data_ptr()
    ld = buf.stride(0)
    r.sb, r.ss = (ld, B * ld) if seq_first else (S * ld, ld)
    if which < 0:
        r.col_base, r.hpg, r.gstride, r.hstride = 0, H, 0, hd
    else:
        r.col_base, r.hpg, r.gstride, r.hstride = which * (D // nshard), H // nshard, 3 * (D // nshard), hd
    r.width = row_width
    return r


def _mask_args(a, attn_mask, key_padding_mask, keep):
    if attn_mask is not None:
        m = attn_mask
        if m.dtype == torch.bool:
            m = torch.zeros(m.shape, dtype=torch.float32, device=m.device).masked_fill_(m, float("-inf"))
        elif m.dtype not in (torch.float32, torch.bfloat16):
            m = m.float()
        if m.dim() != 2 or m.stride(1) != 1:
            m = m.reshape(m.shape[-2], m.shape[-1]).contiguous()
        keep.append(m)
        a.mask, a.mask_ld, a.mask_fp32 = m.data_ptr(), m.stride(0), int(m.dtype == torch.float32)
    if key_padding_mask is not None:
        k = key_padding_mask
        k = (k != 0) if k.dtype != torch.bool else k
        k = k.to(torch.uint8).contiguous()
        keep.append(k)
        a.kpm, a.kpm_ld = k.data_ptr(), k.stride(0)


def _common(a, B, H, Sq, Sk, hd, causal, sm_scale, drop_p, seed, offset, step, dev):
    a.B, a.H, a.Sq, a.Sk, a.head_dim, a.causal = B, H, Sq, Sk, hd, int(bool(causal))
    a.sm_scale = float(sm_scale if sm_scale is not None else hd ** -0.5)
    a.drop_p, a.seed, a.offset = float(drop_p), int(seed), int(offset)
    a.step_ptr = step.data_ptr() if step is not None else None
    a.status = _lib.status_word(dev).data_ptr()


def _check(rc, what):
    _lib.launches += 2 if what.endswith("bwd") else 1
    if rc != 0:
        raise RuntimeError(f"{what}: {_lib.lib().rtp_flash_last_error().decode()}")


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, attn_mask, key_padding_mask, drop_p, seed, offset, step, sm_scale):
        B, Sq, H, hd = q.shape
        Sk = k.shape[1]
        q, k, v = [t if t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0
                   else t.contiguous() for t in (q, k, v)]
        o = torch.empty(B, Sq, H, hd, dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(B * H, Sq, dtype=torch.float32, device=q.device)
        a = _lib.FlashArgs()
        keep = []
        a.q, a.k, a.v, a.o = _ref4(q), _ref4(k), _ref4(v), _ref4(o)
        a.lse = lse.data_ptr()
        _mask_args(a, attn_mask, key_padding_mask, keep)
        _common(a, B, H, Sq, Sk, hd, causal, sm_scale, drop_p, seed, offset, step, q.device)
        _check(_lib.lib().rtp_flash_fwd(C.byref(a), _lib.stream_ptr()), "rtp_flash_fwd")
        ctx.save_for_backward(q, k, v, o, lse, *keep)
        ctx.cfg = (causal, attn_mask is not None, key_padding_mask is not None, drop_p, seed, offset, step, sm_scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, *keep = ctx.saved_tensors
        causal, has_mask, has_kpm, drop_p, seed, offset, step, sm_scale = ctx.cfg
        B, Sq, H, hd = q.shape
        Sk = k.shape[1]
        if do.stride(3) != 1 or any(s % 8 for s in do.stride()[:3]) or do.data_ptr() % 16:
            do = do.contiguous()
        dq = torch.empty(B, Sq, H, hd, dtype=torch.bfloat16, device=q.device)
        dk = torch.empty(B, Sk, H, hd, dtype=torch.bfloat16, device=q.device)
        dv = torch.empty(B, Sk, H, hd, dtype=torch.bfloat16, device=q.device)
        delta = torch.empty_like(lse)
        a = _lib.FlashArgs()
        a.q, a.k, a.v, a.o = _ref4(q), _ref4(k), _ref4(v), _ref4(o)
        a.dout, a.dq, a.dk, a.dv = _ref4(do), _ref4(dq), _ref4(dk), _ref4(dv)
        a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
        it = iter(keep)
        m = next(it) if has_mask else None
        kp = next(it) if has_kpm else None
        _mask_args(a, m, kp, [])
        _common(a, B, H, Sq, Sk, hd, causal, sm_scale, drop_p, seed, offset, step, q.device)
        _check(_lib.lib().rtp_flash_bwd(C.byref(a), _lib.stream_ptr()), "rtp_flash_bwd")
        return dq, dk, dv, None, None, None, None, None, None, None, None


def flash_attention(q, k, v, causal=False, attn_mask=None, key_padding_mask=None, dropout_p=0.0, seed=0, offset=None,
                    step=None, sm_scale=None):
    """``q``: [B, Sq, H, hd], ``k`` / ``v``: [B, Sk, H, hd] (bf16 CUDA views) -> [B, Sq, H, hd].

    ``attn_mask``: additive float (or bool, True = masked) ``[Sq, Sk]``; ``key_padding_mask``: ``[B, Sk]``, True = the key
    is ignored.  Dropout uses the library's counter-based generator: the mask of element (b, h, i, j) depends only on
    (seed, offset, step counter, position), so backward regenerates it."""
    if dropout_p > 0 and offset is None:
        offset = next_dropout_offset()
    return _FlashFn.apply(q, k, v, bool(causal), attn_mask, key_padding_mask, float(dropout_p), seed, offset or 0, step,
                          sm_scale)


class _FlashPackedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, B, S, H, nshard, seq_first, causal, attn_mask, key_padding_mask, drop_p, seed, offset, step):
        T, W = qkv.shape
        D = W // 3
        hd = D // H
        if qkv.stride(1) != 1 or qkv.stride(0) % 8 or qkv.data_ptr() % 16:
            qkv = qkv.contiguous()
        out = torch.empty(T, D, dtype=torch.bfloat16, device=qkv.device)
        lse = torch.empty(B * H, S, dtype=torch.float32, device=qkv.device)
        a = _lib.FlashArgs()
        keep = []
        a.q, a.k, a.v = [_ref_packed(qkv, i, B, S, H, hd, nshard, seq_first, W) for i in range(3)]
        a.o = _ref_packed(out, -1, B, S, H, hd, nshard, seq_first, D)
        a.lse = lse.data_ptr()
        _mask_args(a, attn_mask, key_padding_mask, keep)
        _common(a, B, H, S, S, hd, causal, None, drop_p, seed, offset, step, qkv.device)
        _check(_lib.lib().rtp_flash_fwd(C.byref(a), _lib.stream_ptr()), "rtp_flash_fwd")
        ctx.save_for_backward(qkv, out, lse, *keep)
        ctx.cfg = (B, S, H, nshard, seq_first, causal, attn_mask is not None, key_padding_mask is not None, drop_p, seed,
                   offset, step)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, *keep = ctx.saved_tensors
        B, S, H, nshard, seq_first, causal, has_mask, has_kpm, drop_p, seed, offset, step = ctx.cfg
        T, W = qkv.shape
        D = W // 3
        hd = D // H
        if dout.stride(1) != 1 or dout.stride(0) % 8 or dout.data_ptr() % 16:
            dout = dout.contiguous()
        dqkv = torch.empty(T, W, dtype=torch.bfloat16, device=qkv.device)
        delta = torch.empty_like(lse)
        a = _lib.FlashArgs()
        a.q, a.k, a.v = [_ref_packed(qkv, i, B, S, H, hd, nshard, seq_first, W) for i in range(3)]
        a.dq, a.dk, a.dv = [_ref_packed(dqkv, i, B, S, H, hd, nshard, seq_first, W) for i in range(3)]
        a.o = _ref_packed(out, -1, B, S, H, hd, nshard, seq_first, D)
        a.dout = _ref_packed(dout, -1, B, S, H, hd, nshard, seq_first, D)
        a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
        it = iter(keep)
        m = next(it) if has_mask else None
        kp = next(it) if has_kpm else None
        _mask_args(a, m, kp, [])
        _common(a, B, H, S, S, hd, causal, None, drop_p, seed, offset, step, qkv.device)
        _check(_lib.lib().rtp_flash_bwd(C.byref(a), _lib.stream_ptr()), "rtp_flash_bwd")
        return (dqkv,) + (None,) * 12


def flash_attention_packed(qkv, B, S, H, nshard=1, seq_first=False, causal=False, attn_mask=None,
                           key_padding_mask=None, dropout_p=0.0, seed=0, offset=None, step=None):
    """Self-attention on a packed projection ``qkv`` [tokens, 3 * D]: the columns hold, for each of ``nshard`` head
    groups, the q, k and v blocks of that group's ``H / nshard`` heads side by side (the output layout of a rotated,
    packed QKV projection; ``nshard = 1`` is the plain ``[q | k | v]`` layout).  Tokens are ordered ``b * S + s``
    (``seq_first=False``) or ``s * B + b``.  Returns ``[tokens, D]`` in the same token order."""
    if dropout_p > 0 and offset is None:
        offset = next_dropout_offset()
    return _FlashPackedFn.apply(qkv, B, S, H, nshard, bool(seq_first), bool(causal), attn_mask, key_padding_mask,
                                float(dropout_p), seed, offset or 0, step)
