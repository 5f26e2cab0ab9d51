"""tcgen05 GEMM front-end: ``D = epilogue(A @ B^T (+ C))`` with bf16 operands and fp32 accumulation.

Both operands may be stored K-major (``[rows, K]`` row-major, the ``F.linear`` layout) or MN-major
(``[K, rows]`` row-major), which covers forward (x @ W^T), input gradient (dy @ W) and weight
gradient (dy^T @ x) of a linear layer without materialising a transpose.
"""
import ctypes as C

import torch

from . import _lib

ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2


def _chk2d(t, name):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride, got shape {tuple(t.shape)} stride {t.stride()}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16")


def gemm(a, b, *, a_mn=False, b_mn=False, bias=None, act=ACT_NONE, c=None, out=None, out_dtype=torch.bfloat16,
         mask=None, mask_scale=1.0, drop_p=0.0, seed=0, offset=0, bn=0, num_ctas=0):
    """``out[M,N] = epi(A·Bᵀ)``.

    a: ``[M,K]`` (or ``[K,M]`` when ``a_mn``); b: ``[N,K]`` (or ``[K,N]`` when ``b_mn``).
    Epilogue order: ``+c`` → ``+bias`` → activation → ``mask`` (out = mask>0 ? out*mask_scale : 0) → dropout.
    """
    _chk2d(a, "a")
    _chk2d(b, "b")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if K != Kb:
        raise ValueError(f"contraction mismatch: {K} vs {Kb}")
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    if out.dim() != 2 or out.stride(1) != 1 or out.shape != (M, N):
        raise ValueError("bad out tensor")
    args = _lib.GemmArgs()
    args.a, args.lda, args.a_mn = a.data_ptr(), a.stride(0), int(a_mn)
    args.b, args.ldb, args.b_mn = b.data_ptr(), b.stride(0), int(b_mn)
    args.M, args.N, args.K = M, N, K
    args.d, args.ldd, args.d_fp32 = out.data_ptr(), out.stride(0), int(out.dtype == torch.float32)
    if c is not None:
        args.c, args.ldc, args.c_fp32 = c.data_ptr(), c.stride(0), int(c.dtype == torch.float32)
    if bias is not None:
        if bias.dtype != torch.bfloat16 or not bias.is_contiguous() or bias.numel() != N:
            raise ValueError("bias must be a contiguous bf16 vector of length N")
        args.bias = bias.data_ptr()
    args.act = int(act)
    if mask is not None:
        _chk2d(mask, "mask")
        args.mask, args.ldmask, args.mask_scale = mask.data_ptr(), mask.stride(0), float(mask_scale)
    args.drop_p, args.seed, args.offset = float(drop_p), int(seed), int(offset)
    args.status = _lib.status_word(a.device).data_ptr()
    args.num_ctas, args.bn = int(num_ctas), int(bn)
    _lib.check(_lib.lib().rtp_gemm(C.byref(args), _lib.stream_ptr()), "rtp_gemm")
    return out
