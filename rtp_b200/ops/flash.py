"""Long-sequence causal attention on the tcgen05 GEMM kernel.

The per-head matrices are column windows of the [B*S, H*hd] projections, so no head transpose is materialised:
``scores = Q K^T`` and ``O = P V`` (and the four backward products) are *batched* launches of the rotation GEMM
kernel whose tile coordinates carry the (batch, head) offsets; tiles above the diagonal are skipped and the
contraction of ``P V`` / ``dS K`` stops at the diagonal.  The softmax (forward and backward) is a row kernel over
the bf16 probability matrix, which is kept for backward (``B*H*S*S`` bf16 per layer).

Requirements: bf16 CUDA, ``S % 128 == 0``, ``head_dim`` 64 or 128."""
import ctypes as C

import torch

from . import _lib
from . import kernels as K


def flash_attention_available(seq_len: int, head_dim: int) -> bool:
    return seq_len % 128 == 0 and head_dim in (64, 128)


def _bgemm(a, a_mn, a_rows, a_cols, lda, b, b_mn, b_rows, b_cols, ldb, M, N, Kd, batch, inner, offs, d, ldd, d_bo,
           d_bi, alpha=1.0, causal=0):
    g = _lib.GemmBatched()
    g.a, g.lda, g.a_mn, g.a_rows, g.a_cols = a.data_ptr(), lda, int(a_mn), a_rows, a_cols
    g.b, g.ldb, g.b_mn, g.b_rows, g.b_cols = b.data_ptr(), ldb, int(b_mn), b_rows, b_cols
    g.M, g.N, g.K, g.batch, g.batch_inner = M, N, Kd, batch, inner
    (g.a_bo_mn, g.a_bo_k, g.a_bi_mn, g.a_bi_k, g.b_bo_mn, g.b_bo_k, g.b_bi_mn, g.b_bi_k) = offs
    g.d, g.ldd, g.d_bo, g.d_bi = d.data_ptr(), ldd, d_bo, d_bi
    g.alpha, g.causal, g.bn = alpha, causal, 0
    g.status = _lib.status_word(a.device).data_ptr()
    _lib.check(_lib.lib().rtp_gemm_batched(C.byref(g), _lib.stream_ptr()), "rtp_gemm_batched")


class _CausalAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v):
        B, S, H, hd = q.shape
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        D, BH = H * hd, B * H
        scale = hd ** -0.5
        p = torch.empty(BH, S, S, dtype=torch.bfloat16, device=q.device)
        # scores[z] = Q_z K_z^T : A = Q window (rows b*S.., cols h*hd..), B = K window
        _bgemm(q, False, B * S, D, D, k, False, B * S, D, D, S, S, hd, BH, H, (S, 0, 0, hd, S, 0, 0, hd),
               p, S, H * S * S, S * S, causal=1)
        K.causal_softmax_(p, S, scale)
        o = torch.empty(B, S, H, hd, dtype=torch.bfloat16, device=q.device)
        # O_z = P_z V_z : A = P stack [BH*S, S]; B = V stored [keys, hd] (MN-major window)
        _bgemm(p, False, BH * S, S, S, v, True, B * S, D, D, S, hd, S, BH, H, (H * S, 0, S, 0, 0, S, hd, 0),
               o, D, S * D, hd, causal=2)
        ctx.save_for_backward(q, k, v, p)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, p = ctx.saved_tensors
        B, S, H, hd = q.shape
        D, BH = H * hd, B * H
        scale = hd ** -0.5
        do = do.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        # dV_z = P_z^T dO_z : A = P read transposed (stored [q, keys]), B = dO stored [q, hd]
        _bgemm(p, True, BH * S, S, S, do, True, B * S, D, D, S, hd, S, BH, H, (0, H * S, 0, S, 0, S, hd, 0),
               dv, D, S * D, hd, causal=3)      # only queries at or after a key contribute to it
        # dP_z = dO_z V_z^T
        dp = torch.empty_like(p)
        _bgemm(do, False, B * S, D, D, v, False, B * S, D, D, S, S, hd, BH, H, (S, 0, 0, hd, S, 0, 0, hd),
               dp, S, H * S * S, S * S, causal=1)
        K.causal_softmax_bwd_(p, dp, S, scale)          # dp now holds dS (scaled)
        # dQ_z = dS_z K_z ; dK_z = dS_z^T Q_z
        _bgemm(dp, False, BH * S, S, S, k, True, B * S, D, D, S, hd, S, BH, H, (H * S, 0, S, 0, 0, S, hd, 0),
               dq, D, S * D, hd, causal=2)
        _bgemm(dp, True, BH * S, S, S, q, True, B * S, D, D, S, hd, S, BH, H, (0, H * S, 0, S, 0, S, hd, 0),
               dk, D, S * D, hd, causal=3)
        return dq, dk, dv


def flash_attention(q, k, v, causal=True):
    """q, k, v: [B, S, H, hd] bf16 CUDA -> [B, S, H, hd]."""
    if not causal:
        raise NotImplementedError("only causal attention runs on the batched-GEMM path")
    return _CausalAttention.apply(q, k, v)
