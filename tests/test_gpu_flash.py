"""Flash-attention kernels (tcgen05, online softmax) against a plain fp32 restatement of
softmax(scale * Q K^T + masks) V and its gradients."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _close(a, b, tol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = max(b.abs().max().item(), 1e-6)
    assert err <= tol * ref, (what, err, ref)
    # a stale or misplaced 128 x 128 tile shows as a large relative error of the whole tensor, too
    rel = ((a - b).norm() / (b.norm() + 1e-12)).item()
    assert rel <= tol, (what, "relative", rel)


def _reference(q, k, v, causal=False, attn_mask=None, kpm=None):
    """q: [B, Sq, H, hd], k / v: [B, Sk, H, hd] fp32 leaves -> [B, Sq, H, hd] (fp32 math)."""
    hd = q.shape[-1]
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * hd ** -0.5
    Sq, Sk = s.shape[-2:]
    if causal:
        s = s + torch.full((Sq, Sk), float("-inf"), device=s.device).triu_(1)
    if attn_mask is not None:
        s = s.masked_fill(attn_mask, float("-inf")) if attn_mask.dtype == torch.bool else s + attn_mask.float()
    if kpm is not None:
        s = s.masked_fill(kpm[:, None, None, :], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, v)


def _run_both(q, k, v, **kw):
    from rtp_b200.ops.flash import flash_attention
    from rtp_b200.ops import _lib
    qs, ks, vs = [t.clone().requires_grad_(True) for t in (q, k, v)]
    o = flash_attention(qs, ks, vs, causal=kw.get("causal", False), attn_mask=kw.get("attn_mask"),
                        key_padding_mask=kw.get("kpm"))
    do = torch.randn_like(o)
    o.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    qr, kr, vr = [t.float().requires_grad_(True) for t in (q, k, v)]
    oref = _reference(qr, kr, vr, **kw)
    oref.backward(do.float())
    return (o, qs.grad, ks.grad, vs.grad), (oref, qr.grad, kr.grad, vr.grad)


@pytest.mark.parametrize("B,S,H,hd,causal", [(2, 128, 4, 64, True), (1, 200, 3, 64, True), (1, 1024, 2, 128, True),
                                             (1, 2048, 2, 128, True), (2, 2048, 1, 64, True), (2, 384, 2, 64, False),
                                             (1, 200, 2, 128, False), (3, 40, 2, 64, True)])
def test_flash_attention_matches_fp32_math(B, S, H, hd, causal):
    torch.manual_seed(0)
    q, k, v = [torch.randn(B, S, H, hd, device="cuda", dtype=BF) for _ in range(3)]
    got, ref = _run_both(q, k, v, causal=causal)
    for g, r, name, tol in zip(got, ref, ("o", "dq", "dk", "dv"), (2e-2, 3e-2, 3e-2, 3e-2)):
        _close(g, r, tol, name)


def test_flash_attention_large_scores_need_the_rescale():
    """Scores that grow along the key axis force the running maximum to jump by more than the lazy-rescale gap."""
    torch.manual_seed(1)
    B, S, H, hd = 1, 512, 2, 64
    q = torch.randn(B, S, H, hd, device="cuda", dtype=BF)
    k = torch.randn(B, S, H, hd, device="cuda", dtype=BF)
    k = (k.float() * torch.linspace(0.2, 6.0, S, device="cuda")[None, :, None, None]).to(BF)
    v = torch.randn(B, S, H, hd, device="cuda", dtype=BF)
    got, ref = _run_both(q, k, v, causal=False)
    for g, r, name in zip(got, ref, ("o", "dq", "dk", "dv")):
        _close(g, r, 4e-2, name)


@pytest.mark.parametrize("kind", ["float", "bool", "bf16", "kpm", "both", "cross"])
def test_flash_attention_masks(kind):
    torch.manual_seed(2)
    B, Sq, Sk, H, hd = 2, 200, 200, 2, 64
    if kind == "cross":
        Sq, Sk = 130, 264
    q = torch.randn(B, Sq, H, hd, device="cuda", dtype=BF)
    k = torch.randn(B, Sk, H, hd, device="cuda", dtype=BF)
    v = torch.randn(B, Sk, H, hd, device="cuda", dtype=BF)
    mask = kpm = None
    if kind in ("float", "bf16", "both", "cross"):
        mask = torch.randn(Sq, Sk, device="cuda") * 2
        mask = mask.masked_fill(torch.rand(Sq, Sk, device="cuda") < 0.3, float("-inf"))
        mask[:, 0] = 0.0                              # every query keeps at least one key
        if kind == "bf16":
            mask = mask.to(BF)
    if kind == "bool":
        mask = torch.rand(Sq, Sk, device="cuda") < 0.4
        mask[:, 0] = False
    if kind in ("kpm", "both"):
        kpm = torch.zeros(B, Sk, dtype=torch.bool, device="cuda")
        kpm[0, Sk - 37:] = True
        kpm[1, 5:9] = True
    got, ref = _run_both(q, k, v, attn_mask=mask, kpm=kpm)
    for g, r, name in zip(got, ref, ("o", "dq", "dk", "dv")):
        _close(g, r, 3e-2, name)


@pytest.mark.parametrize("nshard,seq_first", [(1, False), (2, False), (2, True), (4, True)])
def test_flash_attention_packed_projection_layouts(nshard, seq_first):
    """The packed [tokens, 3 D] layout of a rotated QKV projection, both token orders, without any q / k / v copy."""
    from rtp_b200.ops.flash import flash_attention_packed
    from rtp_b200.ops import _lib
    torch.manual_seed(3)
    B, S, H, hd = 2, 256, 4, 64
    D = H * hd
    q, k, v = [torch.randn(B, S, H, hd, device="cuda", dtype=BF) for _ in range(3)]
    hp = H // nshard
    blocks = [t[:, :, j * hp:(j + 1) * hp].reshape(B, S, hp * hd) for j in range(nshard) for t in (q, k, v)]
    packed = torch.cat(blocks, dim=-1)                                        # [B, S, 3 D]
    packed = (packed.transpose(0, 1) if seq_first else packed).reshape(B * S, 3 * D).contiguous().requires_grad_(True)
    out = flash_attention_packed(packed, B, S, H, nshard=nshard, seq_first=seq_first, causal=True)
    do = torch.randn_like(out)
    out.backward(do)
    torch.cuda.synchronize()
    _lib.check_status()
    qr, kr, vr = [t.float().requires_grad_(True) for t in (q, k, v)]
    oref = _reference(qr, kr, vr, causal=True)                                # [B, S, H, hd]
    do4 = do.view(S, B, H, hd).transpose(0, 1) if seq_first else do.view(B, S, H, hd)
    oref.backward(do4.float())
    o4 = out.view(S, B, H, hd).transpose(0, 1) if seq_first else out.view(B, S, H, hd)
    _close(o4, oref, 2e-2, "o")
    gb = [t.grad[:, :, j * hp:(j + 1) * hp].reshape(B, S, hp * hd) for j in range(nshard) for t in (qr, kr, vr)]
    gref = torch.cat(gb, dim=-1)
    gref = (gref.transpose(0, 1) if seq_first else gref).reshape(B * S, 3 * D)
    _close(packed.grad, gref, 3e-2, "dqkv")


def test_flash_attention_dropout_shares_the_stream_of_the_short_sequence_kernels():
    """Same (seed, offset, position) -> same keep mask in every attention kernel of the library, so the flash kernels
    with dropout can be checked against the short-sequence kernels on a shape both support."""
    from rtp_b200.ops.flash import flash_attention_packed
    from rtp_b200.ops import kernels as K, _lib
    torch.manual_seed(4)
    S, B, H, N = 64, 3, 4, 2
    qkv = torch.randn(S * B, 3 * H * 64, device="cuda", dtype=BF)
    do = torch.randn(S * B, H * 64, device="cuda", dtype=BF)
    for causal in (True, False):
        ref_o = K.attn_small_fwd(qkv, S, B, H, nshard=N, causal=causal, drop_p=0.2, seed=7, offset=3)
        ref_g = K.attn_small_bwd(qkv, do, S, B, H, nshard=N, causal=causal, drop_p=0.2, seed=7, offset=3)
        x = qkv.clone().requires_grad_(True)
        o = flash_attention_packed(x, B, S, H, nshard=N, seq_first=True, causal=causal, dropout_p=0.2, seed=7, offset=3)
        o.backward(do)
        torch.cuda.synchronize()
        _lib.check_status()
        _close(o, ref_o, 2e-2, "o")
        _close(x.grad, ref_g, 3e-2, "dqkv")
        # and dropout really drops: the outputs differ from the deterministic ones
        o0 = flash_attention_packed(qkv, B, S, H, nshard=N, seq_first=True, causal=causal)
        assert (o0.float() - o.float()).abs().max().item() > 1e-2


def test_flash_attention_gpt_shape_runs_and_keeps_no_square_matrix():
    """GPT-1.3B attention shape (S 2048, 16 heads of 128): memory held between forward and backward is O(S)."""
    from rtp_b200.ops.flash import flash_attention_packed
    torch.manual_seed(5)
    B, S, H, hd = 2, 2048, 16, 128
    qkv = (torch.randn(B * S, 3 * H * hd, device="cuda", dtype=BF) * 0.5).requires_grad_(True)
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    out = flash_attention_packed(qkv, B, S, H, causal=True)
    held = torch.cuda.memory_allocated() - base
    assert held <= out.numel() * 2 + B * H * S * 4 + (1 << 20), held      # output + one fp32 per row
    out.backward(torch.randn_like(out))
    torch.cuda.synchronize()
    assert torch.isfinite(qkv.grad.float()).all()
