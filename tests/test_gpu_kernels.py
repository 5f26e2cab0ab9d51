"""Memory-bound sm_100a kernels vs plain PyTorch fp32 references."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    assert err <= tol * max(b.float().abs().max().item(), 1e-6), err


@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(rms):
    from rtp_b200.ops import kernels as K
    torch.manual_seed(0)
    M, D = 1000, 2048
    x = torch.randn(M, D, device="cuda", dtype=BF)
    sub = torch.randn(M, D, device="cuda", dtype=BF)
    g = (torch.randn(D, device="cuda") * 0.1 + 1).to(BF)
    b = None if rms else (torch.randn(D, device="cuda") * 0.1).to(BF)
    y, h, mean, rstd = K.norm_fwd(x, sub, g, b, rms=rms)
    hr = (x.float() + sub.float()).to(BF).float().requires_grad_(True)
    gr = g.float().requires_grad_(True)
    br = None if rms else b.float().requires_grad_(True)
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-5) * gr if rms else F.layer_norm(hr, (D,), gr, br, 1e-5)
    _close(y, yr, 1e-2)
    dy = torch.randn(M, D, device="cuda", dtype=BF)
    yr.backward(dy.float())
    dx, dsub, dg, db = K.norm_bwd(dy, h, g, mean, rstd, rms=rms, has_beta=not rms)
    _close(dx, hr.grad, 1e-2)
    _close(dsub, hr.grad, 1e-2)
    _close(dg, gr.grad, 1e-2)
    if not rms:
        _close(db, br.grad, 1e-2)


def test_norm_dropout_mask_is_reproduced_in_backward():
    from rtp_b200.ops import kernels as K
    torch.manual_seed(0)
    M, D = 512, 1024
    x = torch.zeros(M, D, device="cuda", dtype=BF)
    sub = torch.ones(M, D, device="cuda", dtype=BF)
    g = torch.ones(D, device="cuda", dtype=BF)
    y, h, mean, rstd = K.norm_fwd(x, sub, g, None, rms=True, drop_p=0.3, seed=5, offset=9)
    kept = h != 0
    assert abs(kept.float().mean().item() - 0.7) < 0.01
    dy = torch.ones(M, D, device="cuda", dtype=BF)
    dx, dsub, _, _ = K.norm_bwd(dy, h, g, mean, rstd, rms=True, has_beta=False, drop_p=0.3, seed=5, offset=9)
    same = ((dsub != 0) == kept) | (dx == 0)
    assert same.float().mean().item() > 0.999


def test_cross_entropy():
    from rtp_b200.ops import kernels as K
    torch.manual_seed(0)
    M, V = 1000, 10240
    lg = (torch.randn(M, V, device="cuda") * 3).to(BF)
    t = torch.randint(0, V, (M,), device="cuda")
    t[5] = -100
    lr = lg.float().requires_grad_(True)
    lossr = F.cross_entropy(lr, t, reduction="none", ignore_index=-100)
    (lossr.sum() * 0.5).backward()
    l2 = lg.clone()
    loss = K.cross_entropy_(l2, t, grad_scale=0.5)
    _close(loss, lossr, 1e-3)
    _close(l2, lr.grad, 2e-2)


def test_embedding_shards():
    from rtp_b200.ops import kernels as K
    torch.manual_seed(0)
    V, D, S, B, N = 1024, 256, 32, 8, 2
    Ds = D // N
    table = torch.randn(V, D, device="cuda", dtype=BF)
    ids = torch.randint(0, V, (S, B), device="cuda")
    pe = torch.randn(64, D, device="cuda", dtype=BF)
    out = torch.empty(S * B, D, device="cuda", dtype=BF)
    for j in range(N):
        K.embed_fwd(table[:, j * Ds:(j + 1) * Ds].contiguous(), ids.view(-1), out, j * Ds, D=D, scale=16.0, pe=pe,
                    tokens_per_pos=B)
    r = table[ids.view(-1)].float() * 16.0 + pe[:S].float().repeat_interleave(B, 0)
    _close(out, r, 1e-2)
    dy = torch.randn(S * B, D, device="cuda", dtype=BF)
    gt = torch.zeros(V, Ds, device="cuda", dtype=BF)
    K.embed_bwd(gt, ids.view(-1), dy, Ds, D=D, scale=16.0)
    rr = torch.zeros(V, Ds, device="cuda").index_add_(0, ids.view(-1), dy[:, Ds:2 * Ds].float() * 16.0)
    _close(gt, rr, 3e-2)


@pytest.mark.parametrize("S,B,H,N", [(32, 4, 8, 1), (32, 4, 8, 2), (64, 2, 4, 4), (96, 2, 2, 1), (17, 3, 4, 2)])
def test_attention_small(S, B, H, N):
    from rtp_b200.ops import kernels as K
    torch.manual_seed(0)
    D = H * 64
    q, k, v = [torch.randn(S, B, H, 64, device="cuda") for _ in range(3)]
    hp = H // N
    parts = [t[:, :, j * hp:(j + 1) * hp].reshape(S * B, hp * 64) for j in range(N) for t in (q, k, v)]
    qkv = torch.cat(parts, 1).to(BF).contiguous()
    qr, kr, vr = [t.to(BF).float().requires_grad_(True) for t in (q, k, v)]
    o = F.scaled_dot_product_attention(qr.permute(1, 2, 0, 3), kr.permute(1, 2, 0, 3), vr.permute(1, 2, 0, 3),
                                       is_causal=True)
    oref = o.permute(2, 0, 1, 3).reshape(S * B, D)
    out = K.attn_small_fwd(qkv, S, B, H, nshard=N, causal=True)
    _close(out, oref, 2e-2)
    do = torch.randn(S * B, D, device="cuda", dtype=BF)
    oref.backward(do.float())
    dqkv = K.attn_small_bwd(qkv, do, S, B, H, nshard=N, causal=True)
    gparts = [t.grad[:, :, j * hp:(j + 1) * hp].reshape(S * B, hp * 64) for j in range(N) for t in (qr, kr, vr)]
    _close(dqkv, torch.cat(gparts, 1), 2e-2)


@pytest.mark.parametrize("S,B,H,N,causal,p", [(32, 3, 5, 1, True, 0.0), (32, 5, 6, 2, False, 0.1), (64, 3, 3, 1, True, 0.1),
                                              (32, 32, 32, 8, True, 0.1)])
def test_attention_tensor_core_kernels_match_scalar_kernels(S, B, H, N, causal, p):
    """The tcgen05 kernels (S = 32 / 64) and the scalar kernels share the layout and the dropout stream."""
    from rtp_b200.ops import kernels as K
    torch.manual_seed(1)
    qkv = torch.randn(S * B, 3 * H * 64, device="cuda", dtype=BF)
    do = torch.randn(S * B, H * 64, device="cuda", dtype=BF)
    kw = dict(nshard=N, causal=causal, drop_p=p, seed=11, offset=5)
    try:
        K.set_attn_tc(False)
        o_ref = K.attn_small_fwd(qkv, S, B, H, **kw)
        g_ref = K.attn_small_bwd(qkv, do, S, B, H, **kw)
    finally:
        K.set_attn_tc(True)
    o = K.attn_small_fwd(qkv, S, B, H, **kw)
    g = K.attn_small_bwd(qkv, do, S, B, H, **kw)
    torch.cuda.synchronize()
    assert K.attn_tc_error() == 0
    _close(o, o_ref, 2e-2)
    _close(g, g_ref, 3e-2)


def test_colsum_and_adam():
    from rtp_b200.ops import kernels as K
    torch.manual_seed(0)
    x = torch.randn(1000, 2048, device="cuda", dtype=BF)
    _close(K.colsum(x), x.float().sum(0), 1e-3)
    for state_dtype in (torch.float32, BF):
        ps = [torch.randn(n, device="cuda").to(BF) for n in (5000, 2048 * 7 + 3, 100000)]
        gs = [torch.randn_like(p) for p in ps]
        ref_p = [p.float().clone().requires_grad_(True) for p in ps]
        opt = torch.optim.Adam(ref_p, lr=1e-2)
        ms = [torch.zeros(p.numel(), device="cuda", dtype=state_dtype) for p in ps]
        vs = [torch.zeros(p.numel(), device="cuda", dtype=state_dtype) for p in ps]
        plan = K.AdamPlan([(p, g, m, v, 1.0) for p, g, m, v in zip(ps, gs, ms, vs)], "cuda")
        step = torch.zeros(1, dtype=torch.int64, device="cuda")
        for _ in range(3):
            for rp, g in zip(ref_p, gs):
                rp.grad = g.float().clamp(-0.5, 0.5)
            opt.step()
            step += 1
            plan.step(step, 1e-2, 0.9, 0.999, 1e-8, clip_value=0.5)
        for p, rp in zip(ps, ref_p):
            _close(p, rp.detach(), 2e-2)


def test_moe_dispatch_combine_by_index_matches_dense_einsums():
    from rtp_b200.module.top2gate import top2_routing, top2gating
    from rtp_b200.ops import moe as MK
    torch.manual_seed(0)
    S, E, M = 256, 8, 128
    logits = torch.randn(S, E, device="cuda")
    noise = torch.randn(S, E, device="cuda")
    l_aux, idx, loc, gate, valid, cap, _, _ = top2_routing(logits, 1.25, noise)
    _, comb_w, disp_mask = top2gating(logits, 1.25, noise)
    x = torch.randn(S, M, device="cuda", dtype=BF, requires_grad=True)
    gate = gate.detach().requires_grad_(True)
    disp = MK.dispatch(x, idx, loc, valid, E, cap)
    ref_disp = torch.einsum("sec,sm->ecm", disp_mask.float(), x.float())
    _close(disp, ref_disp, 1e-2)
    eo = torch.randn(E, cap, M, device="cuda", dtype=BF, requires_grad=True)
    y = MK.combine(eo, idx, loc, gate, valid)
    ref_y = torch.einsum("sec,ecm->sm", comb_w.float(), eo.float())
    _close(y, ref_y, 2e-2)
    dy = torch.randn_like(y)
    y.backward(dy)
    disp.backward(torch.ones_like(disp))
    eo_r = eo.detach().float().requires_grad_(True)
    torch.einsum("sec,ecm->sm", comb_w.float(), eo_r).backward(dy.float())
    _close(eo.grad, eo_r.grad, 2e-2)
    x_r = x.detach().float().requires_grad_(True)
    torch.einsum("sec,sm->ecm", disp_mask.float(), x_r).sum().backward()
    _close(x.grad, x_r.grad, 1e-2)
    # gate gradient: d y / d gate[s, k] = <dy[s], eo[slot]>
    slot = torch.where(valid, idx * cap + loc, torch.zeros_like(idx))
    ref_dg = (dy.float().unsqueeze(1) * eo.detach().float().reshape(E * cap, M)[slot]).sum(-1) * valid
    _close(gate.grad, ref_dg, 2e-2)


@pytest.mark.parametrize("S,E,cf", [(64, 8, 1.0), (2048, 16, 1.0), (1500, 60, 0.5), (96, 2, 2.0)])
def test_top2_gate_kernels_match_reference_routing(S, E, cf):
    """Fused gating kernels against the dense PyTorch restatement of the reference (same injected noise)."""
    from rtp_b200.module.top2gate import top2_routing
    from rtp_b200.parallel.context import set_backend
    torch.manual_seed(3)
    logits = (torch.randn(S, E, device="cuda") * 2).requires_grad_(True)
    noise = torch.randn(S, E, device="cuda")
    w = torch.randn(S, 2, device="cuda")
    set_backend("functional")
    try:
        ref = top2_routing(logits, cf, noise)
        (ref[3] * w).sum().add(ref[0] * 7.0).backward()
    finally:
        set_backend("auto")
    g_ref = logits.grad.clone()
    logits.grad = None
    out = top2_routing(logits, cf, noise)
    (out[3] * w).sum().add(out[0] * 7.0).backward()
    assert torch.equal(out[1], ref[1]), "experts differ"
    assert torch.equal(out[4], ref[4]), "validity differs"
    assert torch.equal(out[2] * out[4], ref[2] * ref[4]), "slots differ"
    assert out[5] == ref[5]
    _close(out[3], ref[3], 1e-5)
    assert abs(out[0].item() - ref[0].item()) < 1e-6
    _close(logits.grad, g_ref, 1e-4)


def test_rope_kernel():
    from rtp_b200.ops import kernels as K
    from rtp_b200.models.llama import rope_tables
    torch.manual_seed(0)
    B, S, H, hd = 3, 50, 4, 64
    x = torch.randn(B, S, H, hd, device="cuda", dtype=BF, requires_grad=True)
    cos, sin = rope_tables(S, hd, 10000.0, "cuda")
    xr = x.detach().float().requires_grad_(True)
    x1, x2 = xr[..., 0::2], xr[..., 1::2]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    ref = torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1).flatten(-2)
    y = K.rope(x, cos, sin)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref.backward(dy.float())
    _close(y, ref, 1e-2)
    _close(x.grad, xr.grad, 1e-2)


@pytest.mark.parametrize("cin,cout,k,stride,pad", [(32, 64, 3, 1, 0), (16, 32, 3, 2, 1), (8, 24, 5, 1, 2)])
def test_rotated_conv_on_gemm_kernels(cin, cout, k, stride, pad):
    """Conv2d = im2col + rotation GEMM (+ col2im in backward) against F.conv2d in fp32."""
    import torch.nn.functional as F
    from rtp_b200.module.conv import ColumnParallelConv2d
    from rtp_b200.ops import _lib
    torch.manual_seed(0)
    ref = torch.nn.Conv2d(cin, cout, k, stride=stride, padding=pad).cuda()
    m = ColumnParallelConv2d(cin, cout, k, stride=stride, padding=pad, Conv2d_layer=ref, world_size=1, rank=0).cuda().to(BF)
    x = torch.randn(4, cin, 14, 14, device="cuda", dtype=BF, requires_grad=True)
    y = m(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    torch.cuda.synchronize()
    _lib.check_status()
    xr = x.detach().float().requires_grad_(True)
    w = ref.weight.detach().to(BF).float().requires_grad_(True)
    b = ref.bias.detach().to(BF).float().requires_grad_(True)
    yr = F.conv2d(xr, w, b, stride=stride, padding=pad)
    yr.backward(dy.float())
    _close(y, yr, 2e-2)
    _close(x.grad, xr.grad, 3e-2)
    _close(m.conv.weight.grad, w.grad, 3e-2)
    _close(m.conv.bias.grad, b.grad, 3e-2)
