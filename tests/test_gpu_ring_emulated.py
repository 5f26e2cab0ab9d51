"""Multi-rank rotation protocol on ONE GPU: the kernel is launched cooperatively with N x G CTAs, CTA group e
plays rank e on its own workspace, so weight pushes, arrival/credit counters and the travelling-gradient ring
run exactly as across GPUs (peer pointers simply point into the same device)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _close(a, b, tol, what=""):
    err = (a.float() - b.float()).abs().max().item()
    assert err <= tol * max(b.float().abs().max().item(), 1e-6), (what, err)


def _rings(world, slot_bytes, ctas, L, _lib):
    wss = []
    for _ in range(world):
        p = C.c_void_p()
        _lib.check(L.rtp_ws_create_world(slot_bytes, world, C.byref(p)), "ws")
        wss.append(p.value)
    rings = (_lib.Ring * world)()
    for r in range(world):
        rings[r].rank, rings[r].world = r, world
        for q in range(world):
            rings[r].ws[q] = wss[q]
        rings[r].slot_bytes, rings[r].ctas, rings[r].timeout_ns = slot_bytes, ctas, 500_000_000
    return wss, rings


def _status_ok(wss, L, _lib):
    st = C.c_ulonglong(0)
    for w in wss:
        L.rtp_ws_status(w, C.byref(st), _lib.stream_ptr())
        assert st.value == 0, f"rotation kernel reported status {st.value}"


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("shape", [(256, 512, 1024), (1000, 2048, 2048)])
def test_rotated_linear_fwd_bwd(world, mode, shape):
    from rtp_b200.ops import _lib, kernels as K
    L = _lib.lib()
    torch.manual_seed(0)
    M, IN, OUT = shape
    G_ = 148 // world
    full_w = (torch.randn(OUT, IN, device="cuda") * 0.05).to(BF)
    full_b = (torch.randn(OUT, device="cuda") * 0.1).to(BF)
    Os, Ks = (OUT // world, IN) if mode == 0 else (OUT, IN // world)
    bias_off = (Os * Ks + 63) // 64 * 64
    nflat = bias_off + (Os + 63) // 64 * 64
    slot_bytes = (nflat * 2 + 65535) // 65536 * 65536
    wss, rings = _rings(world, slot_bytes, G_, L, _lib)
    ops = (_lib.LinearFwd * world)()
    homes, xs, ys = [], [], []
    for r in range(world):
        flat = torch.zeros(nflat, device="cuda", dtype=BF)
        if mode == 0:
            flat[:Os * Ks] = full_w[r * Os:(r + 1) * Os].reshape(-1)
            flat[bias_off:bias_off + Os] = full_b[r * Os:(r + 1) * Os]
        else:
            flat[:Os * Ks] = full_w[:, r * Ks:(r + 1) * Ks].reshape(-1)
            flat[bias_off:bias_off + Os] = (full_b.float() / world).to(BF)
        x = torch.randn(M, IN, device="cuda", dtype=BF)
        y = torch.zeros(M, OUT, device="cuda", dtype=BF)
        homes.append(flat); xs.append(x); ys.append(y)
        ops[r].mode, ops[r].M, ops[r].in_features, ops[r].out_features = mode, M, IN, OUT
        ops[r].home, ops[r].bias_off, ops[r].shard_bytes = flat.data_ptr(), bias_off, nflat * 2
        ops[r].x, ops[r].ldx, ops[r].y, ops[r].ldy = x.data_ptr(), IN, y.data_ptr(), OUT
    for _ in range(3):      # the counters are monotonic: repeated launches must keep working
        _lib.check(L.rtp_linear_fwd_emu(rings, ops, world, _lib.stream_ptr()), "fwd_emu")
    torch.cuda.synchronize()
    _status_ok(wss, L, _lib)
    for r in range(world):
        _close(ys[r], xs[r].float() @ full_w.float().t() + full_b.float(), 1.5e-2, f"fwd rank {r}")
    bops = (_lib.LinearBwd * world)()
    dys, dxs, gfs, keep = [], [], [], []
    for r in range(world):
        dy = torch.randn(M, OUT, device="cuda", dtype=BF) * 0.1
        dx = torch.zeros(M, IN, device="cuda", dtype=BF)
        gf = torch.zeros(nflat, device="cuda", dtype=BF)
        db = K.colsum(dy)
        dys.append(dy); dxs.append(dx); gfs.append(gf); keep.append(db)
        bops[r].mode, bops[r].M, bops[r].in_features, bops[r].out_features = mode, M, IN, OUT
        bops[r].home, bops[r].bias_off, bops[r].shard_bytes = homes[r].data_ptr(), bias_off, nflat * 2
        bops[r].x, bops[r].ldx, bops[r].dy, bops[r].ldy = xs[r].data_ptr(), IN, dy.data_ptr(), OUT
        bops[r].dx, bops[r].lddx = dx.data_ptr(), IN
        bops[r].grad_home, bops[r].dbias_full = gf.data_ptr(), db.data_ptr()
    for _ in range(2):
        _lib.check(L.rtp_linear_bwd_emu(rings, bops, world, _lib.stream_ptr()), "bwd_emu")
    torch.cuda.synchronize()
    _status_ok(wss, L, _lib)
    gw_full = sum(dys[r].float().t() @ xs[r].float() for r in range(world))
    gb_full = sum(dys[r].float().sum(0) for r in range(world))
    for r in range(world):
        _close(dxs[r], dys[r].float() @ full_w.float(), 1.5e-2, f"dx rank {r}")
        w = gfs[r][:Os * Ks].view(Os, Ks)
        b = gfs[r][bias_off:bias_off + Os]
        if mode == 0:
            _close(w, gw_full[r * Os:(r + 1) * Os], 2e-2, "dW")
            _close(b, gb_full[r * Os:(r + 1) * Os], 2e-2, "db")
        else:
            _close(w, gw_full[:, r * Ks:(r + 1) * Ks], 2e-2, "dW")
            _close(b, gb_full, 2e-2, "db")
    for w in wss:
        L.rtp_ws_destroy(w)


@pytest.mark.parametrize("world", [2, 4])
def test_rotated_embedding_and_reduce_scatter(world):
    from rtp_b200.ops import _lib
    L = _lib.lib()
    torch.manual_seed(0)
    V, D, S, B = 1000, 512, 32, 8
    Ds, T, G_ = D // world, S * B, 148 // world
    table = torch.randn(V, D, device="cuda", dtype=BF)
    pe = torch.randn(64, D, device="cuda", dtype=BF)
    slot_bytes = (V * Ds * 2 + 65535) // 65536 * 65536
    wss, rings = _rings(world, slot_bytes, G_, L, _lib)
    ops = (_lib.EmbedFwd * world)()
    keep, idss, outs = [], [], []
    for r in range(world):
        home = table[:, r * Ds:(r + 1) * Ds].contiguous()
        ids = torch.randint(0, V, (T,), device="cuda")
        out = torch.zeros(T, D, device="cuda", dtype=BF)
        keep.append(home); idss.append(ids); outs.append(out)
        ops[r].home, ops[r].shard_bytes = home.data_ptr(), V * Ds * 2
        ops[r].V, ops[r].Ds, ops[r].D = V, Ds, D
        ops[r].ids, ops[r].T = ids.data_ptr(), T
        ops[r].out, ops[r].ld_out, ops[r].scale = out.data_ptr(), D, 3.0
        ops[r].pe, ops[r].ld_pe, ops[r].tokens_per_pos = pe.data_ptr(), D, B
    for _ in range(3):
        _lib.check(L.rtp_embed_fwd_rot_emu(rings, ops, world, _lib.stream_ptr()), "embed emu")
    torch.cuda.synchronize()
    _status_ok(wss, L, _lib)
    for r in range(world):
        ref = table[idss[r]].float() * 3.0 + pe[:S].float().repeat_interleave(B, 0)
        _close(outs[r], ref, 1e-2, f"embedding rank {r}")
    rops = (_lib.ReduceScatter * world)()
    srcs, routs = [], []
    for r in range(world):
        src = torch.randn(V, D, device="cuda", dtype=BF)
        o = torch.zeros(V, Ds, device="cuda", dtype=BF)
        srcs.append(src); routs.append(o)
        rops[r].src, rops[r].ld, rops[r].rows, rops[r].cols, rops[r].out = src.data_ptr(), D, V, Ds, o.data_ptr()
    for _ in range(2):
        _lib.check(L.rtp_reduce_scatter_cols_emu(rings, rops, world, _lib.stream_ptr()), "rs emu")
    torch.cuda.synchronize()
    _status_ok(wss, L, _lib)
    tot = sum(s.float() for s in srcs)
    for r in range(world):
        _close(routs[r], tot[:, r * Ds:(r + 1) * Ds], 2e-2, f"reduce-scatter rank {r}")
    # the same reduction as ONE hop: block-major contributions go straight to their owners (gradient of the embedding);
    # mixed with the ring version above on the same gradient slots, repeated so that credits and fills interleave
    from rtp_b200.ops import kernels as K
    bops = (_lib.ReduceBlocks * world)()
    blocks, bouts, dys = [], [], []
    for r in range(world):
        dy = torch.randn(T, D, device="cuda", dtype=BF)
        blk = torch.zeros(world, V, Ds, device="cuda", dtype=BF)
        K.embed_bwd_blocks(blk, idss[r], dy, scale=2.0)
        o = torch.zeros(V, Ds, device="cuda", dtype=BF)
        blocks.append(blk); bouts.append(o); dys.append(dy)
        bops[r].src, bops[r].block_elems, bops[r].out = blk.data_ptr(), V * Ds, o.data_ptr()
    for _ in range(3):
        _lib.check(L.rtp_reduce_blocks_emu(rings, bops, world, _lib.stream_ptr()), "reduce blocks emu")
    torch.cuda.synchronize()
    _status_ok(wss, L, _lib)
    dense = torch.zeros(V, D, device="cuda")
    for r in range(world):
        dense.index_add_(0, idss[r], dys[r].float() * 2.0)
    for r in range(world):
        _close(bouts[r], dense[:, r * Ds:(r + 1) * Ds], 3e-2, f"one-hop reduce rank {r}")
    for w in wss:
        L.rtp_ws_destroy(w)


def test_missing_producer_times_out_and_returns():
    """A rank whose peer never runs must not hang: the bounded wait expires, the kernel returns, the status word
    says which wait gave up and the context stays usable."""
    from rtp_b200.ops import _lib
    L = _lib.lib()
    torch.manual_seed(0)
    world, M, IN, OUT = 2, 128, 256, 256
    Os, Ks = OUT // world, IN
    nflat = Os * Ks + 128
    slot_bytes = 1 << 17
    wss, rings = _rings(world, slot_bytes, 8, L, _lib)
    rings[0].timeout_ns = 200_000_000      # 0.2 s
    flat = torch.zeros(nflat, device="cuda", dtype=BF)
    x = torch.randn(M, IN, device="cuda", dtype=BF)
    y = torch.zeros(M, OUT, device="cuda", dtype=BF)
    op = _lib.LinearFwd()
    op.mode, op.M, op.in_features, op.out_features = 0, M, IN, OUT
    op.home, op.bias_off, op.shard_bytes = flat.data_ptr(), Os * Ks, nflat * 2
    op.x, op.ldx, op.y, op.ldy = x.data_ptr(), IN, y.data_ptr(), OUT
    # only rank 0's kernel is launched; nothing ever fills its slot
    _lib.check(L.rtp_linear_fwd(C.byref(rings[0]), C.byref(op), _lib.stream_ptr()), "fwd")
    torch.cuda.synchronize()
    st = C.c_ulonglong(0)
    L.rtp_ws_status(wss[0], C.byref(st), _lib.stream_ptr())
    assert st.value == 2, st.value           # "wait for a peer's data timed out"
    z = torch.ones(4, device="cuda").sum().item()
    assert z == 4.0                          # the context is alive
    for w in wss:
        L.rtp_ws_destroy(w)


def test_serialised_mode_names_the_launch_whose_wait_ran_out():
    """Bisect mode: with ``set_serialize(True)`` every launch is followed by a synchronise and a status read, so the
    exception carries the name of the launch whose bounded wait expired (again a peer that is never launched)."""
    from rtp_b200.ops import _lib
    L = _lib.lib()
    world, M, IN, OUT = 2, 128, 256, 256
    Os, Ks = OUT // world, IN
    nflat = Os * Ks + 128
    wss, rings = _rings(world, 1 << 17, 8, L, _lib)
    rings[0].timeout_ns = 200_000_000      # 0.2 s
    flat = torch.zeros(nflat, device="cuda", dtype=BF)
    x = torch.randn(M, IN, device="cuda", dtype=BF)
    y = torch.zeros(M, OUT, device="cuda", dtype=BF)
    op = _lib.LinearFwd()
    op.mode, op.M, op.in_features, op.out_features = 0, M, IN, OUT
    op.home, op.bias_off, op.shard_bytes = flat.data_ptr(), Os * Ks, nflat * 2
    op.x, op.ldx, op.y, op.ldy = x.data_ptr(), IN, y.data_ptr(), OUT

    def read_status():
        st = C.c_ulonglong(0)
        L.rtp_ws_status(wss[0], C.byref(st), _lib.stream_ptr())
        if st.value:
            raise _lib.RotationTimeout(_lib.STATUS_NAMES.get(st.value, str(st.value)))

    _lib._after_launch_hooks.append(read_status)
    old = _lib.set_serialize(True)
    try:
        with pytest.raises(_lib.RotationTimeout, match="forward of layer 3.*peer's data"):
            _lib.check(L.rtp_linear_fwd(C.byref(rings[0]), C.byref(op), _lib.stream_ptr()), "forward of layer 3")
    finally:
        _lib.set_serialize(old)
        _lib._after_launch_hooks.remove(read_status)
    assert torch.ones(4, device="cuda").sum().item() == 4.0      # the context is alive
    for w in wss:
        L.rtp_ws_destroy(w)


@pytest.mark.parametrize("world,L", [(2, 2), (4, 1), (4, 2)])
def test_rotating_experts_fwd_bwd(world, L):
    """One linear of every expert while the expert blocks rotate: tokens of expert g only ever meet weights of g."""
    from rtp_b200.ops import _lib, kernels as K
    lib = _lib.lib()
    torch.manual_seed(0)
    cap, IN, OUT = 192, 256, 512
    E = world * L
    G_ = (148 // world) & ~1
    blk_w = OUT * IN
    bias_off = blk_w
    stride = blk_w + (OUT + 63) // 64 * 64
    nflat = L * stride
    slot_bytes = (nflat * 2 + 65535) // 65536 * 65536
    wss, rings = _rings(world, slot_bytes, G_, lib, _lib)
    Ws = [(torch.randn(OUT, IN, device="cuda") * 0.05).to(BF) for _ in range(E)]
    Bs = [(torch.randn(OUT, device="cuda") * 0.1).to(BF) for _ in range(E)]
    fops = (_lib.ExpertFwd * world)()
    homes, xs, ys = [], [], []
    for r in range(world):
        flat = torch.zeros(nflat, device="cuda", dtype=BF)
        for e in range(L):
            flat[e * stride:e * stride + blk_w] = Ws[r * L + e].reshape(-1)
            flat[e * stride + bias_off:e * stride + bias_off + OUT] = Bs[r * L + e]
        x = torch.randn(E * cap, IN, device="cuda", dtype=BF)
        y = torch.zeros(E * cap, OUT, device="cuda", dtype=BF)
        homes.append(flat); xs.append(x); ys.append(y)
        o = fops[r]
        o.cap, o.n_local, o.in_features, o.out_features = cap, L, IN, OUT
        o.home, o.expert_stride, o.bias_off, o.shard_bytes = flat.data_ptr(), stride, bias_off, nflat * 2
        o.x, o.ldx, o.y, o.ldy, o.act = x.data_ptr(), IN, y.data_ptr(), OUT, 0
    for _ in range(2):
        _lib.check(lib.rtp_expert_fwd_emu(rings, fops, world, _lib.stream_ptr()), "expert fwd emu")
    torch.cuda.synchronize()
    _status_ok(wss, lib, _lib)
    for r in range(world):
        ref = torch.cat([xs[r][g * cap:(g + 1) * cap].float() @ Ws[g].float().t() + Bs[g].float() for g in range(E)])
        _close(ys[r], ref, 1.5e-2, f"expert fwd rank {r}")
    bops = (_lib.ExpertBwd * world)()
    dys, dxs, gfs, keep = [], [], [], []
    for r in range(world):
        dy = torch.randn(E * cap, OUT, device="cuda", dtype=BF) * 0.1
        dx = torch.zeros(E * cap, IN, device="cuda", dtype=BF)
        gf = torch.zeros(nflat, device="cuda", dtype=BF)
        db = torch.stack([dy[g * cap:(g + 1) * cap].float().sum(0) for g in range(E)]).contiguous()
        dys.append(dy); dxs.append(dx); gfs.append(gf); keep.append(db)
        o = bops[r]
        o.cap, o.n_local, o.in_features, o.out_features = cap, L, IN, OUT
        o.home, o.expert_stride, o.bias_off, o.shard_bytes = homes[r].data_ptr(), stride, bias_off, nflat * 2
        o.x, o.ldx, o.dy, o.ldy = xs[r].data_ptr(), IN, dy.data_ptr(), OUT
        o.dx, o.lddx, o.grad_home, o.dbias_full = dx.data_ptr(), IN, gf.data_ptr(), db.data_ptr()
    for _ in range(2):
        _lib.check(lib.rtp_expert_bwd_emu(rings, bops, world, _lib.stream_ptr()), "expert bwd emu")
    torch.cuda.synchronize()
    _status_ok(wss, lib, _lib)
    for r in range(world):
        ref_dx = torch.cat([dys[r][g * cap:(g + 1) * cap].float() @ Ws[g].float() for g in range(E)])
        _close(dxs[r], ref_dx, 1.5e-2, f"expert dx rank {r}")
        for e in range(L):
            g = r * L + e
            gw = sum(dys[q][g * cap:(g + 1) * cap].float().t() @ xs[q][g * cap:(g + 1) * cap].float() for q in range(world))
            gb = sum(dys[q][g * cap:(g + 1) * cap].float().sum(0) for q in range(world))
            _close(gfs[r][e * stride:e * stride + blk_w].view(OUT, IN), gw, 2e-2, f"expert dW rank {r} e {e}")
            _close(gfs[r][e * stride + bias_off:e * stride + bias_off + OUT], gb, 2e-2, f"expert db rank {r} e {e}")
    for w in wss:
        lib.rtp_ws_destroy(w)


@pytest.mark.parametrize("world", [2, 4])
def test_cross_launch_prefetch_chain(world):
    """Two rotated linears chained A -> B -> B' (backward of B) -> A': every launch reads one weight-slot bank, filled
    by the launch before it, and pushes the next launch's shards into the other bank.  Repeated twice: the counters of
    both banks must stay consistent from step to step."""
    from rtp_b200.ops import _lib, kernels as K
    L = _lib.lib()
    torch.manual_seed(0)
    M, D, H = 512, 1024, 2048
    G_ = 148 // world

    def shard(full_w, full_b, r):
        Os, Ks = full_w.shape[0] // world, full_w.shape[1]
        bias_off = Os * Ks
        flat = torch.zeros(bias_off + Os, device="cuda", dtype=BF)
        flat[:bias_off] = full_w[r * Os:(r + 1) * Os].reshape(-1)
        flat[bias_off:] = full_b[r * Os:(r + 1) * Os]
        return flat, bias_off

    wa = (torch.randn(H, D, device="cuda") * 0.05).to(BF); ba = (torch.randn(H, device="cuda") * 0.1).to(BF)
    wb = (torch.randn(D, H, device="cuda") * 0.05).to(BF); bb = (torch.randn(D, device="cuda") * 0.1).to(BF)
    slot_bytes = ((H * D // world + H) * 2 + 65535) // 65536 * 65536
    wss, rings = _rings(world, slot_bytes, G_, L, _lib)
    fa, fb = [shard(wa, ba, r) for r in range(world)], [shard(wb, bb, r) for r in range(world)]
    xs = [torch.randn(M, D, device="cuda", dtype=BF) for _ in range(world)]
    hs = [torch.zeros(M, H, device="cuda", dtype=BF) for _ in range(world)]
    ys = [torch.zeros(M, D, device="cuda", dtype=BF) for _ in range(world)]
    dys = [torch.randn(M, D, device="cuda", dtype=BF) for _ in range(world)]
    dhs = [torch.zeros(M, H, device="cuda", dtype=BF) for _ in range(world)]
    dxs = [torch.zeros(M, D, device="cuda", dtype=BF) for _ in range(world)]
    ga = [torch.zeros_like(f[0]) for f in fa]; gb = [torch.zeros_like(f[0]) for f in fb]
    A, B = (_lib.LinearFwd * world)(), (_lib.LinearFwd * world)()
    Bb, Ab = (_lib.LinearBwd * world)(), (_lib.LinearBwd * world)()
    for r in range(world):
        for op, (flat, boff), x, y, inf, outf in ((A[r], fa[r], xs[r], hs[r], D, H), (B[r], fb[r], hs[r], ys[r], H, D)):
            op.mode, op.M, op.in_features, op.out_features = 0, M, inf, outf
            op.home, op.bias_off, op.shard_bytes = flat.data_ptr(), boff, flat.numel() * 2
            op.x, op.ldx, op.y, op.ldy = x.data_ptr(), inf, y.data_ptr(), outf
        A[r].bank, A[r].no_self_push = 0, 0
        A[r].next_home, A[r].next_bytes, A[r].next_kind = fb[r][0].data_ptr(), fb[r][0].numel() * 2, 0
        B[r].bank, B[r].no_self_push = 1, 1
        B[r].next_home, B[r].next_bytes, B[r].next_kind = fb[r][0].data_ptr(), fb[r][0].numel() * 2, 1
        for op, (flat, boff), x, dy, dx, g, inf, outf in ((Bb[r], fb[r], hs[r], dys[r], dhs[r], gb[r], H, D),
                                                           (Ab[r], fa[r], xs[r], dhs[r], dxs[r], ga[r], D, H)):
            op.mode, op.M, op.in_features, op.out_features = 0, M, inf, outf
            op.home, op.bias_off, op.shard_bytes = flat.data_ptr(), boff, flat.numel() * 2
            op.x, op.ldx, op.dy, op.ldy = x.data_ptr(), inf, dy.data_ptr(), outf
            op.dx, op.lddx, op.grad_home = dx.data_ptr(), inf, g.data_ptr()
        Bb[r].bank, Bb[r].no_self_push = 0, 1
        Bb[r].next_home, Bb[r].next_bytes, Bb[r].next_kind = fa[r][0].data_ptr(), fa[r][0].numel() * 2, 1
        Ab[r].bank, Ab[r].no_self_push = 1, 1
    for _ in range(2):
        _lib.check(L.rtp_linear_fwd_emu(rings, A, world, _lib.stream_ptr()), "A")
        _lib.check(L.rtp_linear_fwd_emu(rings, B, world, _lib.stream_ptr()), "B")
        _lib.check(L.rtp_linear_bwd_emu(rings, Bb, world, _lib.stream_ptr()), "B'")
        _lib.check(L.rtp_linear_bwd_emu(rings, Ab, world, _lib.stream_ptr()), "A'")
    torch.cuda.synchronize()
    _status_ok(wss, L, _lib)
    dwa = torch.zeros(H, D, device="cuda"); dwb = torch.zeros(D, H, device="cuda")
    for r in range(world):
        h = xs[r].float() @ wa.float().t() + ba.float()
        _close(hs[r], h, 1.5e-2, f"A rank {r}")
        hb = hs[r].float()
        _close(ys[r], hb @ wb.float().t() + bb.float(), 1.5e-2, f"B rank {r}")
        dh = dys[r].float() @ wb.float()
        _close(dhs[r], dh, 2e-2, f"B' dx rank {r}")
        _close(dxs[r], dhs[r].float() @ wa.float(), 2e-2, f"A' dx rank {r}")
        dwb += dys[r].float().t() @ hb
        dwa += dhs[r].float().t() @ xs[r].float()
    for r in range(world):
        Os = D // world
        _close(gb[r][:Os * H].view(Os, H), dwb[r * Os:(r + 1) * Os], 3e-2, f"B' dW rank {r}")
        Os = H // world
        _close(ga[r][:Os * D].view(Os, D), dwa[r * Os:(r + 1) * Os], 3e-2, f"A' dW rank {r}")
    for w in wss:
        L.rtp_ws_destroy(w)
