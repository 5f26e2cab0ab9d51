"""Worker of the multi-GPU tests (one process per GPU, launched by torchrun).

Every case compares the fused sm_100a path AND the functional NCCL path (both bf16) with an fp32 oracle computed from
the unsharded weights and the gathered inputs of all ranks: the fused error must stay within twice the functional
error (plus a small floor), and no 128 x 128 tile of a gradient may be off by more than a few percent of the tensor's
range — a stale or misplaced tile shows there, not in an average."""
import copy
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
BF = torch.bfloat16


def rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def tile_err(a, b, tile=128):
    """Largest max-abs error of any tile x tile block, relative to the range of the reference."""
    a, b = a.float(), b.float()
    if a.dim() == 1:
        a, b = a[None], b[None]
    a, b = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
    d = (a - b).abs()
    R, Cc = d.shape
    pr, pc = (-R) % tile, (-Cc) % tile
    d = F.pad(d, (0, pc, 0, pr))
    blocks = d.view((R + pr) // tile, tile, (Cc + pc) // tile, tile).amax(dim=(1, 3))
    return (blocks.max() / (b.abs().max() + 1e-12)).item()


def gather_cat(t, world, dim=0):
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous())
    return torch.cat(parts, dim=dim)


def main():
    import faulthandler
    faulthandler.dump_traceback_later(200, exit=True)   # a stuck rank prints where and exits instead of hanging
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    from rtp_b200.rotated_tensor_parallel import RotatedTensorParallel
    from rtp_b200.checkpoint import shard_state_dict
    from rtp_b200.inplace.module.attention import WeightParallelMultiheadAttention
    from rtp_b200.inplace.module.linear import WeightParallelLinear, WeightParallelRowLinear
    from rtp_b200.models.transformer_lm_fsdp import TransformerLM as PlainLM
    from rtp_b200.models.transformer_lm_rtp import TransformerLM
    from rtp_b200.models.fused_lm import FusedLMTrainer
    from rtp_b200.module.attention import ParallelMultiheadAttention
    from rtp_b200.module.embedding import ParallelEmbedding
    from rtp_b200.module.linear import ColumnParallelLinear, RowParallelLinear
    from rtp_b200.ops import _lib
    from rtp_b200.optim import ShardedAdam
    from rtp_b200.parallel import engine
    from rtp_b200.parallel.context import get_context, set_backend
    dev = torch.device("cuda", local)
    fails = []

    def check(cond, msg):
        if not cond:
            fails.append(msg)
            print(f"[rank {rank}] FAIL {msg}", flush=True)

    def compare(name, fused, func, oracle, floor=4e-3, tiles=True):
        ef, en = rel_err(fused, oracle), rel_err(func, oracle)
        check(ef <= 2 * en + floor, f"{name}: fused error {ef:.4g} vs functional {en:.4g} (fp32 oracle)")
        if tiles:
            te = tile_err(fused, oracle)
            check(te <= 0.06, f"{name}: worst 128x128 tile off by {te:.3g} of the range")

    def zero_grads(m):
        for p in m.parameters():
            p.grad = None

    def fused_ran(before, what):
        check(_lib.launches > before, f"{what}: no library kernel was launched (fell back to the functional engine)")

    # ------------------------------------------------------------------ rotated linears (out-of-place and in-place)
    for cls, row in ((ColumnParallelLinear, False), (RowParallelLinear, True), (WeightParallelLinear, False),
                     (WeightParallelRowLinear, True)):
        torch.manual_seed(0)
        full = torch.nn.Linear(512, 1024).to(dev).to(BF)
        m = cls(512, 1024, linear_layer=full, device=dev, dtype=BF)
        torch.manual_seed(100 + rank)
        x = torch.randn(200, 512, device=dev, dtype=BF, requires_grad=True)
        dy = torch.randn(200, 1024, device=dev, dtype=BF)
        # fp32 oracle from the unsharded layer and every rank's data
        xa, dya = gather_cat(x.detach(), world), gather_cat(dy, world)
        Wf, bf_ = full.weight.float(), full.bias.float()
        y_or = x.detach().float() @ Wf.t() + bf_
        dx_or = dy.float() @ Wf
        dW_or = dya.float().t() @ xa.float()
        db_or = dya.float().sum(0)
        if row:
            dW_sh, db_sh = dW_or.chunk(world, dim=1)[rank], db_or
        else:
            dW_sh, db_sh = dW_or.chunk(world, dim=0)[rank], db_or.chunk(world)[rank]
        set_backend("functional")
        yf = m(x)
        yf.backward(dy)
        gw_f, gb_f, gx_f = m.linear.weight.grad.clone(), m.linear.bias.grad.clone(), x.grad.clone()
        zero_grads(m)
        x.grad = None
        set_backend("auto")
        for rep in range(2):
            n0 = _lib.launches
            y = m(x)
            y.backward(dy)
            engine.check_all()
            _lib.check_status(dev)
            fused_ran(n0, cls.__name__)
            compare(f"{cls.__name__} y rep {rep}", y, yf, y_or)
            compare(f"{cls.__name__} dx", x.grad, gx_f, dx_or)
            compare(f"{cls.__name__} dW", m.linear.weight.grad, gw_f, dW_sh)
            compare(f"{cls.__name__} db", m.linear.bias.grad, gb_f, db_sh, tiles=False)
            zero_grads(m)
            x.grad = None
        if getattr(m, "inplace", False):
            # a forward without grad leaves every shard at home; two in a row give the same result
            with torch.no_grad():
                y1, y2 = m(x), m(x)
            check(torch.equal(y1, y2) and not m._displaced, f"{cls.__name__}: repeated no-grad forwards differ")
            compare(f"{cls.__name__} no-grad y", y1, yf, y_or)

    # ------------------------------------------------------------------ a head whose width the kernels cannot take
    torch.manual_seed(1)
    full10 = torch.nn.Linear(64, 10 * world).to(dev).to(BF)
    m10 = ColumnParallelLinear(64, 10 * world, linear_layer=full10, device=dev, dtype=BF)
    x10 = torch.randn(16, 64, device=dev, dtype=BF, requires_grad=True)
    y10 = m10(x10)
    y10.sum().backward()            # must not raise in the middle of backward
    check(rel_err(y10, x10.detach().float() @ full10.weight.float().t() + full10.bias.float()) < 2e-2, "10-column head")

    # ------------------------------------------------------------------ embedding (gather + reduce-scatter of the gradient)
    torch.manual_seed(2)
    V, Dm = 512, 256
    femb = nn.Embedding(V, Dm).to(dev).to(BF)
    emb = ParallelEmbedding(V, Dm, Embedding_layer=femb, device=dev, dtype=BF)
    torch.manual_seed(200 + rank)
    ids = torch.randint(0, V, (40, 8), device=dev)
    dE = torch.randn(40, 8, Dm, device=dev, dtype=BF)
    ids_a, dE_a = gather_cat(ids, world), gather_cat(dE, world)
    g_or = torch.zeros(V, Dm, device=dev).index_add_(0, ids_a.reshape(-1), dE_a.reshape(-1, Dm).float())
    set_backend("functional")
    ef = emb(ids)
    ef.backward(dE)
    ge_f = emb.embedding.weight.grad.clone()
    zero_grads(emb)
    set_backend("auto")
    n0 = _lib.launches
    e = emb(ids)
    e.backward(dE)
    engine.check_all()
    fused_ran(n0, "ParallelEmbedding")
    check(torch.equal(e, ef), "embedding forward differs from the functional path")
    compare("embedding dW", emb.embedding.weight.grad, ge_f, g_or.chunk(world, dim=1)[rank], floor=1e-2)

    # ------------------------------------------------------------------ attention: causal, masks, dropout, in-place
    torch.manual_seed(3)
    E_, H_ = 512, 8
    fmha = nn.MultiheadAttention(E_, H_, dropout=0.0).to(dev).to(BF)
    for cls in (ParallelMultiheadAttention, WeightParallelMultiheadAttention):
        for L_, kind in ((32, "causal"), (160, "causal"), (160, "kpm"), (96, "mask")):
            mha = cls(E_, H_, MultiheadAttention_layer=fmha, device=dev, dtype=BF)
            torch.manual_seed(300 + rank)
            xq = torch.randn(L_, 4, E_, device=dev, dtype=BF, requires_grad=True)
            dyq = torch.randn(L_, 4, E_, device=dev, dtype=BF)
            kw = dict(need_weights=False)
            if kind == "causal":
                kw["attn_mask"] = torch.full((L_, L_), float("-inf"), device=dev).triu_(1)
            elif kind == "mask":
                mk = torch.rand(L_, L_, device=dev) < 0.3
                mk[:, 0] = False
                kw["attn_mask"] = mk
            else:
                kp = torch.zeros(4, L_, dtype=torch.bool, device=dev)
                kp[:, L_ - 9:] = True
                kw["key_padding_mask"] = kp
            # fp32 oracle: torch's own attention on the unsharded layer
            f32 = copy.deepcopy(fmha).float()
            xr = xq.detach().float().requires_grad_(True)
            yr = f32(xr, xr, xr, **kw)[0]
            yr.backward(dyq.float())
            set_backend("functional")
            yf = mha(xq, xq, xq, **kw)[0]
            yf.backward(dyq)
            gx_f = xq.grad.clone()
            gin_f = mha.MultiheadAttention.in_proj_weight.grad.clone()
            zero_grads(mha)
            xq.grad = None
            set_backend("auto")
            n0 = _lib.launches
            yk = mha(xq, xq, xq, **kw)[0]
            yk.backward(dyq)
            engine.check_all()
            _lib.check_status(dev)
            fused_ran(n0, f"{cls.__name__} {kind}")
            compare(f"{cls.__name__} L{L_} {kind} y", yk, yf, yr.detach(), floor=1e-2)
            compare(f"{cls.__name__} L{L_} {kind} dx", xq.grad, gx_f, xr.grad, floor=1.5e-2)
            # in_proj gradient of the full layer needs every rank's batch: compare with the functional path
            e_in = rel_err(mha.MultiheadAttention.in_proj_weight.grad, gin_f)
            check(e_in < 3e-2, f"{cls.__name__} L{L_} {kind} d(in_proj): {e_in:.4g} vs functional")
    # training dropout stays on the kernels and really drops
    mha = ParallelMultiheadAttention(E_, H_, dropout=0.2, MultiheadAttention_layer=fmha, device=dev, dtype=BF)
    mha.train()
    xq = torch.randn(64, 4, E_, device=dev, dtype=BF, requires_grad=True)
    n0 = _lib.launches
    ya = mha(xq, xq, xq, need_weights=False, is_causal=True)[0]
    ya.sum().backward()
    fused_ran(n0, "attention with dropout")
    mha.eval()
    yb = mha(xq, xq, xq, need_weights=False, is_causal=True)[0]
    check((ya.float() - yb.float()).abs().max().item() > 1e-2 and torch.isfinite(xq.grad.float()).all().item(),
          "attention dropout had no effect or produced non-finite gradients")
    # attention weights of the last visiting shard (the reference's return value)
    yw, w = mha(xq, xq, xq, need_weights=True, is_causal=True)
    check(w is not None and tuple(w.shape) == (4, 64, 64) and abs(w.float().sum(-1).mean().item() - 1.0) < 2e-2,
          "need_weights: probabilities missing or not normalised")

    # ------------------------------------------------------------------ RotatedTensorParallel(model) on the kernels
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv1 = nn.Conv2d(1, 32, 3, 1)
            self.conv2 = nn.Conv2d(32, 64, 3, 1)
            self.fc1 = nn.Linear(64 * 12 * 12, 128)
            self.fc2 = nn.Linear(128, 16)

        def forward(self, x):
            # smooth activations: with ReLU / max-pooling two bf16 pipelines flip masks near zero and their gradients
            # differ by far more than rounding, which would hide what this case is about (the plumbing of the wrapper)
            x = torch.tanh(self.conv1(x))
            x = F.avg_pool2d(torch.tanh(self.conv2(x)), 2)
            return self.fc2(torch.tanh(self.fc1(torch.flatten(x, 1))))

    torch.manual_seed(4)
    net = Net().to(dev).to(BF)
    ref32 = copy.deepcopy(net).float()
    torch.manual_seed(400 + rank)
    img = torch.randn(32, 1, 28, 28, device=dev, dtype=BF)
    tgt = torch.randint(0, 16, (32,), device=dev)
    # fp32 oracle on the global batch
    img_a, tgt_a = gather_cat(img, world), gather_cat(tgt, world)
    lo = F.cross_entropy(ref32(img_a.float()), tgt_a, reduction="sum") / 32
    lo.backward()
    for inplace in (False, True):
        wrapped = RotatedTensorParallel(copy.deepcopy(net), inplace=inplace)
        res = {}
        for be in ("functional", "auto"):
            set_backend(be)
            zero_grads(wrapped)
            n0 = _lib.launches
            out = wrapped(img)
            (F.cross_entropy(out.float(), tgt, reduction="sum") / 32).backward()
            engine.check_all()
            if be == "auto":
                fused_ran(n0, f"RotatedTensorParallel(inplace={inplace})")
            res[be] = (out.detach().clone(), {n: p.grad.clone() for n, p in wrapped.named_parameters()})
        set_backend("auto")
        out_or = ref32(img.float())
        compare(f"wrapper(inplace={inplace}) logits", res["auto"][0], res["functional"][0], out_or.detach(), floor=1e-2)
        full_g = {n: p.grad for n, p in ref32.named_parameters()}
        for n, g in res["auto"][1].items():
            base = n.replace("module.", "")
            fg = full_g[base]
            if g.shape != fg.shape:                      # a shard: cut the oracle the same way
                dim = [i for i, (a_, b_) in enumerate(zip(g.shape, fg.shape)) if a_ != b_][0]
                fg = fg.chunk(world, dim=dim)[rank]
            compare(f"wrapper(inplace={inplace}) grad {n}", g, res["functional"][1][n], fg, floor=1.5e-2,
                  tiles=g.dim() == 2)

    # ------------------------------------------------------------------ whole LM: fused trainer and module path vs fp32 oracle
    V, D, H, NH, L, S, B = 1024, 512, 1024, 8, 2, 32, 8
    torch.manual_seed(0)
    full = PlainLM(V, D, NH, H, 0.0, 0.1, L)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in full.parameters():
            if p.dim() > 1:
                p.copy_(torch.rand(p.shape, generator=g) * 0.2 - 0.1)
    model = TransformerLM(V, D, NH, H, 0.0, 0.1, L, world, rank)
    model.load_state_dict(shard_state_dict(full.state_dict(), model, rank, world))
    model = model.to(device=dev, dtype=BF)
    ref = copy.deepcopy(model)
    mod = copy.deepcopy(model)
    gd = torch.Generator().manual_seed(7)
    stream = torch.randint(0, V, (S + 1, B * world), generator=gd)
    x = stream[:-1, rank * B:(rank + 1) * B].contiguous().to(dev)
    y = stream[1:, rank * B:(rank + 1) * B].contiguous().to(dev)
    # oracle: the plain model in fp32 on the whole batch (bf16-rounded weights, as every rank holds them)
    full32 = copy.deepcopy(full).to(dev)
    with torch.no_grad():
        for p in full32.parameters():
            p.copy_(p.to(BF).float())
    lo = F.cross_entropy(full32(stream[:-1].to(dev)).view(-1, V), stream[1:].to(dev).reshape(-1))
    lo.backward()
    oracle_g = shard_state_dict({n: p.grad for n, p in full32.named_parameters()}, model, rank, world)
    plan_sum = {n for n, p in model.named_parameters() if getattr(p, "rtp_sum_replicated", None)}
    set_backend("functional")
    loss_f = F.cross_entropy(ref(x).view(-1, V).float(), y.view(-1))
    (loss_f / world).backward()
    set_backend("auto")
    n0 = _lib.launches
    loss_m = F.cross_entropy(mod(x).view(-1, V).float(), y.view(-1))
    (loss_m / world).backward()
    engine.check_all()
    fused_ran(n0, "TransformerLM through modules")
    tr = FusedLMTrainer(model, lr=0.0, clip_value=None, use_graph=False)
    loss = tr.step(x, y)
    tr.check()
    lo_all = torch.tensor([loss.item(), loss_m.item(), loss_f.item()], device=dev)
    dist.all_reduce(lo_all)
    lo_all /= world
    check(abs(lo_all[0].item() - lo.item()) < 2e-2, f"LM loss fused trainer {lo_all[0].item()} vs fp32 {lo.item()}")
    check(abs(lo_all[1].item() - lo.item()) < 2e-2, f"LM loss module path {lo_all[1].item()} vs fp32 {lo.item()}")
    refp, modp = dict(ref.named_parameters()), dict(mod.named_parameters())
    worst = 0.0
    for n, p in model.named_parameters():
        if "norm" in n:
            continue     # replicated: the trainer all-reduces them, plain autograd does not
        og = oracle_g[n].to(dev) * (world if n in plan_sum else 1.0)   # b/N copies receive the full bias gradient
        ef, em, en = rel_err(p.grad, og), rel_err(modp[n].grad, og), rel_err(refp[n].grad, og)
        worst = max(worst, ef, em)
        check(ef <= 2 * en + 1e-2, f"LM grad {n}: fused trainer {ef:.4g} vs functional {en:.4g} (fp32 oracle)")
        check(em <= 2 * en + 1e-2, f"LM grad {n}: module path {em:.4g} vs functional {en:.4g} (fp32 oracle)")
        if p.dim() == 2:
            # the FFN's ReLU flips masks between two bf16 pipelines, so single entries move by several percent of the
            # range; a stale or misplaced tile is off by about the whole range
            te = tile_err(p.grad, og)
            check(te <= 0.25, f"LM grad {n}: worst tile of the fused trainer off by {te:.3g} of the range")
    # ---- training: fused trainer under graph replay, and the module path with dropout + ShardedAdam
    model2 = TransformerLM(V, D, NH, H, 0.1, 0.1, L, world, rank).to(device=dev, dtype=BF)
    model3 = copy.deepcopy(model2)
    tr2 = FusedLMTrainer(model2, lr=1e-3, clip_value=0.05, use_graph=True)
    losses = [tr2.step(x, y).item() for _ in range(25)]
    tr2.check()
    check(losses[-1] < 0.5 * losses[0] and all(v == v for v in losses), f"training losses {losses[::6]}")
    opt = ShardedAdam(model3.parameters(), lr=1e-3, clip_value=0.05)
    model3.train()
    losses3 = []
    n0 = _lib.launches
    for _ in range(25):
        opt.zero_grad(set_to_none=True)
        l3 = F.cross_entropy(model3(x).view(-1, V).float(), y.view(-1))
        (l3 / world).backward()
        opt.step()
        losses3.append(l3.item())
    engine.check_all()
    fused_ran(n0, "module-path training with dropout")
    check(losses3[-1] < 0.5 * losses3[0] and all(v == v for v in losses3), f"module-path training losses {losses3[::6]}")

    # ------------------------------------------------------------------ rotate-only kernel on the real ring
    eng = engine.get_engine(get_context())
    buf = torch.full((1 << 20,), float(rank), device=dev, dtype=torch.float32)
    for step in range(1, world + 1):
        eng.shift_inplace(buf, "down")
        torch.cuda.synchronize()
        check(bool((buf == float((rank + step) % world)).all().item()), f"ring shift down, step {step}")
    eng.shift_inplace(buf, "up")
    torch.cuda.synchronize()
    check(bool((buf == float((rank - 1) % world)).all().item()), "ring shift up")
    _lib.check_status(dev)

    # ------------------------------------------------------------------ slot counters agree across the ring
    try:
        eng.verify_epochs()
    except engine.EpochMismatch as e:
        check(False, f"epoch check: {e}")
    arrive, done, uses = eng.counters()
    check(sum(uses) > 0, "the slot counters moved")

    # ------------------------------------------------------------------ serialised (bisect) mode
    old = _lib.set_serialize(True)
    try:
        lin_ser = ColumnParallelLinear(256, 256).to(dev, torch.bfloat16)
        y_ser = lin_ser(torch.randn(64, 256, device=dev, dtype=torch.bfloat16))
        check(bool(torch.isfinite(y_ser).all().item()), "serialised mode: fused linear")
    finally:
        _lib.set_serialize(old)

    dist.barrier()
    if rank == 0:
        print(f"worst LM grad rel err vs fp32 {worst:.4f}; trainer losses {[round(v, 3) for v in losses[::6]]}; "
              f"module losses {[round(v, 3) for v in losses3[::6]]}", flush=True)
    ok = torch.tensor([0 if fails else 1], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    code = 0 if ok.item() == 1 else 1
    if rank == 0:
        print("MULTI_GPU_OK" if code == 0 else "MULTI_GPU_FAILED", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    # captured graphs still reference NCCL kernels; leave without tearing the communicator down
    os._exit(code)


if __name__ == "__main__":
    main()
