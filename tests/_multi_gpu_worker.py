"""Worker of the multi-GPU tests (one process per GPU, launched by torchrun): the fused sm_100a rotation path
against the functional NCCL path on the same sharded weights."""
import copy
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
BF = torch.bfloat16


def rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def cosine(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return (torch.dot(a, b) / (a.norm() * b.norm() + 1e-20)).item()


def main():
    import faulthandler
    faulthandler.dump_traceback_later(150, exit=True)   # a stuck rank prints where and exits instead of hanging
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    from rtp_b200.checkpoint import shard_state_dict
    from rtp_b200.models.transformer_lm_fsdp import TransformerLM as PlainLM
    from rtp_b200.models.transformer_lm_rtp import TransformerLM
    from rtp_b200.models.fused_lm import FusedLMTrainer
    from rtp_b200.module.linear import ColumnParallelLinear, RowParallelLinear
    from rtp_b200.parallel import engine
    from rtp_b200.parallel.context import set_backend
    dev = torch.device("cuda", local)
    fails = []

    def check(cond, msg):
        if not cond:
            fails.append(msg)
            print(f"[rank {rank}] FAIL {msg}", flush=True)

    # ---- rotated linear modules: fused vs functional
    torch.manual_seed(0)
    for cls in (ColumnParallelLinear, RowParallelLinear):
        full = torch.nn.Linear(512, 1024).to(dev).to(BF)
        m = cls(512, 1024, linear_layer=full, device=dev, dtype=BF)
        torch.manual_seed(100 + rank)
        x = torch.randn(200, 512, device=dev, dtype=BF, requires_grad=True)
        dy = torch.randn(200, 1024, device=dev, dtype=BF)
        set_backend("functional")
        yf = m(x)
        yf.backward(dy)
        gw_f, gx_f = m.linear.weight.grad.clone(), x.grad.clone()
        m.linear.weight.grad = None
        m.linear.bias.grad = None
        x.grad = None
        set_backend("auto")
        for rep in range(2):
            y = m(x)
            y.backward(dy)
            engine.check_all()
            check(rel_err(y, yf) < 1e-2, f"{cls.__name__} forward rep {rep}: {rel_err(y, yf)}")
            check(rel_err(x.grad, gx_f) < 1e-2, f"{cls.__name__} dx: {rel_err(x.grad, gx_f)}")
            check(rel_err(m.linear.weight.grad, gw_f) < 2e-2, f"{cls.__name__} dW: {rel_err(m.linear.weight.grad, gw_f)}")
            m.linear.weight.grad = None
            m.linear.bias.grad = None
            x.grad = None

    # ---- whole LM: fused trainer vs functional autograd path
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
    gd = torch.Generator().manual_seed(7)
    stream = torch.randint(0, V, (S + 1, B * world), generator=gd)
    x = stream[:-1, rank * B:(rank + 1) * B].contiguous().to(dev)
    y = stream[1:, rank * B:(rank + 1) * B].contiguous().to(dev)
    set_backend("functional")
    loss_f = F.cross_entropy(ref(x).view(-1, V).float(), y.view(-1))
    (loss_f / world).backward()
    set_backend("auto")
    tr = FusedLMTrainer(model, lr=0.0, clip_value=None, use_graph=False)
    loss = tr.step(x, y)
    tr.check()
    check(abs(loss.item() - loss_f.item()) < 3e-2, f"LM loss fused {loss.item()} vs functional {loss_f.item()}")
    refp = dict(ref.named_parameters())
    worst = 0.0
    for n, p in model.named_parameters():
        if "norm" in n:
            continue     # replicated: the trainer all-reduces them, plain autograd does not
        # two bf16 pipelines with different rounding points: gradients (sums with cancellation) agree to a few percent
        e = rel_err(p.grad, refp[n].grad)
        worst = max(worst, e)
        check(e < 0.15 and cosine(p.grad, refp[n].grad) > 0.99, f"LM grad {n}: rel {e} cos {cosine(p.grad, refp[n].grad)}")
    # ---- training under graph replay on the ring
    model2 = TransformerLM(V, D, NH, H, 0.1, 0.1, L, world, rank).to(device=dev, dtype=BF)
    tr2 = FusedLMTrainer(model2, lr=1e-3, clip_value=0.05, use_graph=True)
    losses = [tr2.step(x, y).item() for _ in range(25)]
    tr2.check()
    check(losses[-1] < 0.5 * losses[0] and all(v == v for v in losses), f"training losses {losses[::6]}")
    dist.barrier()
    if rank == 0:
        print(f"worst LM grad rel err {worst:.4f}; losses {[round(v, 3) for v in losses[::6]]}", flush=True)
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
