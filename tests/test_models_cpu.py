"""GPT-, Llama- and MoE-shaped rotated LMs on gloo rings vs the same model on a 1-rank ring (the unsharded oracle),
with the weights moved between the two through the generic checkpoint tools (consolidated <-> sharded)."""
import pytest
import torch

from _dist import run_distributed


def _self_group(rank, world):
    import torch.distributed as dist
    groups = [dist.new_group([r]) for r in range(world)]   # every rank must take part in every new_group call
    return groups[rank]


def _compare(rank, world, build, batch_first=True):
    from rtp_b200.checkpoint import shard_full, sharding_plan, consolidate
    from rtp_b200.optim import sync_replicated_grads
    solo = _self_group(rank, world)
    torch.manual_seed(0)
    full = build(solo)                     # identical on every rank
    model = build(None)                    # sharded over the world ring
    plan = sharding_plan(model)
    model.load_state_dict(shard_full(full.state_dict(), plan, rank, world))
    torch.manual_seed(1)
    B, S = 2 * world, 12
    ids = torch.randint(0, 64, (B, S + 1))
    x, y = ids[:, :-1], ids[:, 1:]
    loss_full = full(x, y)
    loss_full.backward()
    sl = slice(2 * rank, 2 * rank + 2)
    logits = model(x[sl])
    assert torch.allclose(logits, full(x)[sl].detach(), atol=2e-5), (logits - full(x)[sl]).abs().max()
    loss = model(x[sl], y[sl])
    (loss / world).backward()
    sync_replicated_grads(model.parameters())
    # gather every rank's state/grad dict and compare the consolidated gradients with the oracle's
    import torch.distributed as dist
    grads = {n: p.grad for n, p in model.named_parameters()}
    gathered = [None] * world
    dist.all_gather_object(gathered, {k: v.clone() for k, v in grads.items()})
    cons = consolidate(gathered, plan)
    fgr = {n: p.grad for n, p in full.named_parameters()}
    for n, g in cons.items():
        ref = fgr[n]
        if plan.get(n, (None,))[0] == "sum":
            g = g / world          # consolidate multiplies b/N shards by N; the gradient needs no such factor
        assert torch.allclose(g, ref, atol=5e-5, rtol=1e-4), (n, (g - ref).abs().max().item())


def _gpt(rank, world):
    from rtp_b200.models.gpt import GPT, GPTConfig
    cfg = GPTConfig(vocab_size=64, d_model=32, n_layers=2, n_heads=4, d_ff=64, max_seq_len=16)
    _compare(rank, world, lambda g: GPT(cfg, group=g))


def _llama(rank, world):
    from rtp_b200.models.llama import Llama, LlamaConfig
    cfg = LlamaConfig(vocab_size=64, d_model=32, n_layers=2, n_heads=4, d_ff=64, max_seq_len=16)
    _compare(rank, world, lambda g: Llama(cfg, group=g))


def _moe(rank, world):
    import rtp_b200.module.top2gate as tg
    from rtp_b200.checkpoint import shard_full, sharding_plan
    from rtp_b200.models.moe_lm import MoELM, MoEConfig
    tg.gumbel_rsample = lambda shape, device: torch.zeros(shape, device=device)
    cfg = MoEConfig(vocab_size=64, d_model=32, n_layers=2, n_heads=4, d_ff=64, n_experts=4, max_seq_len=16)
    solo = _self_group(rank, world)
    torch.manual_seed(0)
    full = MoELM(cfg, group=solo)
    model = MoELM(cfg)
    model.load_state_dict(shard_full(full.state_dict(), sharding_plan(model), rank, world))
    torch.manual_seed(1)
    ids = torch.randint(0, 64, (2, 9))       # the same tokens on every rank, as in the reference's MoE test
    x, y = ids[:, :-1], ids[:, 1:]
    assert torch.allclose(model(x), full(x).detach(), atol=2e-5)
    loss = model(x, y)
    loss.backward()
    assert all(torch.isfinite(p.grad).all() for p in model.parameters() if p.grad is not None)
    assert abs(loss.item() - full(x, y).item()) < 1e-5


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("case", [_gpt, _llama, _moe])
def test_model_family(case, world):
    run_distributed(case, world)


def _chunked_loss(rank, world):
    """LM head + cross-entropy chunk by chunk (no full logits) against the plain path: same loss, same gradients,
    on a rotated head."""
    import copy
    from rtp_b200.models.gpt import GPT, GPTConfig
    torch.manual_seed(0)
    cfg = GPTConfig(vocab_size=64, d_model=32, n_layers=1, n_heads=4, d_ff=64, max_seq_len=16)
    plain = GPT(cfg)
    chunked = copy.deepcopy(plain)
    chunked.cfg = GPTConfig(vocab_size=64, d_model=32, n_layers=1, n_heads=4, d_ff=64, max_seq_len=16, loss_chunk_rows=5)
    torch.manual_seed(1 + rank)
    ids = torch.randint(0, 64, (2, 13))
    x, y = ids[:, :-1], ids[:, 1:].clone()
    y[0, 0] = -100
    l0 = plain(x, y)
    (l0 * 0.5).backward()
    l1 = chunked(x, y)
    (l1 * 0.5).backward()
    assert abs(l0.item() - l1.item()) < 1e-6, (l0.item(), l1.item())
    for (n, p), q in zip(plain.named_parameters(), chunked.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6, rtol=1e-5), (n, (p.grad - q.grad).abs().max().item())


@pytest.mark.parametrize("world", [1, 2])
def test_chunked_head_loss_matches_the_plain_path(world):
    run_distributed(_chunked_loss, world)
