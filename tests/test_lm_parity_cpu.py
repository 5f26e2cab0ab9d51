"""Trajectory parity of the rotated LM with the single-process model on CPU/gloo.

Config: fp32, vocab 1024, ninp 256, nhid 1024, nhead 8, 2 decoder layers, seq_len 32, batch 8,
ids uniform int64 from seed 0, targets = inputs shifted by one, all weights U(-0.1, 0.1), Adam lr 1e-3,
10 steps; the loss (mean over ranks) must match the single-process model to 1e-5 at every step."""
import pytest
import torch
import torch.nn.functional as F

from _dist import run_distributed

V, D, H, NH, L, S, B = 1024, 256, 1024, 8, 2, 32, 8
STEPS = 10


def _data():
    g = torch.Generator().manual_seed(0)
    stream = torch.randint(0, V, (S + 1, B), generator=g, dtype=torch.int64)
    return stream[:-1], stream[1:]


def _reference_losses():
    from rtp_b200.models.transformer_lm_fsdp import TransformerLM
    torch.manual_seed(0)
    model = TransformerLM(V, D, NH, H, 0.0, 0.1, L)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in model.parameters():
            p.copy_(torch.rand(p.shape, generator=g) * 0.2 - 0.1)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    x, y = _data()
    losses = []
    for _ in range(STEPS):
        opt.zero_grad()
        loss = F.cross_entropy(model(x).view(-1, V), y.reshape(-1))
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return model, losses


def _load_from_full(rtp_model, full_model, rank, world):
    """Shard the single-process weights into the rotated model (sharding rules of the reference)."""
    from rtp_b200.checkpoint import shard_state_dict
    sd = shard_state_dict(full_model.state_dict(), rtp_model, rank, world)
    rtp_model.load_state_dict(sd)


def _worker(rank, world, inplace, ref_losses):
    import torch.distributed as dist
    from rtp_b200.models.transformer_lm_fsdp import TransformerLM as PlainLM
    from rtp_b200.optim import ShardedAdam
    if inplace:
        from rtp_b200.inplace.models.transformer_lm_rtp_inplace import TransformerLM
    else:
        from rtp_b200.models.transformer_lm_rtp import TransformerLM
    torch.manual_seed(0)
    full = PlainLM(V, D, NH, H, 0.0, 0.1, L)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in full.parameters():
            p.copy_(torch.rand(p.shape, generator=g) * 0.2 - 0.1)
    model = TransformerLM(V, D, NH, H, 0.0, 0.1, L, world, rank)
    _load_from_full(model, full, rank, world)
    opt = ShardedAdam(model.parameters(), lr=1e-3)
    x, y = _data()
    bs = B // world
    xs, ys = x[:, rank * bs:(rank + 1) * bs], y[:, rank * bs:(rank + 1) * bs]
    for step in range(STEPS):
        opt.zero_grad()
        loss = F.cross_entropy(model(xs).view(-1, V), ys.reshape(-1))
        (loss / world).backward()
        opt.step()
        t = loss.detach().clone()
        dist.all_reduce(t)
        mean_loss = t.item() / world
        assert abs(mean_loss - ref_losses[step]) < 1e-5, (step, mean_loss, ref_losses[step])


@pytest.mark.parametrize("world,inplace", [(2, False), (4, False), (2, True)])
def test_lm_trajectory_matches_single_process(world, inplace):
    _, losses = _reference_losses()
    run_distributed(_worker, world, inplace, losses, timeout=600)
