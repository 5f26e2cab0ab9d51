"""Sharded checkpoints end to end on gloo ranks: save -> load on the same ring (weights, optimizer moments, step and
RNG: the resumed run continues bit-exactly), and re-sharding 2 -> 4 -> 2 ranks bit-exactly."""
import os
import tempfile

import torch
import torch.nn.functional as F

from tests._dist import run_distributed

V, D, NH, H, L, S, B = 64, 32, 4, 64, 2, 8, 4


def _make(world, rank, seed=0):
    from rtp_b200.models.transformer_lm_rtp import TransformerLM
    torch.manual_seed(seed)
    return TransformerLM(V, D, NH, H, 0.1, 0.1, L, world, rank)


def _batch(rank, step):
    g = torch.Generator().manual_seed(1000 * step + rank)
    stream = torch.randint(0, V, (S + 1, B), generator=g)
    return stream[:-1], stream[1:]


def _train(model, opt, world, rank, steps, start=0):
    losses = []
    model.train()
    for s in range(start, start + steps):
        x, y = _batch(rank, s)
        opt.zero_grad()
        loss = F.cross_entropy(model(x).view(-1, V), y.reshape(-1))
        (loss / world).backward()
        opt.step()
        losses.append(loss.item())
    return losses


def _save_load_worker(rank, world, directory):
    from rtp_b200.checkpoint import load_sharded, save_sharded
    from rtp_b200.optim import ShardedAdam
    model = _make(world, rank)
    opt = ShardedAdam(model.parameters(), lr=1e-2, clip_value=0.5)
    _train(model, opt, world, rank, 3)
    save_sharded(directory, model, opt, step=3)
    expect = _train(model, opt, world, rank, 3, start=3)          # dropout is on: the RNG matters
    # a fresh process state: other weights, other optimizer, other RNG position
    model2 = _make(world, rank, seed=99)
    opt2 = ShardedAdam(model2.parameters(), lr=1e-2, clip_value=0.5)
    torch.manual_seed(12345)
    step = load_sharded(directory, model2, opt2)
    assert step == 3
    got = _train(model2, opt2, world, rank, 3, start=3)
    assert got == expect, (got, expect)
    for (n, p), (_, q) in zip(model.named_parameters(), model2.named_parameters()):
        assert torch.equal(p, q), n


def test_save_then_load_resumes_bit_exactly():
    with tempfile.TemporaryDirectory() as d:
        run_distributed(_save_load_worker, 2, d)
        assert sorted(os.listdir(d)) == ["manifest.json", "rank0-of-2.pt", "rank1-of-2.pt"]


def _save_worker(rank, world, directory):
    from rtp_b200.checkpoint import save_sharded
    model = _make(world, rank)
    save_sharded(directory, model, step=7)


def _load_other_ring_worker(rank, world, src, dst):
    from rtp_b200.checkpoint import load_sharded, save_sharded
    model = _make(world, rank, seed=42)
    assert load_sharded(src, model) == 7
    save_sharded(dst, model, step=7)


def test_reshard_2_to_4_to_2_is_bit_exact():
    from rtp_b200.checkpoint import consolidate, reshard
    with tempfile.TemporaryDirectory() as d2, tempfile.TemporaryDirectory() as d4, tempfile.TemporaryDirectory() as d2b:
        run_distributed(_save_worker, 2, d2)
        run_distributed(_load_other_ring_worker, 4, d2, d4)          # load_sharded re-shards on the fly
        run_distributed(_load_other_ring_worker, 2, d4, d2b)
        for r in range(2):
            a = torch.load(os.path.join(d2, f"rank{r}-of-2.pt"), weights_only=False)["model"]
            b = torch.load(os.path.join(d2b, f"rank{r}-of-2.pt"), weights_only=False)["model"]
            assert a.keys() == b.keys()
            for k in a:
                assert torch.equal(a[k], b[k]), k
        # the offline utility gives the same shards as the on-the-fly path
        import json
        sds2 = [torch.load(os.path.join(d2, f"rank{r}-of-2.pt"), weights_only=False)["model"] for r in range(2)]
        sds4 = [torch.load(os.path.join(d4, f"rank{r}-of-4.pt"), weights_only=False)["model"] for r in range(4)]
        plan2 = {k: tuple(v) for k, v in json.load(open(os.path.join(d2, "manifest.json")))["plan"].items()}
        plan4 = {k: tuple(v) for k, v in json.load(open(os.path.join(d4, "manifest.json")))["plan"].items()}
        for r, sd in enumerate(reshard(sds2, plan2, plan4, 4)):
            for k in sd:
                assert torch.equal(sd[k], sds4[r][k]), (r, k)
        full2, full4 = consolidate(sds2, plan2), consolidate(sds4, plan4)
        for k in full2:
            assert torch.equal(full2[k], full4[k]), k
