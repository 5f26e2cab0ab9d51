"""``RotatedTensorParallel(model)`` vs the unwrapped model on gloo rings (reference: test_net.py:135-177 wraps
the MNIST Net and compares output + dim-0-sharded grads; here also MHA, embedding, in-place and N=4)."""
import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from _dist import run_distributed


class Net(nn.Module):
    """The MNIST network of the reference's examples (rtp_mnist.py / benchmarks/rtp_mnist.py:42-66)."""

    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 32, 3, 1)
        self.conv2 = nn.Conv2d(32, 64, 3, 1)
        self.fc1 = nn.Linear(9216, 128)
        self.fc2 = nn.Linear(128, 10)     # 10 % 4 != 0 -> row split at N=4

    def forward(self, x):
        x = F.relu(self.conv1(x))
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        x = torch.flatten(x, 1)
        return F.log_softmax(self.fc2(F.relu(self.fc1(x))), dim=1)


class Tiny(nn.Module):
    def __init__(self):
        super().__init__()
        self.emb = nn.Embedding(16, 8)
        self.attn = nn.MultiheadAttention(8, 4)
        self.norm = nn.LayerNorm(8)
        self.out = nn.Linear(8, 16)

    def forward(self, ids):
        x = self.emb(ids)
        x = self.norm(x + self.attn(x, x, x, need_weights=False)[0])
        return self.out(x)


def _worker(rank, world, inplace):
    from rtp_b200.rotated_tensor_parallel import RotatedTensorParallel, FlyweightWarpper
    from rtp_b200.optim import sync_replicated_grads
    torch.manual_seed(0)
    # --- MNIST net
    full = Net()
    x = torch.randn(2 * world, 1, 28, 28)
    y = torch.randint(0, 10, (2 * world,))
    F.nll_loss(full(x), y, reduction="sum").div(2 * world).backward()
    wrapped = RotatedTensorParallel(copy.deepcopy(full).apply(lambda m: None), inplace=inplace)
    sl = slice(2 * rank, 2 * rank + 2)
    out = wrapped(x[sl])
    assert torch.allclose(out, full(x).detach()[sl], atol=1e-5), (out - full(x)[sl]).abs().max()
    F.nll_loss(out, y[sl], reduction="sum").div(2 * world).backward()
    assert isinstance(wrapped.module.fc1, FlyweightWarpper)
    g = wrapped.module.fc1.module.weight.grad
    assert torch.allclose(g, torch.chunk(full.fc1.weight.grad, world, 0)[rank], atol=1e-5)
    g = wrapped.module.conv2.module.weight.grad
    assert torch.allclose(g, torch.chunk(full.conv2.weight.grad, world, 0)[rank], atol=1e-4)
    if 10 % world == 0:
        assert torch.allclose(wrapped.module.fc2.module.bias.grad, torch.chunk(full.fc2.bias.grad, world)[rank], atol=1e-5)
    else:   # row split: full-length bias stored as b/N, full gradient on every rank
        assert torch.allclose(wrapped.module.fc2.module.bias.grad, full.fc2.bias.grad, atol=1e-5)
        assert torch.allclose(wrapped.module.fc2.module.bias * world, full.fc2.bias, atol=1e-6)
    assert "module.fc1.module.weight" in wrapped.state_dict()
    # --- embedding + attention + replicated LayerNorm
    full2 = Tiny()
    ids = torch.randint(0, 16, (5, 2 * world))
    full2(ids).square().sum().backward()
    w2 = RotatedTensorParallel(copy.deepcopy(full2), inplace=inplace)
    out2 = w2(ids[:, sl])
    assert torch.allclose(out2, full2(ids).detach()[:, sl], atol=1e-5)
    out2.square().sum().backward()
    assert isinstance(w2.module.attn, FlyweightWarpper)      # the rotating attention is really installed
    sync_replicated_grads(w2.parameters())
    assert torch.allclose(w2.module.norm.weight.grad, full2.norm.weight.grad, atol=1e-4)
    assert torch.allclose(w2.module.emb.module.weight.grad, torch.chunk(full2.emb.weight.grad, world, 1)[rank], atol=1e-5)
    assert torch.allclose(w2.module.attn.module.out_proj.weight.grad,
                          torch.chunk(full2.attn.out_proj.weight.grad, world, 1)[rank], atol=1e-5)


@pytest.mark.parametrize("world,inplace", [(1, False), (2, False), (2, True), (4, False)])
def test_wrapper(world, inplace):
    run_distributed(_worker, world, inplace)
