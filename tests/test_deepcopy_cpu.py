"""Rotated modules survive copy.deepcopy inside an initialised process group (the copy shares the ring)."""
import copy

import torch

from _dist import run_distributed


def _worker(rank, world):
    from rtp_b200.models.transformer_lm_rtp import TransformerLM
    torch.manual_seed(0)
    m = TransformerLM(64, 16, 2, 32, 0.0, 0.1, 1, world, rank)
    c = copy.deepcopy(m)
    x = torch.randint(0, 64, (5, 2))
    assert torch.allclose(m(x), c(x))
    c[3].linear.linear.weight.data.add_(1.0)                       # the copy owns its own flat buffers
    assert not torch.allclose(m(x), c(x))
    assert c[3].linear.ring is m[3].linear.ring


def test_deepcopy():
    run_distributed(_worker, 2)
