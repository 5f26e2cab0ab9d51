"""Rotated modules vs their plain torch counterparts on CPU/gloo rings of 1, 2 and 4 ranks.

Pattern of the reference's tests (tests/test_linear.py:117-186 etc.): build the full layer and the full
batch identically on every rank, slice the batch by rank, build the rotated layer from the full layer,
compare the output with the rank's slice and the (ring-reduced) shard gradients with the matching
slices of the full gradients.  Unlike the reference, this also runs at N=4, in-place, and repeats the
forward under no_grad."""
import pytest
import torch
import torch.nn.functional as F

from _dist import run_distributed

WORLDS = [1, 2, 4]


def _close(a, b, tol=1e-5, what=""):
    assert torch.allclose(a, b, atol=tol, rtol=tol), f"{what}: max diff {(a - b).abs().max().item()}"


def _linear(rank, world, inplace):
    from rtp_b200.module.linear import ColumnParallelLinear, RowParallelLinear
    torch.manual_seed(0)
    full = torch.nn.Linear(8, 8)
    x = torch.randn(8 * world, 8)
    tgt = torch.randint(0, 8, (8 * world,))
    F.cross_entropy(full(x), tgt, reduction="sum").div(8 * world).backward()
    ref_out = full(x).detach()
    sl = slice(rank * 8, (rank + 1) * 8)
    for cls in (ColumnParallelLinear, RowParallelLinear):
        m = cls(8, 8, linear_layer=full)
        m.inplace = inplace
        xs = x[sl].clone().requires_grad_(True)
        out = m(xs)
        _close(out, ref_out[sl], what=f"{cls.__name__} out")
        F.cross_entropy(out, tgt[sl], reduction="sum").div(8 * world).backward()
        dim = 1 if cls is RowParallelLinear else 0
        _close(m.linear.weight.grad, torch.chunk(full.weight.grad, world, dim=dim)[rank], what="dW")
        if cls is ColumnParallelLinear:
            _close(m.linear.bias.grad, torch.chunk(full.bias.grad, world)[rank], what="db")
        else:
            _close(m.linear.bias.grad, full.bias.grad, what="db(row)")
            _close(m.linear.bias * world, full.bias, what="row bias is b/N")
        for _ in range(2):  # forward-only passes leave the shards at home
            with torch.no_grad():
                _close(m(xs), ref_out[sl], what="no_grad repeat")
        assert set(m.state_dict().keys()) == {"linear.weight", "linear.bias"}


def _embedding(rank, world, inplace):
    from rtp_b200.module.embedding import ParallelEmbedding
    torch.manual_seed(0)
    full = torch.nn.Embedding(8, 8)
    ids = torch.randint(0, 8, (8 * world, 3))
    w = torch.randn(8 * world, 3, 8)
    (full(ids) * w).sum().backward()
    sl = slice(rank * 8, (rank + 1) * 8)
    m = ParallelEmbedding(8, 8, world, rank, Embedding_layer=full)
    m.inplace = inplace
    out = m(ids[sl])
    _close(out, full(ids).detach()[sl], what="embedding out")
    (out * w[sl]).sum().backward()
    _close(m.embedding.weight.grad, torch.chunk(full.weight.grad, world, dim=1)[rank], what="embedding grad")
    assert list(m.state_dict().keys()) == ["embedding.weight"]


def _attention(rank, world, inplace):
    from rtp_b200.module.attention import ParallelMultiheadAttention
    torch.manual_seed(0)
    E, H, L, B = 8, 4, 5, 2 * world
    full = torch.nn.MultiheadAttention(E, H)
    with torch.no_grad():
        full.in_proj_bias.normal_()
        full.out_proj.bias.normal_()
    x = torch.randn(L, B, E)
    mask = torch.full((L, L), float("-inf")).triu_(1)
    out_ref, w_ref = full(x, x, x, attn_mask=mask)
    out_ref.square().sum().backward()
    sl = slice(rank * 2, (rank + 1) * 2)
    m = ParallelMultiheadAttention(E, H, world, rank, MultiheadAttention_layer=full)
    m.inplace = inplace
    xs = x[:, sl].clone().requires_grad_(True)
    with torch.no_grad():
        out, w = m(xs, xs, xs, attn_mask=mask, need_weights=True)
        _close(out, out_ref.detach()[:, sl], what="mha out need_weights=True")
        assert w is not None and w.shape == (2, L, L)
    out, w = m(xs, xs, xs, attn_mask=mask, need_weights=False)
    _close(out, out_ref.detach()[:, sl], what="mha out need_weights=False")
    out.square().sum().backward()
    Es = E // world
    ipw = full.in_proj_weight.grad
    exp = torch.cat([ipw[k * E + rank * Es: k * E + (rank + 1) * Es] for k in range(3)])
    _close(m.MultiheadAttention.in_proj_weight.grad, exp, what="in_proj_weight grad")
    ipb = full.in_proj_bias.grad
    expb = torch.cat([ipb[k * E + rank * Es: k * E + (rank + 1) * Es] for k in range(3)])
    _close(m.MultiheadAttention.in_proj_bias.grad, expb, what="in_proj_bias grad")
    _close(m.MultiheadAttention.out_proj.weight.grad, torch.chunk(full.out_proj.weight.grad, world, dim=1)[rank],
           what="out_proj.weight grad")
    _close(m.MultiheadAttention.out_proj.bias.grad, full.out_proj.bias.grad, what="out_proj.bias grad")
    assert set(m.state_dict().keys()) == {"MultiheadAttention.in_proj_weight", "MultiheadAttention.in_proj_bias",
                                          "MultiheadAttention.out_proj.weight", "MultiheadAttention.out_proj.bias"}


def _conv(rank, world, inplace):
    from rtp_b200.module.conv import ColumnParallelConv2d
    torch.manual_seed(0)
    full = torch.nn.Conv2d(8, 8, 3, padding=1)
    x = torch.randn(2 * world, 8, 6, 6)
    full(x).square().sum().backward()
    sl = slice(rank * 2, (rank + 1) * 2)
    m = ColumnParallelConv2d(8, 8, 3, padding=1, Conv2d_layer=full)
    m.inplace = inplace
    out = m(x[sl])
    _close(out, full(x).detach()[sl], what="conv out")
    out.square().sum().backward()
    _close(m.conv.weight.grad, torch.chunk(full.weight.grad, world)[rank], tol=1e-4, what="conv dW")
    _close(m.conv.bias.grad, torch.chunk(full.bias.grad, world)[rank], tol=1e-4, what="conv db")


def _moe(rank, world, inplace):
    """Rotating experts == all-to-all experts (same data on every rank, as in tests/test_moe.py:136-194)."""
    import rtp_b200.module.top2gate as tg
    from rtp_b200.module.moe import MOELayer, WeightMOELayer
    from rtp_b200.module.top2gate import Top2Gate, WeightTop2Gate
    torch.manual_seed(0)
    d, S = 8, 4 * world
    E = world  # one local expert per rank
    noise = torch.randn(S, E)
    tg.gumbel_rsample = lambda shape, device: noise  # deterministic second choice
    gate = Top2Gate(d, E)
    all_experts = [torch.nn.Linear(d, d) for _ in range(E)]
    x = torch.randn(S, 1, d)
    # all-to-all baseline
    import copy
    base = MOELayer(copy.deepcopy(gate), copy.deepcopy(all_experts[rank]))
    out_ref = base(x)
    out_ref.square().sum().backward()
    # rotating
    wgate = WeightTop2Gate(d, E, gate=gate)
    rot = WeightMOELayer(wgate, copy.deepcopy(all_experts[rank]))
    rot.inplace = inplace
    wgate.inplace = inplace
    out = rot(x)
    _close(out, out_ref.detach(), tol=1e-5, what="moe out")
    out.square().sum().backward()
    # expert grads: baseline expert saw tokens of all ranks through the all-to-all; rotation sums over ranks
    _close(rot.experts[0].weight.grad, base.experts[0].weight.grad, tol=1e-5, what="expert dW")
    _close(rot.experts[0].bias.grad, base.experts[0].bias.grad, tol=1e-5, what="expert db")
    # gate grad: baseline gate is replicated and sees local tokens only; rotated gate shard sums over ranks
    _close(wgate.wg.weight.grad, world * base.gate.wg.weight.grad[rank:rank + 1], tol=1e-5, what="gate grad")
    _close(rot.l_aux, base.l_aux, what="l_aux")


def _all_cases(rank, world, inplace):
    for case in (_linear, _embedding, _attention, _conv, _moe):
        try:
            case(rank, world, inplace)
        except Exception as e:
            raise AssertionError(f"{case.__name__} failed: {e}") from e


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("inplace", [False, True])
def test_rotated_modules(world, inplace):
    run_distributed(_all_cases, world, inplace)


def _inplace_displaced_guard(rank, world):
    from rtp_b200.module.linear import ColumnParallelLinear
    torch.manual_seed(0)
    m = ColumnParallelLinear(8, 8)
    m.inplace = True
    x = torch.randn(4, 8, requires_grad=True)
    y = m(x)
    if world > 1:
        with pytest.raises(RuntimeError):
            m(x)          # shards are displaced until backward runs
    y.sum().backward()
    m(x).sum().backward()


def test_inplace_displaced_guard():
    run_distributed(_inplace_displaced_guard, 2)


def test_rotating_experts_with_one_gate_row_per_rank_on_eight_ranks():
    """The MoE case on a ring of 8: one expert and ONE row of the gate weight per rank (the shape of the 8-GPU runs)."""
    run_distributed(_moe, 8, False, timeout=300)
