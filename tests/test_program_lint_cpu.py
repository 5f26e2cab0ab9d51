"""The host-side lint of the rotation programs: clean on the shapes and ring sizes the library is used with, and it
notices each kind of damage a builder bug would do (the lint's own self-test through its injection switch)."""
import pytest

from rtp_b200.utils import lint


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_linear_programs_are_clean(world):
    for mode, (M, i, o) in [(0, (1024, 2048, 6144)), (1, (1024, 2048, 2048)), (0, (1000, 512, 1024)),
                            (0, (8192, 2048, 32000)), (1, (256, 4096, 512))]:
        if (o % world if mode == 0 else i % world):
            continue
        for bwd in (False, True):
            n, lines = lint.lint_linear(world, mode, M, i, o, backward=bwd)
            assert n == 0, (world, mode, M, i, o, bwd, lines[:5])


@pytest.mark.parametrize("world,n_local", [(2, 4), (4, 2), (8, 1)])
def test_expert_programs_are_clean(world, n_local):
    for bwd in (False, True):
        n, lines = lint.lint_experts(world, n_local, 2560, 2048, 8192, backward=bwd)
        assert n == 0, (world, n_local, bwd, lines[:5])


@pytest.mark.parametrize("inject,needle", [(1, "producers announce it"), (2, "not a multiple of 8 elements"),
                                           (3, "matching credit"), (4, "write the same bytes"),
                                           (5, "outside the slot")])
def test_the_lint_notices_damage(inject, needle):
    n, lines = lint.lint_linear(4, 0, 1024, 2048, 2048, backward=False, inject=inject)
    assert n > 0 and any(needle in ln for ln in lines), (inject, lines[:6])


def test_a_shard_that_does_not_fit_its_slot_is_refused():
    n, lines = lint.lint_linear(2, 0, 1024, 2048, 2048, slot_bytes=1 << 16)
    assert n == 1 and "larger than workspace slot" in lines[0]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_prefetch_chain_of_a_training_step_is_clean(world):
    """The rotated linears of an LM step chained by cross-launch prefetch: every shard a launch waits for is pushed by
    exactly one launch (itself or its predecessor) into the bank it reads."""
    for (M, D, H, V, layers) in ((1024, 2048, 2048, 10240, 10), (4096, 1024, 4096, 8192, 2)):
        n, lines = lint.lint_chain(world, lint.lm_chain(M, D, H, V, layers))
        assert n == 0, (world, D, lines[:6])


def test_the_chain_lint_notices_a_wrong_bank_and_an_unread_prefetch():
    chain = lint.lm_chain(1024, 2048, 2048, 10240, 2)
    n, lines = lint.lint_chain(4, chain, flip_bank_at=3)
    assert n > 0 and any("the chain gives it bank" in ln for ln in lines), lines[:6]
    # a backward launch that needs no input gradient would never read (and never release) the shards pushed ahead for it
    last = len(chain) - 1
    chain[last] = chain[last][:6] + (0,)
    n, lines = lint.lint_chain(4, chain)
    assert n > 0 and any("pushed ahead" in ln for ln in lines), lines[:6]


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_embedding_and_one_hop_reduce_programs_are_clean(world):
    for (V, D, T) in ((10240, 2048, 1024), (32000, 5120, 8192)):
        n, lines = lint.lint_transport(world, "embedding", V, D, T)
        assert n == 0, (world, "embedding", lines[:4])
        n, lines = lint.lint_transport(world, "reduce", V * (D // world))
        assert n == 0, (world, "reduce", lines[:4])
    # a block that does not fit its gradient slot is refused by the builder
    if world > 1:
        n, lines = lint.lint_transport(world, "reduce", 1 << 20, slot_bytes=1 << 16)
        assert n == 1 and "larger than workspace slot" in lines[0]
