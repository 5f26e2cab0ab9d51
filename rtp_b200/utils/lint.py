"""Static check of the rotation programs, on any machine (no GPU needed).

``lint_linear`` / ``lint_experts`` build the kernel programs of EVERY rank of a made-up ring exactly as a launch would
(same builders, tensor maps recorded by a host stand-in) and check what the kernel relies on: every tiled copy starts
on a 16-byte boundary of its innermost coordinate, tile segments divide the output evenly, no two tiles of
non-accumulating phases write the same bytes, and the cross-rank counter protocol is consistent (exactly one producer
per arrival counter that a rank waits on, the producer waits for the matching credit in its own flag block and writes
inside the counter's slot, the consumer reports the slot done, fill counts advance identically on every rank).  It is
the protocol's race detector for shapes and ring sizes that no test has run on hardware; ``python -m
rtp_b200.utils.lint`` sweeps the model configurations of ``bench.py``."""
import ctypes as C
from typing import List, Tuple

from ..ops import _lib


def _fn(name):
    L = _lib.lib()
    f = getattr(L, name)
    ints = [C.c_int] * 2 + [C.c_ulonglong] + [C.c_int] * (8 if name == "rtp_lint_linear" else 7)
    f.argtypes = ints + [C.c_char_p, C.c_int]
    f.restype = C.c_int
    return f


def lint_linear(world: int, mode: int, M: int, in_features: int, out_features: int, bias: bool = True,
                backward: bool = False, need_dx: bool = True, ctas: int = 148, slot_bytes: int = 1 << 30,
                inject: int = 0) -> Tuple[int, List[str]]:
    """Programs of one rotated linear (``mode`` 0 = column, 1 = row) on a ring of ``world`` ranks.  Returns (number of
    problems, one line per problem)."""
    buf = C.create_string_buffer(8192)
    n = _fn("rtp_lint_linear")(world, ctas, slot_bytes, mode, M, in_features, out_features, int(bias), int(backward),
                               int(need_dx), inject, buf, 8192)
    return n, [ln for ln in buf.value.decode().splitlines() if ln]


def lint_experts(world: int, n_local: int, cap: int, in_features: int, out_features: int, bias: bool = True,
                 backward: bool = False, need_dx: bool = True, ctas: int = 148, slot_bytes: int = 1 << 30
                 ) -> Tuple[int, List[str]]:
    """Programs of one linear of every rotating expert (``n_local`` experts per rank, ``cap`` tokens per expert)."""
    buf = C.create_string_buffer(8192)
    n = _fn("rtp_lint_experts")(world, ctas, slot_bytes, n_local, cap, in_features, out_features, int(bias),
                                int(backward), int(need_dx), buf, 8192)
    return n, [ln for ln in buf.value.decode().splitlines() if ln]


def lint_chain(world: int, launches, ctas: int = 148, slot_bytes: int = 1 << 30, flip_bank_at: int = -1
               ) -> Tuple[int, List[str]]:
    """A chain of rotated linears with cross-launch prefetch, as ``FusedLMTrainer`` issues them (launch k reads
    weight-slot bank ``k & 1`` and pushes the shards of launch k + 1 into the other bank).  ``launches``: one tuple
    ``(mode, M, in_features, out_features, bias, backward, need_dx)`` per launch.  ``flip_bank_at`` builds that launch
    with the wrong bank, to test the lint itself."""
    f = _lib.lib().rtp_lint_linear_chain
    f.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_int, C.POINTER(C.c_int), C.c_int, C.c_char_p, C.c_int]
    f.restype = C.c_int
    flat = [int(v) for l in launches for v in l]
    assert len(flat) == 7 * len(launches)
    arr = (C.c_int * len(flat))(*flat)
    buf = C.create_string_buffer(8192)
    n = f(world, ctas, slot_bytes, len(launches), arr, flip_bank_at, buf, 8192)
    return n, [ln for ln in buf.value.decode().splitlines() if ln]


def lint_transport(world: int, kind: str, a: int, b: int = 0, c: int = 0, ctas: int = 148, slot_bytes: int = 1 << 30
                   ) -> Tuple[int, List[str]]:
    """The programs without GEMM tiles: ``kind`` "embedding" (rotated lookup: a = vocabulary, b = embedding dim, c =
    tokens) or "reduce" (one-hop reduce of ``world`` blocks of ``a`` elements, the embedding gradient's route)."""
    f = _lib.lib().rtp_lint_transport
    f.argtypes = [C.c_int, C.c_int, C.c_ulonglong, C.c_int, C.c_longlong, C.c_longlong, C.c_longlong, C.c_char_p, C.c_int]
    f.restype = C.c_int
    buf = C.create_string_buffer(8192)
    n = f(world, ctas, slot_bytes, {"embedding": 0, "reduce": 1}[kind], a, b, c, buf, 8192)
    if n < 0:
        raise ValueError(_lib.lib().rtp_last_error().decode())
    return n, [ln for ln in buf.value.decode().splitlines() if ln]


def lm_chain(M: int, D: int, H: int, V: int, layers: int):
    """The chain of a transformer LM step: per layer QKV (column), attention output (row), FFN up and down (column),
    then the head, and the same linears backwards."""
    per_layer = [(0, M, D, 3 * D), (1, M, D, D), (0, M, D, H), (0, M, H, D)]
    fwd = per_layer * layers + [(0, M, D, V)]
    return [(m, t, i, o, 1, 0, 1) for (m, t, i, o) in fwd] + [(m, t, i, o, 1, 1, 1) for (m, t, i, o) in reversed(fwd)]


def sweep(worlds=(1, 2, 3, 4, 5, 6, 7, 8)) -> int:
    """Every rotated linear of the README LM, GPT-1.3B, Llama-13B and the MoE config on every ring size."""
    shapes = []
    # (tokens, in, out, mode)
    for D, H, V, M in ((2048, 2048, 10240, 1024), (2048, 8192, 50304, 16384), (5120, 13824, 32000, 8192)):
        shapes += [(M, D, 3 * D, 0), (M, D, D, 1), (M, D, H, 0), (M, H, D, 0), (M, D, V, 0)]
    total = 0
    for N in worlds:
        for (M, i, o, mode) in shapes:
            if (o % N if mode == 0 else i % N) or ((o // N) % 8 if mode == 0 else (i // N) % 8):
                continue
            for bwd in (False, True):
                n, lines = lint_linear(N, mode, M, i, o, backward=bwd)
                total += n
                for ln in lines[:4]:
                    print(f"world {N} {'row' if mode else 'column'} {M}x{i}->{o} {'backward' if bwd else 'forward'}: {ln}")
        for (nl, cap) in ((8 // N, 2560),) if 8 % N == 0 else ():
            for (i, o) in ((2048, 8192), (8192, 2048)):
                for bwd in (False, True):
                    n, lines = lint_experts(N, nl, cap, i, o, backward=bwd)
                    total += n
                    for ln in lines[:4]:
                        print(f"world {N} experts x{nl} {i}->{o} {'backward' if bwd else 'forward'}: {ln}")
        for (V, D, T) in ((10240, 2048, 1024), (50304, 2048, 16384), (32000, 5120, 8192)):
            if D % (8 * N) == 0:
                for kind, args in (("embedding", (V, D, T)), ("reduce", (V * (D // N),))):
                    n, lines = lint_transport(N, kind, *args)
                    total += n
                    for ln in lines[:4]:
                        print(f"world {N} {kind} V{V} D{D}: {ln}")
        if N > 1:
            for (M, D, H, V, layers) in ((1024, 2048, 2048, 10240, 10), (16384, 2048, 8192, 50304, 2)):
                if (3 * D) % (8 * N) or H % (8 * N) or V % (8 * N):
                    continue
                n, lines = lint_chain(N, lm_chain(M, D, H, V, layers))
                total += n
                for ln in lines[:6]:
                    print(f"world {N} chain D{D} H{H} V{V} x{layers}: {ln}")
    return total


if __name__ == "__main__":
    n = sweep()
    print(f"{n} problem(s)")
    raise SystemExit(1 if n else 0)
