"""Guard bands around kernel outputs: a debug aid that catches out-of-bounds writes of a kernel without a memory
checker.  ``guarded_empty`` returns a view into a larger buffer whose margins hold a canary pattern;
``check_guards`` verifies that the margins are intact after the kernels under test have run."""
from typing import List, Tuple

import torch

_CANARY = {torch.bfloat16: -1.625, torch.float32: -1.625, torch.float16: -1.625, torch.int32: 0x5A5A5A5A,
           torch.int64: 0x5A5A5A5A, torch.uint8: 0xA5}

_live: List[Tuple[torch.Tensor, int, int, str]] = []


def guarded_empty(shape, dtype=torch.bfloat16, device="cuda", band: int = 4096, name: str = ""):
    """A contiguous tensor of ``shape`` with ``band`` canary elements before and after it (band is rounded up so that the
    payload keeps a 256-byte alignment)."""
    n = 1
    for s in shape:
        n *= int(s)
    item = torch.empty((), dtype=dtype).element_size()
    band = (band * item + 255) // 256 * 256 // item
    buf = torch.full((band + n + band,), _CANARY[dtype], dtype=dtype, device=device)
    _live.append((buf, band, n, name))
    return buf[band:band + n].view(*shape)


def check_guards(clear: bool = True):
    """Raises AssertionError naming the first tensor whose guard band was overwritten."""
    try:
        for buf, band, n, name in _live:
            c = torch.tensor(_CANARY[buf.dtype], dtype=buf.dtype, device=buf.device)
            head_ok = bool((buf[:band] == c).all())
            tail_ok = bool((buf[band + n:] == c).all())
            assert head_ok, f"guard band BEFORE tensor {name!r} was overwritten"
            assert tail_ok, f"guard band AFTER tensor {name!r} was overwritten"
    finally:
        if clear:
            _live.clear()
