"""Dispatch of rotated layers onto the fused sm_100a kernels (filled in by rtp_b200.parallel.engine)."""
import torch

from .context import get_backend


def use_fused(x: torch.Tensor, flat: torch.Tensor) -> bool:
    """Fused path: bf16 CUDA tensors, unless the functional backend was requested explicitly."""
    be = get_backend()
    if be == "functional":
        return False
    ok = x.is_cuda and flat.is_cuda and flat.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
    if be == "fused" and not ok:
        raise RuntimeError("backend 'fused' needs bf16 CUDA tensors")
    return ok


def linear(module, x, row=False):
    from .engine import fused_linear
    return fused_linear(module, x, row=row)


def linear_ok(row, in_f, out_f, world):
    """Shapes that the fused kernels cannot take (a feature count that is not a multiple of 8, e.g. a 10-class head)
    run on the functional engine instead."""
    from .engine import fused_linear_ok
    return fused_linear_ok(row, in_f, out_f, world)
