"""Device-side timing. The reference times with ``time.time()`` and one synchronize at the end
(benchmarks/rtp_benchmark.py:146,205-208); here every number is taken with CUDA events on the launching stream
and reduced with MAX over the ranks of the ring."""
import contextlib
import os
import time

import torch
import torch.distributed as dist


def max_over_ranks(value: float, group=None) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return value
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.item()


class DeviceTimer:
    """``with DeviceTimer() as t: ...`` then ``t.ms`` (CUDA events on GPU, perf_counter on CPU)."""

    def __init__(self, device=None, group=None, reduce_max=True):
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.group, self.reduce_max = group, reduce_max
        self.ms = None

    def __enter__(self):
        if self.cuda:
            torch.cuda.synchronize()
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e1 = torch.cuda.Event(enable_timing=True)
            self.e0.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self.e1.record()
            torch.cuda.synchronize()
            ms = self.e0.elapsed_time(self.e1)
        else:
            ms = (time.perf_counter() - self.t0) * 1e3
        self.ms = max_over_ranks(ms, self.group) if self.reduce_max else ms
        return False


_NVTX = os.environ.get("RTP_NVTX", "0") not in ("", "0")


def set_nvtx(on: bool) -> bool:
    """Switches the NVTX ranges of the library on or off (``RTP_NVTX=1`` does the same); returns the old setting."""
    global _NVTX
    old, _NVTX = _NVTX, bool(on)
    return old


@contextlib.contextmanager
def nvtx_range(name: str):
    """A named NVTX range around a group of launches (the trainer marks forward / backward of every layer, the head
    and the optimizer), visible to any timeline tool that reads NVTX; free when switched off."""
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield
