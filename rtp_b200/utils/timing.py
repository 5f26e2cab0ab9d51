"""Device-side timing. The reference times with ``time.time()`` and one synchronize at the end
(benchmarks/rtp_benchmark.py:146,205-208); here every number is taken with CUDA events on the launching stream
and reduced with MAX over the ranks of the ring."""
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
