"""Console + JSONL metrics. Console lines follow the reference's benchmark output
(``| batch {i} | wps {..} | loss {..} | ppl {..}``, benchmarks/rtp_benchmark.py:192-203); every record is also
appended to a JSONL file when a path is given."""
import json
import math
import time
from typing import Optional

import torch


def peak_memory_gib(device=None) -> float:
    """``allocated_bytes.all.peak`` in GiB, the reference's memory metric (benchmarks/rtp_benchmark.py:233-237)."""
    if not torch.cuda.is_available():
        return 0.0
    return torch.cuda.memory_stats(device)["allocated_bytes.all.peak"] / 2 ** 30


class MetricsLogger:
    def __init__(self, path: Optional[str] = None, rank: int = 0, quiet: bool = False):
        self.path, self.rank, self.quiet = path, rank, quiet
        self.t0 = time.time()

    def log(self, **record):
        record.setdefault("t", time.time() - self.t0)
        record.setdefault("rank", self.rank)
        if self.path and self.rank == 0:
            with open(self.path, "a") as f:
                f.write(json.dumps(record) + "\n")
        return record

    def batch(self, i: int, wps: float, loss: float):
        if self.rank == 0 and not self.quiet:
            ppl = math.exp(loss) if loss < 50 else float("inf")
            print("| batch {:5d} | wps {:5.2f} | loss {:5.2f} | ppl {:8.2f}".format(i, wps, loss, ppl), flush=True)
        return self.log(kind="batch", batch=i, wps=wps, loss=loss)

    def summary(self, **kw):
        if self.rank == 0 and not self.quiet:
            print(" ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in kw.items()), flush=True)
        return self.log(kind="summary", **kw)
