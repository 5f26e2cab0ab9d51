"""Device-side step counter of the library's counter-based dropout generator.

Every dropout mask of the kernels depends only on (seed, offset of the call site, step counter, position).  The counter
lives on the device so that a training step captured in a CUDA graph draws fresh masks at every replay: the optimizers
advance it (one ``add_`` kernel, capturable) at the end of ``step()``."""
import torch

_steps = {}


def step_tensor(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    t = _steps.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int64, device=dev)
        _steps[key] = t
    return t


def advance(device=None):
    step_tensor(device).add_(1)
