"""Whole-step CUDA-graph capture for models built from rotated modules.

The module path launches a few hundred short kernels per step; launched eagerly from Python the step is bound by the
host.  ``GraphedStep`` captures one complete training step (forward, loss, backward, gradient sync, optimizer) once and
replays it: the rotation kernels, the attention / norm / Adam kernels and NCCL's small all-reduce are all capturable, and
the dropout masks stay fresh because they depend on a device-side step counter (``rtp_b200.ops.rng``).

Rules for ``step_fn(*static_inputs) -> loss tensor``: no host synchronisation (``.item()``, ``engine.check_all()``), and
``optimizer.zero_grad(set_to_none=False)`` so that gradient buffers keep their addresses."""
import torch
import torch.distributed as dist


class GraphedStep:
    def __init__(self, step_fn, example_inputs, warmup: int = 3):
        self.step_fn = step_fn
        self.static_in = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(warmup):              # sizes workspaces, builds plans, fills caches, warms NCCL up
                step_fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_out = step_fn(*self.static_in)

    def __call__(self, *inputs):
        for dst, src in zip(self.static_in, inputs):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_out
