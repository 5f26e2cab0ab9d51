"""One rotated linear (forward, then fused backward) on a ring of real GPUs: graph-replay timing and the kernel's own
timeline (``%globaltimer`` stamps of CTA 0 of rank 0: phase waits, tiles, signals, pushes).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m rtp_b200.bench.ring_case \
        --tokens 1024 --in-features 2048 --out-features 2048

Used for the multi-GPU summaries under profiles/.  Run with NCCL_NVLS_ENABLE=0 when ranks may leave early."""
import argparse
import ctypes as C
import datetime
import os
import sys

import torch
import torch.distributed as dist


def _g(t, base, i):
    v = int(t[i])
    return (v - base) / 1e3 if v > 0 else float("nan")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1024, help="rows of the activation matrix")
    ap.add_argument("--in-features", type=int, default=2048)
    ap.add_argument("--out-features", type=int, default=2048)
    ap.add_argument("--calls", type=int, default=10, help="launches per captured graph")
    a = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=120))
    from ..ops import _lib
    from ..parallel import engine as E
    from ..parallel.context import RingContext
    L = _lib.lib()
    L.rtp_debug_set_trace.argtypes = [C.c_void_p]
    dev, bf = "cuda", torch.bfloat16
    M, K_, Nf = a.tokens, a.in_features, a.out_features
    Os = Nf // world
    eng = E.FusedEngine(RingContext(dist.group.WORLD, rank, world), (Os * K_ + Os) * 2)
    flat = torch.randn(Os * K_ + Os, device=dev, dtype=bf) * 0.02
    info = (True, Os * K_, (Os * K_ + Os) * 2)
    x = torch.randn(M, K_, device=dev, dtype=bf)
    out = torch.empty(M, Nf, device=dev, dtype=bf)
    dy = torch.randn(M, Nf, device=dev, dtype=bf)
    dx = torch.empty(M, K_, device=dev, dtype=bf)
    gflat = torch.empty_like(flat)
    dbias = torch.empty(Nf, device=dev, dtype=torch.float32)
    tr = torch.zeros(1024, dtype=torch.int64, device=dev)

    def fwd():
        E.linear_fwd_raw(eng, flat, info, x, False, K_, Nf, out=out)

    def bwd():
        E.linear_bwd_raw(eng, flat, info, x, dy, False, K_, Nf, grad_out=gflat, dx_out=dx, dbias_buf=dbias)

    for name, f in (("forward", fwd), ("backward", bwd)):
        for _ in range(5):
            f()
        torch.cuda.synchronize()
        dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(a.calls):
                f()
        dist.barrier()
        g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        t_graph = e0.elapsed_time(e1) * 1e3 / a.calls
        # timeline of the last of four back-to-back launches (the stamps of the earlier ones are overwritten)
        tr.zero_()
        L.rtp_debug_set_trace(tr.data_ptr())
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2):
            for _ in range(4):
                f()
        L.rtp_debug_set_trace(None)
        dist.barrier()
        g2.replay()
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            t = tr.cpu()
            base = int(t[3 * 256 + 64])
            print(f"== {name}, {world} ranks, M {M} in {K_} out {Nf}: {t_graph:.1f} us per call (graph replay of {a.calls})")
            print("   kernel entry 0.00 | set-up done %.2f | tear-down %.2f" % (_g(t, base, 3 * 256 + 65), _g(t, base, 3 * 256 + 70)))
            for p in range(16):
                o = 3 * 256 + 128 + p * 4
                if int(t[o]) == 0:
                    break
                print("   phase %d: start %.2f | waits done %.2f | tiles done %.2f | signalled %.2f"
                      % (p, _g(t, base, o), _g(t, base, o + 1), _g(t, base, o + 2), _g(t, base, o + 3)))
            for j in range(8):
                o = 3 * 256 + 200 + j * 4
                if int(t[o]) == 0:
                    break
                print("   push %d: start %.2f | credit %.2f | signalled %.2f" % (j, _g(t, base, o), _g(t, base, o + 1), _g(t, base, o + 2)))
        sys.stdout.flush()
    _lib.check_status()
    dist.barrier()
    os._exit(0)   # live CUDA graphs make process-group destruction hang


if __name__ == "__main__":
    main()
