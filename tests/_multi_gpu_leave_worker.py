"""Worker of the multi-GPU failure test: two ranks train with the fused kernels; after a step has completed on every
rank (nothing in flight: synchronize + barrier) the last rank leaves in an orderly way.  The survivors learn of it on
the host, through the heartbeat store, BEFORE they launch another rotation kernel, so no kernel ever waits for the
missing peer."""
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import faulthandler
    faulthandler.dump_traceback_later(120, exit=True)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=60))
    from rtp_b200.models.fused_lm import FusedLMTrainer
    from rtp_b200.models.transformer_lm_rtp import TransformerLM
    from rtp_b200.utils.watchdog import Heartbeat, RankFailure
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, timeout_s=20.0)
    torch.manual_seed(0)
    model = TransformerLM(512, 256, 4, 512, 0.0, 0.1, 2, world, rank).to(device="cuda", dtype=torch.bfloat16)
    trainer = FusedLMTrainer(model, lr=1e-3, use_graph=False)
    ids = torch.randint(0, 512, (32, 4), device="cuda")
    for step in range(3):
        hb.check()
        loss = trainer.step(ids, ids)
        torch.cuda.synchronize()
        hb.beat(step)
    trainer.check()
    torch.cuda.synchronize()
    dist.barrier()                       # every rank is between steps, nothing in flight
    if rank == world - 1:
        hb.leave()
        print("LEFT", flush=True)
        time.sleep(1.0)
        os._exit(0)
    time.sleep(0.5)
    try:
        hb.check()                       # must raise before the next launch
        print("NOT_DETECTED", flush=True)
        os._exit(1)
    except RankFailure as e:
        assert e.failed_rank == world - 1
        if rank == 0:
            print(f"DETECTED rank {e.failed_rank} left; final loss {float(loss):.3f}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
