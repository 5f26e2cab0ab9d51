"""Failure detection on the host (gloo ranks, no GPU involved): a rank that leaves between steps or stops beating is
reported through the store before the survivors start their next step; a short process-group timeout ends a
collective whose peer never joins."""
import datetime
import os
import time

import pytest
import torch
import torch.distributed as dist

from _dist import run_distributed, _free_port


def _leaver(rank, world):
    from rtp_b200.utils.watchdog import Heartbeat, RankFailure
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, timeout_s=2.0)
    dist.barrier()
    for step in range(3):
        hb.check()
        t = torch.ones(1)
        dist.all_reduce(t)
        hb.beat(step)
    dist.barrier()
    if rank == world - 1:
        hb.leave()                      # orderly exit between steps, nothing in flight
        time.sleep(1.0)
        return
    time.sleep(0.3)
    with pytest.raises(RankFailure) as ei:
        hb.check()                      # the survivors learn of it before their next collective
    assert ei.value.failed_rank == world - 1


def _silent(rank, world):
    from rtp_b200.utils.watchdog import Heartbeat, RankFailure
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, timeout_s=0.5)
    dist.barrier()
    if rank == 0:
        time.sleep(2.0)                 # rank 0 hangs on the host and stops beating
        return
    deadline = time.time() + 5
    failed = None
    while time.time() < deadline and failed is None:
        hb.beat(0)
        try:
            hb.check()
        except RankFailure as e:
            failed = e.failed_rank
        time.sleep(0.1)
    assert failed == 0


def test_rank_leaving_between_steps_is_detected():
    run_distributed(_leaver, 3)


def test_silent_rank_is_detected_by_heartbeat_timeout():
    run_distributed(_silent, 2)


def _short_pg_timeout(rank, world, port):
    # second process group with a short timeout: a collective whose peer never joins raises instead of hanging
    os.environ["MASTER_PORT"] = str(port)
    pg = dist.new_group(list(range(world)), timeout=datetime.timedelta(seconds=2), backend="gloo")
    dist.barrier()
    if rank == 1:
        time.sleep(4.0)                 # never joins the collective in time
        return
    t = torch.ones(1)
    with pytest.raises(RuntimeError):
        dist.all_reduce(t, group=pg)


def test_collective_with_missing_peer_times_out():
    run_distributed(_short_pg_timeout, 2, _free_port())


def test_status_word_maps_to_exception():
    from rtp_b200.ops import _lib
    assert issubclass(_lib.RotationTimeout, RuntimeError)
    assert "peer" in _lib.STATUS_NAMES[2] and "slot" in _lib.STATUS_NAMES[3]
