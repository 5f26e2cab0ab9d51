"""Host-side failure detection for a ring.

The reference has none: a dead rank hangs NCCL forever.  Here (1) every device-side wait is bounded and reports
through a status word (``rtp_b200.ops._lib.RotationTimeout``), and (2) ranks publish a heartbeat in the
process-group store between steps; a rank whose peer stopped beating learns of it on the host *before* it launches
the next rotation kernel and raises ``RankFailure`` instead of waiting on a counter that will never move.
Recovery is restart from a sharded checkpoint (optionally on a smaller ring: ``checkpoint.load_sharded``).
"""
import threading
import time
from typing import Optional



class RankFailure(RuntimeError):
    def __init__(self, rank: int, age: float):
        super().__init__(f"rank {rank} has not published a heartbeat for {age:.1f} s")
        self.failed_rank = rank


class Heartbeat:
    """``hb = Heartbeat(store, rank, world); hb.beat(step)`` after every step; ``hb.check()`` before every step."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "rtp_hb"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s, self.prefix = timeout_s, prefix
        self._last_seen = {r: (None, time.time()) for r in range(world)}
        self.beat(-1)

    def _key(self, r):
        return f"{self.prefix}/{r}"

    def beat(self, step: int):
        self.store.set(self._key(self.rank), f"{step}:{time.time()}")

    def leave(self):
        """Announce an orderly exit between steps (no kernels or collectives in flight)."""
        self.store.set(self._key(self.rank), "left:0")

    def check(self):
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = self.store.get(self._key(r)).decode()
            except Exception:
                val = None
            if val is not None and val.startswith("left"):
                raise RankFailure(r, 0.0)
            prev, seen = self._last_seen[r]
            if val != prev:
                self._last_seen[r] = (val, now)
            elif now - seen > self.timeout_s:
                raise RankFailure(r, now - seen)


class StatusWatchdog(threading.Thread):
    """Polls a callable (e.g. ``engine.check_all``) and records the first exception; the training loop reads
    ``.error`` between steps. The poll synchronises the stream, so use a coarse period."""

    def __init__(self, poll, period_s: float = 5.0):
        super().__init__(daemon=True)
        self.poll, self.period_s = poll, period_s
        self.error: Optional[BaseException] = None
        self._stop_evt = threading.Event()

    def run(self):
        while not self._stop_evt.wait(self.period_s):
            try:
                self.poll()
            except BaseException as e:  # noqa: BLE001
                self.error = e
                return

    def stop(self):
        self._stop_evt.set()
