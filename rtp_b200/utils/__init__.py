"""Run-time utilities: device timing, metrics/JSONL logging, host-side watchdog, synthetic data."""
from .timing import DeviceTimer, max_over_ranks  # noqa: F401
from .metrics import MetricsLogger, peak_memory_gib  # noqa: F401
from .watchdog import Heartbeat, RankFailure  # noqa: F401
