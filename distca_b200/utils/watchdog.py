"""Host-side failure detection: a step watchdog and a heartbeat over the process-group store.

* ``StepWatchdog``: if a step does not finish within the deadline the process reports and exits
  with a non-zero code instead of hanging the job (the reference arms ``SIGALRM`` around its first
  warm-up step because "it may suggest our all2all kernel failed",
  tests/test_e2e_combined.py:1383-1419).
* ``Heartbeat``: every rank bumps a key in a ``torch.distributed`` store between steps; ``dead_ranks``
  lists the ranks whose counter stopped, so survivors learn of a lost rank on the host, before
  their next launch, and never wait for it on the device.
"""
from __future__ import annotations

import os
import sys
import threading
import time
import traceback


class StepWatchdog:
    def __init__(self, timeout_s: float, what: str = "training step", on_timeout=None):
        self.timeout_s, self.what = timeout_s, what
        self.on_timeout = on_timeout
        self._timer: threading.Timer | None = None
        self.fired = False

    def _fire(self) -> None:
        self.fired = True
        if self.on_timeout is not None:
            self.on_timeout()
            return
        sys.stderr.write(f"[watchdog] {self.what} exceeded {self.timeout_s:.0f} s; stacks follow\n")
        for tid, frame in sys._current_frames().items():
            sys.stderr.write(f"--- thread {tid}\n" + "".join(traceback.format_stack(frame)))
        sys.stderr.flush()
        os._exit(3)

    def __enter__(self):
        self.fired = False
        self._timer = threading.Timer(self.timeout_s, self._fire)
        self._timer.daemon = True
        self._timer.start()
        return self

    def __exit__(self, *exc):
        if self._timer is not None:
            self._timer.cancel()
        return False


class Heartbeat:
    def __init__(self, store, rank: int, world: int, prefix: str = "hb"):
        self.store, self.rank, self.world, self.prefix = store, rank, world, prefix
        self._last: dict[int, tuple[int, float]] = {}

    def beat(self) -> None:
        self.store.add(f"{self.prefix}/{self.rank}", 1)

    def dead_ranks(self, stale_after_s: float) -> list[int]:
        """Ranks whose counter has not moved for ``stale_after_s`` seconds (as seen by this rank)."""
        now = time.time()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = int(self.store.add(f"{self.prefix}/{r}", 0))
            last = self._last.get(r)
            if last is None or v != last[0]:
                self._last[r] = (v, now)
            elif now - last[1] > stale_after_s:
                dead.append(r)
        return dead

    # ---- background beating: proves the PROCESS is alive while a long step runs ----
    def start(self, interval_s: float = 0.5) -> None:
        """Beat from a daemon thread every ``interval_s`` seconds until :meth:`stop` (or process exit)."""
        if getattr(self, "_thread", None) is not None:
            return
        self._stop = threading.Event()

        def run():
            while not self._stop.wait(interval_s):
                try:
                    self.beat()
                except Exception:       # the store went away (job shutting down)
                    return
        self.beat()
        self._thread = threading.Thread(target=run, name="distca-heartbeat", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        if getattr(self, "_thread", None) is not None:
            self._stop.set()
            self._thread.join(timeout=2.0)
            self._thread = None


class RankLost(RuntimeError):
    """Raised on the host, before the next launch, when another rank's heartbeat stopped."""


class StepGuard:
    """What both trainers put around every step: ``check()`` before anything is launched (raises
    :class:`RankLost` when a peer's heartbeat has stopped, so no kernel ever waits on the device for a rank
    that is gone) and ``watch()`` around the step (a step that exceeds the deadline dumps all Python stacks
    and ends the process with exit code 3). Heartbeats use the process group's own store; with a single
    process only the watchdog is active.

    Environment: ``DISTCA_STEP_TIMEOUT_S`` (default 3600), ``DISTCA_HEARTBEAT_STALE_S`` (default 10, 0 = off).
    """

    def __init__(self, rank: int = 0, world: int = 1, store=None, step_timeout_s: float | None = None,
                 stale_after_s: float | None = None, on_timeout=None, beat_interval_s: float = 0.5):
        self.step_timeout_s = float(os.environ.get("DISTCA_STEP_TIMEOUT_S", 3600.0)) if step_timeout_s is None else step_timeout_s
        self.stale_after_s = float(os.environ.get("DISTCA_HEARTBEAT_STALE_S", 10.0)) if stale_after_s is None else stale_after_s
        self.on_timeout = on_timeout
        self.hb = None
        if world > 1 and store is not None and self.stale_after_s > 0:
            self.hb = Heartbeat(store, rank, world, prefix="distca_hb")
            self.hb.start(beat_interval_s)
            self.hb.dead_ranks(self.stale_after_s)      # first observation of every peer's counter

    @staticmethod
    def for_process_group(**kw) -> "StepGuard":
        """Guard over the default process group's store (single process: watchdog only)."""
        import torch.distributed as dist
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return StepGuard(**kw)
        from torch.distributed.distributed_c10d import _get_default_store
        return StepGuard(dist.get_rank(), dist.get_world_size(), _get_default_store(), **kw)

    def check(self) -> None:
        if self.hb is not None:
            dead = self.hb.dead_ranks(self.stale_after_s)
            if dead:
                raise RankLost(f"ranks {dead} stopped sending heartbeats: not launching the next step")

    def watch(self, what: str = "training step") -> StepWatchdog:
        return StepWatchdog(self.step_timeout_s, what, self.on_timeout)

    def close(self) -> None:
        if self.hb is not None:
            self.hb.stop()
            self.hb = None
