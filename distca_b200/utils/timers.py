"""Device-side phase timers (CUDA events on the launching stream; no host synchronisation
until :meth:`PhaseTimers.summary` is called). Disabled timers cost one dict lookup.

The reference records per-tick CUDA-event timings behind ``UNIFIED_RECORD_TICK_TIMES``
(distca/runtime/megatron/ping_pong/tick_ops.py:368-444).
"""
from __future__ import annotations

from collections import defaultdict
from contextlib import contextmanager

import torch


class PhaseTimers:
    """``phase(name)`` brackets a piece of a step. With ``enabled`` it records a CUDA-event pair (device time,
    read back in :meth:`summary`); with ``nvtx`` it also opens an NVTX range of that name, so a timeline shows
    every phase of every layer and tick (the reference's per-tick / per-phase ranges,
    distca/runtime/megatron/ping_pong/transformer_block.py:242-341)."""

    def __init__(self, enabled: bool = False, nvtx: bool = False):
        self.prefix = ""            # prepended to phase names (the recompute pass reports as "re_<phase>")
        self.enabled = enabled and torch.cuda.is_available()
        self.nvtx = nvtx and torch.cuda.is_available()
        self._pairs: dict[str, list] = defaultdict(list)

    @contextmanager
    def phase(self, name: str):
        if not self.enabled and not self.nvtx:
            yield
            return
        name = self.prefix + name
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)
        if self.enabled:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        try:
            yield
        finally:
            if self.enabled:
                b.record()
                self._pairs[name].append((a, b))
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    def summary(self, reset: bool = True) -> dict[str, float]:
        """Total milliseconds per phase since the last reset (synchronises the device)."""
        if not self.enabled:
            return {}
        torch.cuda.synchronize()
        out = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self._pairs.items()}
        if reset:
            self._pairs.clear()
        return out


GLOBAL = PhaseTimers(False)


def enable(flag: bool = True) -> None:
    GLOBAL.enabled = flag and torch.cuda.is_available()


def enable_nvtx(flag: bool = True) -> None:
    """NVTX ranges for every phase (and, through :func:`layer`, every layer pass)."""
    GLOBAL.nvtx = flag and torch.cuda.is_available()


@contextmanager
def layer(kind: str, index: int):
    """NVTX range around one layer's forward / recompute / backward; phases inside a recompute pass are
    reported under ``re_<phase>`` so that forward and recompute time can be told apart."""
    old = GLOBAL.prefix
    if kind == "recompute":
        GLOBAL.prefix = "re_"
    if GLOBAL.nvtx:
        torch.cuda.nvtx.range_push(f"{kind}.layer{index}")
    try:
        yield
    finally:
        GLOBAL.prefix = old
        if GLOBAL.nvtx:
            torch.cuda.nvtx.range_pop()


def phase(name: str):
    return GLOBAL.phase(name)
