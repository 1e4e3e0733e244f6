"""Optional tracing helpers: a ``torch.profiler`` context that writes a chrome trace for a window
of steps, and a Python call tracer for "where is this rank stuck" questions.

Reference: distca/utils/torch_profiler.py:7-44 (``ProfilerCtx``), distca/utils/traceback.py:42-84
(``TraceFunctions``). Device-side timing of this repository's own phases is in ``utils/timers.py``.
"""
from __future__ import annotations

import os
import sys
import time


class ProfilerCtx:
    """``with ProfilerCtx(out_dir, rank, enabled): step()`` -> ``<out_dir>/trace.rank{r}.json``."""

    def __init__(self, out_dir: str | None, rank: int = 0, enabled: bool = True, with_stack: bool = False):
        self.path = os.path.join(out_dir, f"trace.rank{rank}.json") if out_dir else None
        self.enabled = enabled and self.path is not None
        self.with_stack = with_stack
        self.prof = None

    def __enter__(self):
        if self.enabled:
            import torch
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            os.makedirs(os.path.dirname(self.path), exist_ok=True)
            self.prof = torch.profiler.profile(activities=acts, with_stack=self.with_stack, record_shapes=False)
            self.prof.__enter__()
        return self

    def __exit__(self, *exc):
        if self.prof is not None:
            self.prof.__exit__(*exc)
            self.prof.export_chrome_trace(self.path)
        return False


class TraceFunctions:
    """Logs every Python call (and return, with its duration) of functions whose file path contains
    ``match`` while the context is active. Heavy: for debugging a hang on one rank, not for timing."""

    def __init__(self, match: str = "distca_b200", out=None, max_depth: int = 6):
        self.match, self.out, self.max_depth = match, out or sys.stderr, max_depth
        self.depth = 0
        self.t0: list[float] = []

    def _trace(self, frame, event, arg):
        code = frame.f_code
        if self.match not in code.co_filename:
            return None
        if event == "call":
            if self.depth < self.max_depth:
                self.out.write(f"{'  ' * self.depth}-> {code.co_name} ({os.path.basename(code.co_filename)}:{frame.f_lineno})\n")
            self.depth += 1
            self.t0.append(time.perf_counter())
            return self._trace
        if event == "return":
            self.depth = max(0, self.depth - 1)
            dt = (time.perf_counter() - self.t0.pop()) * 1e3 if self.t0 else 0.0
            if self.depth < self.max_depth:
                self.out.write(f"{'  ' * self.depth}<- {code.co_name} {dt:.2f} ms\n")
        return self._trace

    def __enter__(self):
        sys.settrace(self._trace)
        return self

    def __exit__(self, *exc):
        sys.settrace(None)
        return False


def install_rank_excepthook(rank: int | None = None, out=None) -> None:
    """Uncaught exceptions print as ``path:line: in function`` lines (clickable in editors and CI logs) followed by
    the error with the rank in front, so that in the interleaved output of many ranks it is clear who failed
    where. Reference: distca/utils/traceback.py:15-33 (``EXPERIMENT_PYTHON_BETTER_TRACEBACK``)."""
    import traceback

    def hook(exc_type, exc, tb):
        f = out or sys.stderr
        r = rank
        if r is None:
            try:
                import torch.distributed as dist
                r = dist.get_rank() if dist.is_initialized() else int(os.environ.get("RANK", "0"))
            except Exception:
                r = int(os.environ.get("RANK", "0"))
        for fr in traceback.extract_tb(tb):
            f.write(f"{os.path.abspath(fr.filename)}:{fr.lineno}: in {fr.name}\n")
            if fr.line:
                f.write(f"    {fr.line}\n")
        f.write(f"[rank {r}] {exc_type.__name__}: {exc}\n")
        f.flush()
    sys.excepthook = hook
