"""Helper of tests/test_bench_cpu.py (not a test): runs ``bench.main()`` on CPU ranks with wall-clock stand-ins for
the few CUDA timing calls it makes, so that everything else of the benchmark program (batch staging, the timed
loops, the reductions over ranks, the JSON line with its roofline and balance blocks) is executed without a GPU."""
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class _Event:
    def __init__(self, enable_timing=False):
        self.t = None

    def record(self, stream=None):
        self.t = time.perf_counter()

    def elapsed_time(self, other):
        return (other.t - self.t) * 1e3

    def synchronize(self):
        pass


torch.cuda.Event = _Event
torch.cuda.synchronize = lambda *a, **k: None
torch.cuda.reset_peak_memory_stats = lambda *a, **k: None
torch.cuda.mem_get_info = lambda *a, **k: (1 << 30, 2 << 30)

import bench  # noqa: E402

if __name__ == "__main__":
    sys.argv = ["bench.py", "--gpus", os.environ.get("WORLD_SIZE", "1"), "--model", "tiny", "--seq-len", "1024",
                "--steps", "1", "--warmup", "1", "--dist", "loguniform64"] + sys.argv[1:]
    bench.main()
