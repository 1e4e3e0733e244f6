"""Logging, memory tracking, NVTX ranges, plan inspection and run artifacts.

* ``get_logger``: rank-aware logger (rank 0 also goes to stdout, every rank to ``<dir>/logs/rank{r}.log``),
  like the reference's per-rank files and tee (distca/utils/logging.py:96-216).
* ``MemoryLog``: torch allocated / peak / reserved (+ NVML used when available) appended to
  ``mem.rank{r}.jsonl`` (distca/mem.py:44-117, ``EXPERIMENT_LOG_MEMORY_USAGE``).
* ``nvtx_range``: NVTX push/pop context manager (the reference wraps every tick and phase,
  distca/runtime/megatron/ping_pong/transformer_block.py:242-341).
* ``inspect_plan``: per-pair megabyte matrix, largest per-rank buffer need and the time the traffic
  would take at a given bandwidth -> one ``plan_inspect.jsonl`` line
  (distca/utils/network_inspect.py:49-152, which assumes 40 MB/ms; NVLink 5 measured here is 770 MB/ms).
* ``RunArtifacts``: ``config.json``, ``benchmark.raw.jsonl``, ``benchmark.json`` and ``summary.log``
  (tests/test_e2e_combined.py:1699-1780).
"""
from __future__ import annotations

import contextlib
import json
import logging
import os
import statistics
import sys
import time

import torch


def get_logger(name: str = "distca_b200", rank: int = 0, out_dir: str | None = None,
               level: str | int | None = None) -> logging.Logger:
    log = logging.getLogger(f"{name}.r{rank}")
    if log.handlers:
        return log
    lvl = level if level is not None else os.environ.get("DISTCA_LOG_LEVEL", "INFO")
    log.setLevel(lvl)
    log.propagate = False
    fmt = logging.Formatter(f"[%(asctime)s r{rank} %(levelname).1s] %(message)s", "%H:%M:%S")
    if rank == 0 or os.environ.get("DISTCA_LOG_ALL_RANKS", "0") == "1":
        h = logging.StreamHandler(sys.stdout)
        h.setFormatter(fmt)
        log.addHandler(h)
    if out_dir:
        os.makedirs(os.path.join(out_dir, "logs"), exist_ok=True)
        fh = logging.FileHandler(os.path.join(out_dir, "logs", f"rank{rank}.log"))
        fh.setFormatter(fmt)
        log.addHandler(fh)
    return log


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class MemoryHistory:
    """Allocation history of the PyTorch caching allocator: ``start()`` begins recording, an out-of-memory error
    writes ``oom.rank{r}.pickle`` (the state at the failing allocation), ``dump()`` writes
    ``memory.rank{r}.pickle`` (e.g. after the first steps); both open in PyTorch's memory visualiser. The
    reference does this under ``--record-memory-history`` (distca/runtime/megatron/model_patch.py:204-215) and
    plots a timeline in its tests (tests/test_megatron_e2e.py:395-424). The peer arenas are ``cudaMalloc``'d by
    this repository's library and do not appear there: ``MemoryLog`` reports them through NVML. Without a GPU
    every method does nothing and returns ``None``."""

    def __init__(self, out_dir: str | None, rank: int, max_entries: int = 100000):
        self.dir, self.rank, self.max_entries = out_dir, rank, max_entries
        self.active = False

    def _path(self, stem: str) -> str:
        os.makedirs(self.dir, exist_ok=True)
        return os.path.join(self.dir, f"{stem}.rank{self.rank}.pickle")

    def start(self):
        if self.dir is None or not torch.cuda.is_available():
            return None
        torch.cuda.memory._record_memory_history(max_entries=self.max_entries)
        self.active = True

        def on_oom(device, alloc, device_alloc, device_free):
            torch.cuda.memory._dump_snapshot(self._path("oom"))
        torch._C._cuda_attach_out_of_memory_observer(on_oom)
        return self

    def dump(self):
        if not self.active:
            return None
        path = self._path("memory")
        torch.cuda.memory._dump_snapshot(path)
        return path

    def stop(self) -> None:
        if self.active:
            torch.cuda.memory._record_memory_history(enabled=None)
            self.active = False


class MemoryLog:
    def __init__(self, out_dir: str | None, rank: int, enabled: bool = True):
        self.enabled = enabled and out_dir is not None
        self.path = os.path.join(out_dir, f"mem.rank{rank}.jsonl") if self.enabled else None
        self.rank = rank
        self._nvml = None
        if self.enabled:
            os.makedirs(out_dir, exist_ok=True)
            try:
                import pynvml
                pynvml.nvmlInit()
                self._nvml = pynvml
            except Exception:
                self._nvml = None

    def log(self, tag: str, **extra) -> dict:
        rec = {"tag": tag, "t": time.time(), "rank": self.rank, **extra}
        if torch.cuda.is_available():
            gib = float(1 << 30)
            rec.update(allocated_gib=torch.cuda.memory_allocated() / gib,
                       peak_gib=torch.cuda.max_memory_allocated() / gib,
                       reserved_gib=torch.cuda.memory_reserved() / gib)
            if self._nvml is not None:
                try:
                    h = self._nvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
                    rec["nvml_used_gib"] = self._nvml.nvmlDeviceGetMemoryInfo(h).used / gib
                except Exception:
                    pass
        if self.enabled:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
        return rec


def inspect_plan(plan, world: int, link_mb_per_ms: float = 770.0) -> dict:
    """Traffic summary of one CAD plan (forward dispatch bytes; the return path moves the Q part back)."""
    mat = [[int(x) for x in plan.rank(r).send_bytes] for r in range(world)]
    out_b = [sum(v for j, v in enumerate(row) if j != i) for i, row in enumerate(mat)]
    in_b = [sum(mat[i][j] for i in range(world) if i != j) for j in range(world)]
    worst = max(out_b + in_b) if world > 1 else 0
    return {
        "world": world,
        "mb_matrix": [[round(v / 1e6, 3) for v in row] for row in mat],
        "max_send_mb": max(out_b) / 1e6 if out_b else 0.0,
        "max_recv_mb": max(in_b) / 1e6 if in_b else 0.0,
        "q_rows": [int(plan.rank(r).q_rows) for r in range(world)],
        "kv_rows": [int(plan.rank(r).kv_rows) for r in range(world)],
        "est_dispatch_ms": worst / 1e6 / link_mb_per_ms,
        "imbalance_before": plan.imbalance_before,
        "imbalance_after": plan.imbalance_after,
        "tolerance": plan.tolerance_used,
    }


class RunArtifacts:
    def __init__(self, out_dir: str | None, rank: int):
        self.dir, self.rank = out_dir, rank
        self.records: list[dict] = []
        if out_dir and rank == 0:
            os.makedirs(out_dir, exist_ok=True)

    def write_config(self, cfg: dict) -> None:
        if self.dir and self.rank == 0:
            with open(os.path.join(self.dir, "config.json"), "w") as f:
                json.dump(cfg, f, indent=2, default=str)

    def step(self, rec: dict) -> None:
        self.records.append(rec)
        if self.dir and self.rank == 0:
            with open(os.path.join(self.dir, "benchmark.raw.jsonl"), "a") as f:
                f.write(json.dumps(rec, default=float) + "\n")

    def plan(self, rec: dict) -> None:
        if self.dir and self.rank == 0:
            with open(os.path.join(self.dir, "plan_inspect.jsonl"), "a") as f:
                f.write(json.dumps(rec, default=float) + "\n")

    def finish(self, warmup: int = 1) -> dict:
        recs = self.records[warmup:] or self.records
        if not recs:
            return {}
        ms = [r["step_ms"] for r in recs]
        tps = [r["tokens_per_s"] for r in recs]
        summary = {"steps": len(recs), "mean_step_ms": statistics.fmean(ms), "median_step_ms": statistics.median(ms),
                   "mean_tokens_per_s": statistics.fmean(tps), "last_loss": recs[-1].get("loss")}
        for k in ("exposed_dispatch_ms", "attn_imbalance"):
            vals = [r[k] for r in recs if r.get(k) is not None]
            if vals:
                summary[f"mean_{k}"] = statistics.fmean(vals)
        if self.dir and self.rank == 0:
            with open(os.path.join(self.dir, "benchmark.json"), "w") as f:
                json.dump(summary, f, indent=2)
            with open(os.path.join(self.dir, "summary.log"), "w") as f:
                for k, v in summary.items():
                    f.write(f"{k}: {v}\n")
        return summary


class MetricsSink:
    """Per-step metrics to Weights & Biases when the package is installed and ``enabled``; otherwise (no
    network / no package) the same records go to ``<out_dir>/metrics.offline.jsonl`` so a run can be
    uploaded later. Only rank 0 reports, like the reference (distca/utils/wandb_driver.py:89-132)."""

    def __init__(self, enabled: bool, rank: int, project: str, run_name: str | None, config: dict,
                 out_dir: str | None):
        self.run, self.file = None, None
        if not enabled or rank != 0:
            return
        try:
            import wandb  # noqa: F401
            self.run = wandb.init(project=project, name=run_name, config=config)
        except Exception:     # not installed, or no network to log in with
            if out_dir:
                os.makedirs(out_dir, exist_ok=True)
                self.file = open(os.path.join(out_dir, "metrics.offline.jsonl"), "a")

    def log(self, record: dict) -> None:
        flat = {k: v for k, v in record.items() if isinstance(v, (int, float)) and v is not None}
        if self.run is not None:
            self.run.log(flat, step=int(record.get("step", 0)))
        elif self.file is not None:
            self.file.write(json.dumps(flat) + "\n")
            self.file.flush()

    def close(self) -> None:
        if self.run is not None:
            self.run.finish()
        if self.file is not None:
            self.file.close()


def fused_path_rooflines(phases_ms: dict, steps: int, *, tokens_per_rank: int, hidden: int, qkv_dim: int, layers: int,
                         passes_qkv: int, attn_flops_fwd_per_rank: float, remote_dispatch_bytes: float,
                         remote_return_bytes: float, grad_bytes_in: float, param_bytes_out: float,
                         optimizer_hbm_bytes: float, peaks: dict) -> dict:
    """Achieved / roofline of every fused compute + communication path of one step, from the CUDA-event phase
    timers. The roofline time of a path is the slower of its FLOPs at the GEMM peak, its bytes over NVLink at the
    link bandwidth and its bytes through HBM at the copy bandwidth (``peaks``: ``bf16_tflops``, ``hbm_gbs``,
    ``link_gbs``). Times are per step and per rank; a fraction near 1 means the path runs at its roofline."""
    def ph(*names):
        return sum(v for k, v in phases_ms.items() if k.removeprefix("re_") in names) / max(1, steps)

    def row(ms, flops=0.0, link_bytes=0.0, hbm_bytes=0.0):
        t_f = flops / (peaks["bf16_tflops"] * 1e12) * 1e3
        t_l = link_bytes / (peaks["link_gbs"] * 1e9) * 1e3
        t_h = hbm_bytes / (peaks["hbm_gbs"] * 1e9) * 1e3
        roof = max(t_f, t_l, t_h)
        bound = {t_f: "tensor", t_l: "nvlink", t_h: "hbm"}[roof]
        return {"ms": round(ms, 2), "roofline_ms": round(roof, 2), "bound": bound,
                "fraction_of_roofline": round(roof / ms, 3) if ms > 0 else None}
    out = {}
    qkv_flops = 2.0 * tokens_per_rank * hidden * qkv_dim * layers * passes_qkv
    out["qkv_gemm_rope_dispatch"] = row(ph("gemm_qkv"), qkv_flops, remote_dispatch_bytes * layers * passes_qkv)
    out["attention_forward_with_output_return"] = row(ph("cad_attn_fwd"), attn_flops_fwd_per_rank,
                                                      remote_return_bytes * layers)
    out["attention_backward_with_gradient_return"] = row(ph("cad_attn_bwd"), 2.5 * attn_flops_fwd_per_rank,
                                                         (remote_dispatch_bytes + remote_return_bytes) * layers)
    out["gradient_reduce_scatter_adam_all_gather"] = row(ph("optimizer"), 0.0, grad_bytes_in + param_bytes_out,
                                                         optimizer_hbm_bytes)
    return out
