"""Python face of the C++ CAD planner (``distca_b200._planner``, built from ``csrc/planner``).

``Planner.plan(docs_per_seq)`` lays the documents out on the ranks, balances core-attention work
across the attention servers and returns a ``Plan`` whose per-rank tables drive the runtime
(:mod:`distca_b200.parallel.cad`). ``AsyncPlanner`` plans the next step on a host thread while the
current one runs (the C++ calls release the GIL).

Reference counterparts: ``Planner`` / ``Item`` / ``batch_to_items_*`` / ``cp_list_to_mlp_list``
(distca/planner/planner.py:58-328, 550-829) and ``from_planner_output``
(distca/runtime/compute_metadata.py:642-734).
"""
from __future__ import annotations

import importlib
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass

from ..models.config import ModelConfig


def _ext():
    try:
        return importlib.import_module("distca_b200._planner")
    except ImportError:
        from .. import build
        build.build_planner()
        return importlib.import_module("distca_b200._planner")


def chunk_flops(q: int, kv: int) -> int:
    """Query-key pairs of ``q`` queries whose last one sees ``kv`` keys (bottom-right causal)."""
    return q * kv - (q * (q - 1)) // 2


@dataclass
class PlannerConfig:
    world: int                       # attention-server ranks (dp x pp)
    tokens_per_rank: int
    tolerance: float = 0.1
    q_row_bytes: int = 8192
    kv_row_bytes: int = 2048
    max_q_rows: int = 0              # arena capacity (rows) per server; 0 = unlimited
    max_kv_rows: int = 0
    per_task_overhead_flops: float = 0.0
    cost_model: dict | None = None   # see default_cost_model(); None = balance query-key pairs like the reference
    speed: list | None = None        # relative speed per server (None = equal shares)

    @staticmethod
    def for_model(cfg: ModelConfig, world: int, tokens_per_rank: int, tp: int = 1, elt: int = 2,
                  **kw) -> "PlannerConfig":
        return PlannerConfig(world=world, tokens_per_rank=tokens_per_rank,
                             q_row_bytes=cfg.q_dim // tp * elt, kv_row_bytes=cfg.kv_dim // tp * elt, **kw)


class Planner:
    def __init__(self, cfg: PlannerConfig):
        self.cfg = cfg
        self.ext = _ext()
        o = self.ext.PlannerOptions()
        o.world, o.tokens_per_rank, o.tolerance = cfg.world, cfg.tokens_per_rank, cfg.tolerance
        d = self.ext.ModelDims()
        d.q_row_bytes, d.kv_row_bytes = cfg.q_row_bytes, cfg.kv_row_bytes
        o.dims = d
        o.max_q_rows, o.max_kv_rows = cfg.max_q_rows, cfg.max_kv_rows
        o.per_task_overhead_flops = cfg.per_task_overhead_flops
        if cfg.cost_model:
            c = self.ext.CostModel()
            c.enabled = True
            c.tile = int(cfg.cost_model.get("tile", 128))
            c.ms_per_tile_pair = float(cfg.cost_model["ms_per_tile_pair"])
            c.ms_per_q_tile = float(cfg.cost_model.get("ms_per_q_tile", 0.0))
            c.ms_per_task = float(cfg.cost_model.get("ms_per_task", 0.0))
            o.cost = c
        if cfg.speed is not None:
            o.speed = [float(v) for v in cfg.speed]
        self.options = o
        self.dims = d

    def set_speed(self, speed) -> None:
        """Relative speed of every attention server (``None`` = equal): the balancer gives server ``r`` the
        share ``speed[r] / sum(speed)`` of the predicted attention time. Fed back by the runtime from the
        measured time of earlier steps."""
        self.options.speed = [] if speed is None else [float(v) for v in speed]

    def plan(self, docs_per_seq: list[list[int]], with_dummy: bool = False):
        """``docs_per_seq``: document lengths of every sequence of the batch, in rank order."""
        return self.ext.plan_batch([list(map(int, b)) for b in docs_per_seq], self.options, with_dummy)

    def plan_fixed(self, docs_per_rank: list[list[int]]):
        """Plan for documents that already live on their ranks (``docs_per_rank[r]`` may be empty)."""
        return self.ext.plan_fixed([list(map(int, b)) for b in docs_per_rank], self.options)

    def plan_fixed_cp(self, docs_per_rank: list[list[int]], min_len: int = 0):
        """Baseline: per-document context parallelism (every document of at least ``min_len`` tokens is cut
        into 2 x world chunks, head-tail paired over the servers; no balancer). The reference's
        comparison point is Megatron context parallelism with per-document masks
        (distca/runtime/megatron/per_doc_cp_attn.py)."""
        min_len = min_len or 2 * 128 * self.cfg.world
        return self.ext.plan_fixed_cp([list(map(int, b)) for b in docs_per_rank], self.options, int(min_len))

    def plan_fixed_water_fill(self, docs_per_rank: list[list[int]]):
        """Legacy policy: relocate only the single most expensive document, filling every other server
        up to the mean (the reference's first planner, distca/planner/equal_flops.py:168-379)."""
        return self.ext.plan_fixed_water_fill([list(map(int, b)) for b in docs_per_rank], self.options)

    def items(self, docs_per_seq, with_dummy: bool = False) -> list[dict]:
        f = self.ext.batch_to_items_with_dummy if with_dummy else self.ext.batch_to_items
        return f([list(map(int, b)) for b in docs_per_seq], self.cfg.tokens_per_rank, self.cfg.world)

    def balanced_items(self, docs_per_seq) -> list[dict]:
        return self.ext.balance_only([list(map(int, b)) for b in docs_per_seq], self.options)

    def fa2a_matrices(self, plan):
        return self.ext.fa2a_matrices(plan, self.dims)

    def simulate(self, plan, time_model):
        return self.ext.simulate(plan, time_model, self.dims)


def cp_list_to_mlp_list(cp_list, world: int, tokens_per_rank: int) -> list[list[int]]:
    return _ext().cp_list_to_mlp_list([list(map(int, b)) for b in cp_list], world, tokens_per_rank)


class AsyncPlanner:
    """Plans ahead on a worker thread: ``submit`` the documents of step N+1, ``result`` when needed."""

    def __init__(self, planner: Planner):
        self.planner = planner
        self.pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="cad-planner")
        self._pending: dict[int, Future] = {}

    def submit(self, step: int, docs_per_seq, post=None) -> None:
        def work():
            plan = self.planner.plan(docs_per_seq)
            return post(plan) if post is not None else plan
        self._pending[step] = self.pool.submit(work)

    def result(self, step: int):
        return self._pending.pop(step).result()

    def shutdown(self) -> None:
        self.pool.shutdown(wait=False, cancel_futures=True)


def default_cost_model(heads_q: int = 32, kind: str = "b200") -> dict:
    """Tile-granular cost of core attention, forward + backward, for the balancer (``PlannerConfig.cost_model``).

    ``b200``: least-squares fit of ``ms = a * tile_pairs + b * query_tiles`` to this repository's kernels on one
    B200 with 32 query / 8 KV heads of 128 (``kernel_bench --kernel attn_fwd / attn_bwd``: one document of 8192
    tokens 0.535 + 1.732 ms, of 32768 tokens 7.24 + 25.59 ms, sixteen of 2048 tokens 0.664 + 2.035 ms), scaled
    by the number of query heads on the rank. A query tile costs as much as 3.6 tile pairs, so a server full of
    short documents is slower per query-key pair than one holding a single long document, which counting pairs
    alone (the reference's balancer, distca/planner/planner.py:366-378) does not see."""
    if kind != "b200":
        raise ValueError(kind)
    s = heads_q / 32.0
    return {"tile": 128, "ms_per_tile_pair": 9.68e-4 * s, "ms_per_q_tile": 3.5e-3 * s, "ms_per_task": 0.0}


def _sweep_rows(source) -> list[dict]:
    """Rows of ``python -m distca_b200.utils.kernel_bench --kernel attn_sweep`` (one JSON object per line; a path, an
    open file or an iterable of lines / dicts). Lines that are not sweep rows are skipped."""
    import json
    if isinstance(source, (str, bytes)) or hasattr(source, "__fspath__"):
        with open(source) as f:
            lines = list(f)
    else:
        lines = list(source)
    rows = []
    for ln in lines:
        if isinstance(ln, dict):
            d = ln
        else:
            ln = ln.strip()
            if not ln.startswith("{"):
                continue
            try:
                d = json.loads(ln)
            except ValueError:
                continue
        if d.get("kernel") == "attn_sweep" and "fwd_ms" in d and "bwd_ms" in d:
            rows.append(d)
    return rows


def cost_model_from_sweep(source, heads_q: int | None = None, tile: int = 128) -> dict:
    """Fit the balancer's cost model to a measured sweep: relative least squares of
    ``fwd_ms + bwd_ms = a * tile_pairs + b * query_tiles`` over the sweep's workloads (every workload counts alike,
    whatever its size). ``heads_q``: query heads on the rank the model is for (default: the sweep's own); the
    constants scale with it. This is how the constants of :func:`default_cost_model` are re-derived for another
    GPU, clock or kernel version (the reference loads its profile tables the same way,
    distca/timemodule/compute.py:23-72)."""
    import numpy as np
    rows = _sweep_rows(source)
    if len(rows) < 2:
        raise ValueError("a cost-model fit needs at least two attn_sweep rows")
    X, y = [], []
    for d in rows:
        n = int(d["seqlen"]) // tile
        docs = int(d.get("docs", 1))
        X.append([float(d.get("tile_pairs", docs * n * (n + 1) // 2)), float(d.get("query_tiles", docs * n))])
        y.append(float(d["fwd_ms"]) + float(d["bwd_ms"]))
    X, y = np.asarray(X), np.asarray(y)
    w = 1.0 / y
    coef, *_ = np.linalg.lstsq(X * w[:, None], y * w, rcond=None)
    a, b = float(coef[0]), float(max(coef[1], 0.0))
    if a <= 0.0:
        raise ValueError(f"fit gave a non-positive cost per tile pair ({a}); the sweep does not span enough lengths")
    pred = X @ np.array([a, b])
    sweep_heads = int(rows[0].get("heads", [32])[0]) if isinstance(rows[0].get("heads"), (list, tuple)) else 32
    s = (heads_q or sweep_heads) / float(sweep_heads)
    return {"tile": tile, "ms_per_tile_pair": a * s, "ms_per_q_tile": b * s, "ms_per_task": 0.0,
            "max_rel_err": float(np.max(np.abs(pred - y) / y)), "workloads": len(rows)}


def time_model_from_sweep(source, base: str = "b200"):
    """The simulator's time model with its attention table replaced by the sweep's whole-document forward times
    (rows with one document), everything else as in :func:`default_time_model`."""
    rows = sorted((r for r in _sweep_rows(source) if int(r.get("docs", 1)) == 1), key=lambda r: int(r["seqlen"]))
    if len(rows) < 2:
        raise ValueError("a time-model table needs at least two single-document attn_sweep rows")
    tm = default_time_model(base)
    tm.attn_len = [float(r["seqlen"]) for r in rows]
    tm.attn_ms = [float(r["fwd_ms"]) for r in rows]
    return tm


class NetworkModel:
    """Time of a collective as a function of the bytes one rank moves: per ``(operation, world size)`` a table
    of measured ``(bytes, milliseconds)`` points, interpolated linearly; below the smallest point the time is that
    point's (launch and signalling latency), above the largest it grows in proportion (bandwidth). World sizes
    without a table use the nearest measured one. The reference keeps the same kind of tables for NCCL all-reduce
    and all-gather on H100 (distca/timemodule/network.py:3-97); these are filled by
    ``python -m distca_b200.utils.net_bench`` (:meth:`from_sweep`)."""

    def __init__(self, tables: dict | None = None):
        self.tables: dict = {}
        for (op, world), pts in (tables or {}).items():
            self.tables[(op, int(world))] = sorted((float(b), float(ms)) for b, ms in pts)

    def ops(self) -> list:
        return sorted({op for op, _ in self.tables})

    def ms(self, op: str, world: int, nbytes: float) -> float:
        if world <= 1 or nbytes <= 0:
            return 0.0
        worlds = [w for o, w in self.tables if o == op]
        if not worlds:
            raise KeyError(f"no table for {op!r}")
        pts = self.tables[(op, min(worlds, key=lambda w: (abs(w - world), w)))]
        if nbytes <= pts[0][0]:
            return pts[0][1]
        if nbytes >= pts[-1][0]:
            return pts[-1][1] * nbytes / pts[-1][0]
        for (b0, t0), (b1, t1) in zip(pts, pts[1:]):
            if b0 <= nbytes <= b1:
                return t0 + (t1 - t0) * (nbytes - b0) / (b1 - b0)
        return pts[-1][1]

    def gbytes_per_s(self, op: str, world: int, nbytes: float) -> float:
        t = self.ms(op, world, nbytes)
        return nbytes / t / 1e6 if t > 0 else 0.0

    @staticmethod
    def from_sweep(source) -> "NetworkModel":
        """From the JSON lines of ``net_bench`` (``{"kernel": "net_sweep", "op", "world", "bytes_per_rank", "ms"}``)."""
        import json
        if isinstance(source, (str, bytes)) or hasattr(source, "__fspath__"):
            with open(source) as f:
                lines = list(f)
        else:
            lines = list(source)
        tables: dict = {}
        for ln in lines:
            if not isinstance(ln, dict):
                ln = ln.strip()
                if not ln.startswith("{"):
                    continue
                try:
                    ln = json.loads(ln)
                except ValueError:
                    continue
            if ln.get("kernel") == "net_sweep" and ln.get("ms") is not None:
                tables.setdefault((ln["op"], int(ln["world"])), []).append((ln["bytes_per_rank"], ln["ms"]))
        if not tables:
            raise ValueError("no net_sweep rows")
        return NetworkModel(tables)


def default_network_model(kind: str = "b200") -> NetworkModel:
    """Measured on one 8 x B200 NVSwitch box (CUDA events, maximum over ranks, bytes = what one rank sends to other
    GPUs): ``push`` is this repository's peer-store kernel together with its signal round trip (the dispatch
    micro-benchmark), ``all_to_all`` the pack + NCCL ``all_to_all_single`` + unpack twin of the same traffic,
    ``all_reduce`` NCCL at 1 GiB (725 GB/s bus bandwidth), ``peer_copy`` a plain copy into a peer's memory
    (770 GB/s per direction)."""
    if kind != "b200":
        raise ValueError(kind)
    MB = 1e6
    return NetworkModel({
        ("push", 2): [(23.9 * MB, 0.098), (297.1 * MB, 0.772)],
        ("push", 8): [(24.5 * MB, 0.145), (1038.4 * MB, 1.937)],
        ("all_to_all", 2): [(23.9 * MB, 0.236), (297.1 * MB, 2.535)],
        ("all_to_all", 8): [(24.5 * MB, 0.528), (1038.4 * MB, 3.597)],
        ("all_reduce", 8): [(2**30, 2.0 * (7 / 8) * 2**30 / 725e9 * 1e3)],
        ("peer_copy", 2): [(2**30, 2**30 / 770e9 * 1e3)],
    })


def default_time_model(kind: str = "b200"):
    """Attention/linear cost tables. ``b200``: measured with this repository's kernels on one B200
    (whole causal document, 32 query / 8 KV heads of 128, forward); ``h100``: the reference's
    FlashAttention-2 profile (distca/profiling/data/compute-attn-H100.csv, 64/4 heads)."""
    tm = _ext().TimeModel()
    if kind == "b200":
        tm.attn_len = [2048.0, 8192.0, 32768.0, 131072.0]
        tm.attn_ms = [0.0415, 0.535, 7.24, 112.0]
        # everything of a Llama-3-8B layer that is not core attention, forward only, per token, from the phase
        # timers of a 128K-token step on one GPU (GEMMs forward 1443 ms + norms + SwiGLU over 32 layers)
        tm.linear_ms_per_token = 1480.0 / 32 / 131072
        tm.link_gbytes_per_s = 770.0
    elif kind == "h100":
        tm.attn_len = [4096.0, 8192.0, 16384.0, 32768.0, 65536.0]
        tm.attn_ms = [1.06, 3.71, 13.50, 51.89, 206.29]
        tm.link_gbytes_per_s = 40.0
    else:
        raise ValueError(kind)
    return tm
