"""Regression sweep over (model, layout, mode, document distribution) cases: one training run per case
through ``pretrain_llama.py``, results collected into one table.

    python -m distca_b200.sweep --output-dir runs/sweep --gpus-per-node 8 \\
        --case "llama3-8b 1 1 4 131072 distca 2 2 2 4d-cad" \\
        --case "llama3-8b 1 1 1 131072 baseline 4 1 2 4d-percp" \\
        --dist "mixture 0.0" --dist "prolong 0.3" --steps 5

A case is the reference's positional tuple (benchmarks/example-4d-parallel/run4d.sh:34-55, 49-121):

    model  nodes  batch  microbatches  tokens  mode  dp  pp  tp  [comment]

``mode``: ``distca`` (core-attention disaggregation), ``baseline`` (per-document context parallelism with
all-gathered K/V, no disaggregation), ``perseq`` (per-sequence context parallelism: packed sequences cut over the
ranks wherever their documents end), ``local`` (every rank attends to its own documents), ``wlbllm`` (the
reference's third arm: per-document CP attention over workload-balanced packs, ``--packing wlb``). ``--cases-file`` reads one case per line (``#`` comments).
A distribution is ``name change_long_doc_ratio``. ``nodes`` > 1 needs ``--nodes host1,host2,...`` (ssh, see
:mod:`distca_b200.launch`). ``--dry-run`` (or ``DRY_RUN=1``) prints the commands only.

Every run writes its own directory under ``--output-dir`` (``config.json``, ``benchmark.json``,
``benchmark.raw.jsonl``, ``plan_inspect.jsonl``, logs); the sweep appends one line per finished case to
``sweep.jsonl`` and prints a table at the end. A case that fails (non-zero exit, e.g. the pre-flight memory
estimate with ``--quit-if-maybe-oom``) is recorded with its exit code and the sweep goes on.
"""
from __future__ import annotations

import argparse
import json
import os
import shlex
import sys
import time
from dataclasses import asdict, dataclass

from . import launch

MODES = ("distca", "baseline", "perseq", "local", "wlbllm")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@dataclass
class Case:
    model: str
    nodes: int
    batch: int
    microbatches: int
    tokens: int
    mode: str
    dp: int
    pp: int
    tp: int
    comment: str = ""

    @staticmethod
    def parse(text: str) -> "Case":
        f = shlex.split(text, comments=True)
        if len(f) < 9:
            raise ValueError(f"a case needs 9 fields (model nodes batch microbatches tokens mode dp pp tp [comment]): {text!r}")
        c = Case(f[0], int(f[1]), int(f[2]), int(f[3]), int(f[4]), f[5], int(f[6]), int(f[7]), int(f[8]), " ".join(f[9:]))
        if c.mode not in MODES:
            raise ValueError(f"mode {c.mode!r} not in {MODES}")
        if min(c.nodes, c.batch, c.microbatches, c.tokens, c.dp, c.pp, c.tp) < 1:
            raise ValueError(f"non-positive field in {text!r}")
        return c

    @property
    def world(self) -> int:
        return self.dp * self.pp * self.tp

    def name(self, dist: str, ratio: float) -> str:
        tag = f"{self.model}.n{self.nodes}.b{self.batch}.mb{self.microbatches}.t{self.tokens}.{self.mode}" \
              f".dp{self.dp}pp{self.pp}tp{self.tp}.{dist}{ratio:g}"
        return tag.replace("/", "_")


def script_args(c: Case, dist: str, ratio: float, out_dir: str, steps: int, gpus_per_node: int,
                extra: list[str]) -> list[str]:
    """Arguments of ``pretrain_llama.py`` for one case (the reference's ELONGATE_FACTOR rule included:
    documents of the sampled data sets are stretched by ``tokens / 65536``, run4d.sh:118-121)."""
    if c.world != c.nodes * gpus_per_node:
        raise ValueError(f"{c}: dp*pp*tp = {c.world} but nodes*gpus = {c.nodes * gpus_per_node}")
    if c.mode in ("baseline", "perseq", "wlbllm") and c.pp > 1:
        raise ValueError(f"{c}: the per-document CP baseline runs without pipeline stages (use dp x tp)")
    a = [os.path.join(ROOT, "pretrain_llama.py"), "--model", c.model, "--num-nodes", str(c.nodes),
         "--num-gpus-per-node", str(gpus_per_node), "--tp-size", str(c.tp), "--pp-size", str(c.pp),
         "--dp-size", str(c.dp), "--num-tokens", str(c.tokens), "--num-batches", str(c.batch),
         "--num-microbatch", str(c.microbatches), "--sample-name", dist, "--change-long-doc-ratio", str(ratio),
         "--elongate-factor", str(max(1, c.tokens // 65536)), "--max-sample-id", str(steps), "--output-dir", out_dir]
    if c.mode == "distca":
        a.append("--cad")
    elif c.mode == "local":
        a.append("--no-cad")
    elif c.mode == "perseq":
        a += ["--baseline-mode", "perseq"]
    elif c.mode == "wlbllm":
        a += ["--baseline-mode", "percp", "--packing", "wlb"]
    else:
        a += ["--baseline-mode", "percp"]
    return a + list(extra)


def read_result(out_dir: str) -> dict:
    p = os.path.join(out_dir, "benchmark.json")
    if not os.path.exists(p):
        return {}
    with open(p) as f:
        return json.load(f)


def format_table(rows: list[dict]) -> str:
    cols = ["case", "mode", "layout", "dist", "rc", "tokens/s", "step ms", "exposed ms", "imbalance", "loss"]
    table = [cols]
    for r in rows:
        res = r.get("result", {})

        def num(k, fmt):
            return format(res[k], fmt) if res.get(k) is not None else "-"
        table.append([r["comment"] or r["name"], r["mode"], f"dp{r['dp']}pp{r['pp']}tp{r['tp']}",
                      f"{r['dist']} {r['ratio']:g}", str(r["rc"]), num("mean_tokens_per_s", ".0f"),
                      num("mean_step_ms", ".1f"), num("mean_exposed_dispatch_ms", ".1f"),
                      num("mean_attn_imbalance", ".3f"), num("last_loss", ".4f")])
    width = [max(len(row[i]) for row in table) for i in range(len(cols))]
    return "\n".join("  ".join(cell.ljust(w) for cell, w in zip(row, width)).rstrip() for row in table)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--case", action="append", default=[], help="'model nodes batch microbatches tokens mode dp pp tp [comment]'")
    ap.add_argument("--cases-file", default=None)
    ap.add_argument("--dist", action="append", default=[], help="'sample_name change_long_doc_ratio' (default: 'mixture 0.0')")
    ap.add_argument("--steps", type=int, default=int(os.environ.get("MAX_SAMPLE_ID", 5)))
    ap.add_argument("--nodes", default="localhost")
    ap.add_argument("--gpus-per-node", type=int, default=8)
    ap.add_argument("--port", type=int, default=29500)
    ap.add_argument("--output-dir", default=os.environ.get("OUTPUT_DIR_PREFIX", "runs/sweep"))
    ap.add_argument("--max-cases", type=int, default=100)
    ap.add_argument("--dry-run", action="store_true", default=os.environ.get("DRY_RUN", "0") == "1")
    ap.add_argument("--nsys", action="store_true", default=os.environ.get("ENABLE_NSYS", "0") == "1",
                    help="wrap every run in nsys (one report per node in the run's directory)")
    ap.add_argument("extra", nargs=argparse.REMAINDER, help="-- further pretrain_llama.py arguments for every case")
    a = ap.parse_args(argv)
    texts = list(a.case)
    if a.cases_file:
        with open(a.cases_file) as f:
            texts += [ln for ln in (x.strip() for x in f) if ln and not ln.startswith("#")]
    if not texts:
        ap.error("no cases (--case / --cases-file)")
    cases = [Case.parse(t) for t in texts]
    dists = []
    for d in a.dist or ["mixture 0.0"]:
        f = d.split()
        dists.append((f[0], float(f[1]) if len(f) > 1 else 0.0))
    extra = a.extra[1:] if a.extra and a.extra[0] == "--" else a.extra
    all_nodes = [n for n in a.nodes.split(",") if n]
    rows, done = [], 0
    print(f"{len(cases) * len(dists)} runs ({len(cases)} cases x {len(dists)} distributions)", flush=True)
    for dist, ratio in dists:
        for c in cases:
            if done >= a.max_cases:
                break
            done += 1
            name = c.name(dist, ratio)
            out_dir = os.path.join(a.output_dir, name)
            row = {**asdict(c), "name": name, "dist": dist, "ratio": ratio, "dir": out_dir, "rc": None, "result": {}}
            try:
                args = script_args(c, dist, ratio, out_dir, a.steps, a.gpus_per_node, extra)
                nodes = all_nodes[:c.nodes]
                if len(nodes) < c.nodes:
                    raise ValueError(f"{c}: needs {c.nodes} nodes, --nodes lists {len(all_nodes)}")
            except ValueError as e:
                row.update(rc=-1, error=str(e))
                print(f"[skip] {e}", flush=True)
                rows.append(row)
                continue
            largv = ["--nodes", ",".join(nodes), "--gpus-per-node", str(a.gpus_per_node), "--port", str(a.port + done % 50),
                     "--workdir", ROOT, "--output-dir", out_dir, "--no-duplicate-log"]
            if a.nsys:
                largv += ["--nsys", os.path.join(out_dir, "nsys")]
            if a.dry_run:
                largv.append("--dry-run")
            print(f"[run {done}] {name}  ({c.comment})" if c.comment else f"[run {done}] {name}", flush=True)
            t0 = time.time()
            row["rc"] = launch.main(largv + ["--", *args])
            row["wall_s"] = round(time.time() - t0, 1)
            if not a.dry_run:
                row["result"] = read_result(out_dir)
                os.makedirs(a.output_dir, exist_ok=True)
                with open(os.path.join(a.output_dir, "sweep.jsonl"), "a") as f:
                    f.write(json.dumps(row) + "\n")
            rows.append(row)
    if not a.dry_run:
        print(format_table(rows), flush=True)
    return 0 if all(r["rc"] == 0 for r in rows) else 1


if __name__ == "__main__":
    sys.exit(main())
