"""Planner-side tools that need no GPU:

* ``recommend_buffer_gb``: run the planner over sampled batches and report the largest receive
  arena any server needed, i.e. the smallest ``--comm-buffer-gb`` that never forces the tolerance
  ladder to back off (reference: distca/planner/buffer_size_adjust.py:37-119).
* ``compare_policies``: simulated step time of core-attention disaggregation, per-document context
  parallelism and workload-balanced packing on the same sampled batches (reference:
  distca/simulator/compare.py:21-78, there with CP-SAT models; here with the planner itself and the
  measured time model).

* ``search_layouts``: what-if over the parallel layouts of a GPU count: for every (tp, pp, dp) with
  ``tp * pp * dp = gpus`` the simulated time of one step (linear layers from the per-token time model scaled by
  tp, core attention from the planner's balanced plan and the attention table, tensor-parallel collectives and
  core-attention dispatch over the link, the 1F1B bubble for ``pp > 1``), with and without disaggregation. The
  reference searches (tp, cp) per worker with a CP-SAT model (distca/simulator/optimizers/attnserver.py:147-310);
  the layouts of one box are few enough to enumerate.

    python -m distca_b200.planner.tools buffer --world 8 --tokens 131072 --dist mixture
    python -m distca_b200.planner.tools compare --world 8 --tokens 131072 --dist mixture
    python -m distca_b200.planner.tools layouts --world 8 --tokens 131072 --dist mixture
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from ..data.synthetic import SyntheticBatches
from ..data.wlb import balance_documents
from ..models.config import get_model_config
from . import Planner, PlannerConfig, chunk_flops, default_time_model


def _planner(model: str, world: int, tokens: int, tolerance: float, tp: int = 1) -> Planner:
    cfg = get_model_config(model)
    return Planner(PlannerConfig.for_model(cfg, world, tokens, tp=tp, tolerance=tolerance))


def recommend_buffer_gb(model: str, world: int, tokens: int, dist: str, iterations: int = 50,
                        tolerance: float = 0.02, tp: int = 1, seed: int = 0) -> dict:
    p = _planner(model, world, tokens, tolerance, tp)
    src = SyntheticBatches(tokens, world, dist, seed)
    q_b, kv_b = p.cfg.q_row_bytes, p.cfg.kv_row_bytes
    worst_q = worst_kv = worst_send = 0
    for _ in range(iterations):
        plan = p.plan_fixed(src.next_doc_lens())
        for r in range(world):
            rp = plan.rank(r)
            worst_q, worst_kv = max(worst_q, int(rp.q_rows)), max(worst_kv, int(rp.kv_rows))
            sb = np.asarray(rp.send_bytes)
            worst_send = max(worst_send, int(sb.sum() - sb[r]))
    recv = worst_q * q_b + 2 * worst_kv * kv_b
    return {"world": world, "tokens_per_rank": tokens, "iterations": iterations,
            "max_q_rows": worst_q, "max_kv_rows": worst_kv, "max_remote_send_mb": worst_send / 1e6,
            "receive_arena_gb": recv / 2**30, "recommended_comm_buffer_gb": float(np.ceil(recv / 2**30 * 1.1))}


def compare_policies(model: str, world: int, tokens: int, dist: str, iterations: int = 20,
                     tolerance: float = 0.02, seed: int = 0) -> dict:
    p = _planner(model, world, tokens, tolerance)
    tm = default_time_model("b200")
    src = SyntheticBatches(tokens, world, dist, seed)
    out = {"cad": [], "per_document_cp": [], "local": [], "wlb_packing": []}
    traffic = {"cad": [], "per_document_cp": []}
    for _ in range(iterations):
        docs = src.next_doc_lens()
        for name, plan in (("cad", p.plan_fixed(docs)), ("per_document_cp", p.plan_fixed_cp(docs))):
            sim = p.simulate(plan, tm)
            out[name].append(max(sim.attn_ms))
            traffic[name].append(sum(float(np.asarray(plan.rank(r).send_bytes).sum() - plan.rank(r).send_bytes[r])
                                     for r in range(world)) / world / 1e6)
        whole = lambda L: tm.attn_ms_for(L, L)
        out["local"].append(max(sum(whole(L) for L in d) for d in docs))
        bins = balance_documents([L for d in docs for L in d], world, 2 * tokens)
        out["wlb_packing"].append(max(sum(whole(L) for L in b) for b in bins))
    return {"world": world, "tokens_per_rank": tokens, "dist": dist,
            "attention_ms_per_layer_forward_max_over_ranks": {k: float(np.mean(v)) for k, v in out.items()},
            "remote_mb_per_rank_per_layer": {k: float(np.mean(v)) for k, v in traffic.items()},
            "note": "wlb_packing leaves ranks with unequal token counts (linear layers unbalanced); not modelled here"}


def search_layouts(model: str, gpus: int, tokens: int, dist: str, iterations: int = 10, tolerance: float = 0.02,
                   seed: int = 0, microbatches: int | None = None, seqs_per_step: int | None = None) -> dict:
    """Simulated milliseconds per step (forward + backward = 3 x forward linear, 3.3 x forward attention) of a
    fixed global batch of ``seqs_per_step`` packed sequences (default: one per GPU) under every layout."""
    cfg = get_model_config(model)
    tm = default_time_model("b200")
    seqs = seqs_per_step or gpus
    src = SyntheticBatches(tokens, seqs, dist, seed)
    batches = [src.next_doc_lens() for _ in range(iterations)]
    L = cfg.num_layers
    link = tm.link_gbytes_per_s * 1e6            # bytes per ms
    scale_lin = cfg.flops_per_token_linear() / get_model_config("llama3-8b").flops_per_token_linear() * 32 / L
    rows = []
    for tp in (t for t in (1, 2, 4, 8) if gpus % t == 0 and cfg.heads_kv % t == 0):
        for pp in (p for p in (1, 2, 4) if (gpus // tp) % p == 0 and L % p == 0):
            dp = gpus // (tp * pp)
            if seqs % dp:
                continue
            M = microbatches or max(pp, seqs // dp)
            if (seqs // dp) % M and pp > 1:
                continue
            per_rank_seqs = seqs // dp                       # sequences a data-parallel rank sees per step
            res = {}
            for cad in (False, True):
                tot = 0.0
                for packs in batches:
                    per_rank = [sum(packs[r * per_rank_seqs:(r + 1) * per_rank_seqs], []) for r in range(dp)]
                    tok_rank = per_rank_seqs * tokens
                    lin = 3.0 * tm.linear_ms_per_token * scale_lin * tok_rank / tp * (L / pp)
                    # tensor-parallel collectives: 4 all-gathers / reduce-scatters of [tokens, hidden] per layer pass, x3 passes
                    tp_comm = 0.0 if tp == 1 else 3 * 4 * (tok_rank * cfg.hidden * 2 * (tp - 1) / tp) / link * (L / pp)
                    servers = dp * pp
                    if cad and servers > 1:
                        p = Planner(PlannerConfig.for_model(cfg, servers, max(sum(d) for d in per_rank) or tokens, tp=tp,
                                                            tolerance=tolerance))
                        # every pipeline stage serves: spread the data-parallel ranks' documents over dp x pp servers
                        docs = [per_rank[r % dp] if r < dp else [] for r in range(servers)]
                        plan = p.plan_fixed(docs)
                        sim = p.simulate(plan, tm)
                        # the plan spreads ONE layer's attention of all sequences in flight over dp x pp servers; every
                        # server serves all L layers (its own stage's layers for pp different micro-batches)
                        attn = 3.3 * max(sim.attn_ms) * cfg.heads_q / 32 / tp * L
                        disp = 4 * max(sim.comm_ms) / tp * L
                    else:
                        whole = lambda n: tm.attn_ms_for(n, n)
                        attn = 3.3 * max(sum(whole(x) for x in d) for d in per_rank) * cfg.heads_q / 32 / tp * (L / pp)
                        disp = 0.0
                    bubble = (pp - 1) / (M + pp - 1) if pp > 1 else 0.0
                    if cad and servers > 1 and pp > 1:
                        # idle pipeline slots serve attention: the servers' attention work fills the bubble first
                        busy = lin + tp_comm
                        tot += busy + max(busy * bubble / (1.0 - bubble), attn + disp)
                    else:
                        stage = lin + tp_comm + attn + disp
                        tot += stage / (1.0 - bubble) if pp > 1 else stage
                res["cad" if cad else "local"] = tot / len(batches)
            rows.append({"tp": tp, "pp": pp, "dp": dp, "microbatches": M if pp > 1 else 1,
                         "step_ms_local_attention": round(res["local"], 1), "step_ms_cad": round(res["cad"], 1)})
    rows.sort(key=lambda r: min(r["step_ms_local_attention"], r["step_ms_cad"]))
    return {"model": cfg.name, "gpus": gpus, "tokens_per_sequence": tokens, "sequences_per_step": seqs, "dist": dist,
            "layouts": rows, "note": "simulated from the attention table, the per-token linear time and the link "
                                     "bandwidth of the B200 time model; memory limits are not checked here"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("tool", choices=["buffer", "compare", "layouts"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--dist", default="mixture")
    ap.add_argument("--iterations", type=int, default=20)
    ap.add_argument("--tolerance", type=float, default=0.02)
    a = ap.parse_args()
    f = {"buffer": recommend_buffer_gb, "compare": compare_policies, "layouts": search_layouts}[a.tool]
    print(json.dumps(f(a.model, a.world, a.tokens, a.dist, a.iterations, a.tolerance)))


if __name__ == "__main__":
    main()
