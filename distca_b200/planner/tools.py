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
from . import Planner, PlannerConfig, chunk_flops, default_network_model, default_time_model


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
    out = {"cad": [], "per_document_cp": [], "per_sequence_cp": [], "local": [], "wlb_packing": []}
    traffic = {"cad": [], "per_document_cp": []}
    for _ in range(iterations):
        docs = src.next_doc_lens()
        for name, plan in (("cad", p.plan_fixed(docs)), ("per_document_cp", p.plan_fixed_cp(docs))):
            sim = p.simulate(plan, tm)
            out[name].append(max(sim.attn_ms))
            traffic[name].append(sum(float(np.asarray(plan.rank(r).send_bytes).sum() - plan.rank(r).send_bytes[r])
                                     for r in range(world)) / world / 1e6)
        whole = lambda L: tm.attn_ms_for(L, L)
        from ..parallel.percp import perseq_layout
        flat = [L for d in docs for L in d]
        out["per_sequence_cp"].append(max(sum(tm.attn_ms_for(b - a, b) for _, a, b, _ in perseq_layout(flat, world, r, tokens))
                                          for r in range(world)))
        out["local"].append(max(sum(whole(L) for L in d) for d in docs))
        bins = balance_documents([L for d in docs for L in d], world, 2 * tokens)
        out["wlb_packing"].append(max(sum(whole(L) for L in b) for b in bins))
    return {"world": world, "tokens_per_rank": tokens, "dist": dist,
            "attention_ms_per_layer_forward_max_over_ranks": {k: float(np.mean(v)) for k, v in out.items()},
            "remote_mb_per_rank_per_layer": {k: float(np.mean(v)) for k, v in traffic.items()},
            "note": "wlb_packing leaves ranks with unequal token counts (linear layers unbalanced); not modelled here"}


# Calibration of the step model against one measured Llama-3-8B step on one B200 (131072 tokens, long/short
# mixture, keep_attn: CUDA-event phase timers, ms per step): GEMMs forward + recompute 2853, GEMMs backward 2784,
# norms 63 + 59, SwiGLU backward 109, RoPE backward 21, LM head 422, attention forward 2848 / backward 8437,
# optimizer and host 240.
BWD_OVER_FWD_LINEAR = 2.0        # (2784 + 59 + 109 + 21) / forward linear time
RECOMPUTE_OVER_FWD_LINEAR = 0.95  # the recompute pass skips the FC2 GEMM
BWD_OVER_FWD_ATTENTION = 2.96    # 8437 / 2848: the backward kernels run at a lower fraction of peak
ATTENTION_IN_STEP = 1.26         # the attention table was timed in isolation (burst clocks, 1.20 PFLOP/s at these lengths);
                                 # inside a power-capped step the same kernel ran at 0.95 PFLOP/s
LM_HEAD_MS_PER_TOKEN = 422.0 / 131072       # forward + backward, vocabulary 128256 x hidden 4096
OPTIMIZER_MS_8B = 240.0          # sharded AdamW over 8.03e9 parameters on one GPU
STORE_LINK_EFFICIENCY = 0.70     # peer stores from many CTAs against the measured peer copy (536 of 770 GB/s)
TILE_LOAD_GBS = 300.0            # per-tile remote TMA loads (p2p-tile): coarse; the measured TP > 1 steps imply 135-570 GB/s


def _tp_comm_ms(cfg, tok: int, tp: int, layers: float, link_bytes_per_ms: float, recompute: str, transport: str,
                network=None) -> float:
    """Time of a tensor-parallel rank's all-gathers that is NOT hidden behind GEMMs, per step. ``gather``: every
    shard pushed once, then a local GEMM (serial); ``tile``: the GEMM loads remote tiles itself and re-fetches a
    tile once per N tile that uses it; ``nccl``: library collectives, all-gathers and reduce-scatters serial. The
    reduce-scatters of the peer transports ride in GEMM epilogues."""
    if tp == 1:
        return 0.0
    shard = tok * cfg.hidden * 2 * (tp - 1) / tp               # bytes one all-gather / reduce-scatter moves per rank
    passes_ag = 2 + (2 if recompute != "none" else 0) + 4      # forward n1, n2; recompute n1, n2; backward dy, n2, dh, n1
    passes_rs = 2 + (1 if recompute != "none" else 0) + 2
    if transport == "nccl":
        return (passes_ag + passes_rs) * shard / link_bytes_per_ms * layers
    # one peer-store all-gather: measured (`net_bench`'s push_all_gather table, bytes = one rank's own shard) when the
    # network model has it, else the link at the efficiency the dispatch kernel's stores reach
    if network is not None and "push_all_gather" in network.ops():
        push = lambda b: network.ms("push_all_gather", tp, b / (tp - 1))
    else:
        push = lambda b: b / (link_bytes_per_ms * STORE_LINK_EFFICIENCY)
    if transport == "gather":
        return passes_ag * push(shard) * layers
    # per-tile loads: operand bytes x N tiles of the consuming GEMM (QKV, FC1 forward and recompute; dact, dattn backward)
    nt = lambda n: max(1.0, n / tp / 256.0)
    fwd = nt(cfg.qkv_dim) + nt(2 * cfg.ffn)
    bwd = nt(cfg.ffn) + nt(cfg.q_dim)
    tiles = fwd * (2 if recompute != "none" else 1) + bwd
    gathers = 2                                                # n2, n1 for the weight gradients (pushed once)
    return (tiles * shard / (TILE_LOAD_GBS * 1e6) + gathers * push(shard)) * layers


def predict_step_ms(cfg, tm, packs: list[list[int]], tokens: int, tp: int, pp: int, dp: int, microbatches: int,
                    mode: str, recompute: str = "keep_attn", tp_transport: str = "gather",
                    tolerance: float = 0.02, network=None) -> dict:
    """Predicted milliseconds of one training step (forward, recompute, backward, optimizer) of the global batch
    ``packs`` (document lengths per packed sequence, ``len(packs)`` a multiple of ``dp``) under one layout.
    ``mode``: ``cad`` (core attention spread over the dp x pp servers by the planner), ``local`` (every rank attends
    to its own documents) or ``percp`` / ``perseq`` (per-document / per-sequence context parallelism over the dp ranks,
    all-gathered K/V; no pipeline stages). ``network``: a :class:`~distca_b200.planner.NetworkModel` (default: the measured B200 tables)
    for the peer-store all-gathers and, where it has a table, the NCCL all-gather of the baseline. Returns the
    parts as well."""
    if network is None:
        network = default_network_model("b200")
    L = cfg.num_layers
    ref = get_model_config("llama3-8b")
    per_rank_seqs = len(packs) // dp
    per_rank = [sum(packs[r * per_rank_seqs:(r + 1) * per_rank_seqs], []) for r in range(dp)]
    tok_rank = per_rank_seqs * tokens
    link = tm.link_gbytes_per_s * 1e6                                  # bytes per ms
    passes_lin = 1.0 + BWD_OVER_FWD_LINEAR + (RECOMPUTE_OVER_FWD_LINEAR if recompute != "none" else 0.0)
    passes_attn = 1.0 + BWD_OVER_FWD_ATTENTION + (1.0 if recompute == "full" else 0.0)
    scale_lin = cfg.flops_per_token_linear() / ref.flops_per_token_linear() * ref.num_layers / L   # per layer
    lin = passes_lin * tm.linear_ms_per_token * scale_lin * tok_rank / tp * (L / pp)
    lm = LM_HEAD_MS_PER_TOKEN * tok_rank / tp * (cfg.vocab * cfg.hidden) / (ref.vocab * ref.hidden)
    opt = OPTIMIZER_MS_8B * (cfg.flops_per_token_linear() / ref.flops_per_token_linear()) / (tp * pp * dp)
    tp_comm = _tp_comm_ms(cfg, tok_rank, tp, L / pp, link, recompute, tp_transport, network)
    heads = ATTENTION_IN_STEP * cfg.heads_q / 32.0 / tp
    whole = lambda n: tm.attn_ms_for(n, n)
    disp = 0.0
    if mode == "perseq":
        assert pp == 1, "the per-sequence CP baseline has no pipeline stages"
        # every packed sequence cut into 2 x dp chunks wherever its documents end: tokens are balanced, causal work
        # is not; the step waits for the rank whose chunks hold the ends of the long documents
        from ..parallel.percp import perseq_layout
        docs = [x for p_ in packs for x in p_]
        per = [sum(tm.attn_ms_for(b - a, b) for _, a, b, _ in perseq_layout(docs, dp, r, tokens)) for r in range(dp)]
        kv_bytes = sum(docs) * 2 * cfg.kv_dim / tp * 2 * (dp - 1) / dp
        passes_kv = 1 + (1 if recompute != "none" else 0) + 1 + 1
        one = network.ms("all_gather", dp, kv_bytes / max(dp - 1, 1)) if "all_gather" in network.ops() else kv_bytes / link
        disp = passes_kv * one * L
        attn = passes_attn * max(per) * heads * L
    elif mode == "percp":
        assert pp == 1, "the per-document CP baseline has no pipeline stages"
        # every document cut into 2 x dp chunks, every rank holds a head and a tail chunk: 1 / dp of each document's
        # pairs, but 2 query chunks per document and rank (short documents pay the per-tile cost dp times over)
        docs = [x for d in per_rank for x in d]
        attn_fwd = 0.0
        for x in docs:
            c = max(1, x // (2 * dp))
            attn_fwd += max(whole(x) / dp, 2.0 * whole(min(c, 128)))   # at least two (partial) tiles of work per document
        kv_bytes = sum(docs) * 2 * cfg.kv_dim / tp * 2 * (dp - 1) / dp  # K and V of every other rank, bf16
        passes_kv = 1 + (1 if recompute != "none" else 0) + 1 + 1       # all-gather fwd, recompute, bwd; reduce-scatter dK/dV
        one = network.ms("all_gather", dp, kv_bytes / max(dp - 1, 1)) if "all_gather" in network.ops() else kv_bytes / link
        disp = passes_kv * one * L
        attn = passes_attn * attn_fwd * heads * L
        servers = dp
    elif mode == "cad" and dp * pp > 1:
        servers = dp * pp
        p = Planner(PlannerConfig.for_model(cfg, servers, max(sum(d) for d in per_rank) or tokens, tp=tp, tolerance=tolerance))
        # every pipeline stage serves: the data-parallel ranks' documents are spread over dp x pp servers
        plan = p.plan_fixed([per_rank[r % dp] if r < dp else [] for r in range(servers)])
        sim = p.simulate(plan, tm)
        # the plan spreads ONE layer's attention of all sequences in flight over dp x pp servers; every server
        # serves all L layers (its own stage's layers for pp different micro-batches)
        attn = passes_attn * max(sim.attn_ms) * heads * L
        disp = (4 if recompute != "none" else 3) * max(sim.comm_ms) / tp * L
    else:
        attn = passes_attn * max(sum(whole(x) for x in d) for d in per_rank) * heads * (L / pp)
    bubble = (pp - 1) / (microbatches + pp - 1) if pp > 1 else 0.0
    busy = lin + tp_comm + lm
    if mode == "cad" and dp * pp > 1 and pp > 1:
        # idle pipeline slots serve attention: the servers' attention work fills the bubble first
        step = busy + max(busy * bubble / (1.0 - bubble), attn + disp)
    else:
        stage = busy + attn + disp
        step = stage / (1.0 - bubble) if pp > 1 else stage
    return {"step_ms": step + opt, "linear_ms": lin, "lm_head_ms": lm, "tp_comm_ms": tp_comm, "attention_ms": attn,
            "dispatch_ms": disp, "optimizer_ms": opt, "bubble_fraction": bubble}


def search_layouts(model: str, gpus: int, tokens: int, dist: str, iterations: int = 10, tolerance: float = 0.02,
                   seed: int = 0, microbatches: int | None = None, seqs_per_step: int | None = None,
                   recompute: str = "keep_attn", tp_transport: str = "gather", comm_buffer_gb: float = 4.0,
                   capacity_gb: float = 180.0, time_model=None, network=None) -> dict:
    """Predicted milliseconds per training step of a fixed global batch of ``seqs_per_step`` packed sequences
    (default: one per GPU) under every (tp, pp, dp) layout of ``gpus`` GPUs, with local attention, with core-attention
    disaggregation and (layouts without pipeline stages) with the per-document CP baseline."""
    cfg = get_model_config(model)
    tm = time_model if time_model is not None else default_time_model("b200")
    seqs = seqs_per_step or gpus
    src = SyntheticBatches(tokens, seqs, dist, seed)
    batches = [src.next_doc_lens() for _ in range(iterations)]
    L = cfg.num_layers
    rows = []
    for tp in (t for t in (1, 2, 4, 8) if gpus % t == 0 and cfg.heads_kv % t == 0):
        for pp in (p for p in (1, 2, 4) if (gpus // tp) % p == 0 and L % p == 0):
            dp = gpus // (tp * pp)
            if seqs % dp:
                continue
            M = microbatches or max(pp, seqs // dp)
            if (seqs // dp) % M and pp > 1:
                continue
            res = {}
            for mode in ("local", "cad") + (("percp", "perseq") if pp == 1 and dp > 1 else ()):
                res[mode] = float(np.mean([predict_step_ms(cfg, tm, packs, tokens, tp, pp, dp, M, mode, recompute,
                                                           tp_transport, tolerance, network)["step_ms"] for packs in batches]))
            row = {"tp": tp, "pp": pp, "dp": dp, "microbatches": M if pp > 1 else 1,
                   "step_ms_local_attention": round(res["local"], 1), "step_ms_cad": round(res["cad"], 1)}
            if "percp" in res:
                row["step_ms_percp"] = round(res["percp"], 1)
                row["step_ms_perseq"] = round(res["perseq"], 1)
            # per-GPU memory of the layout with disaggregation (tokens of one micro-batch per data-parallel rank)
            from ..models.config import ParallelConfig
            from ..utils.guards import estimate_memory_gb
            tok_mb = (seqs // dp) * tokens // (M if pp > 1 else 1)
            est = estimate_memory_gb(cfg, ParallelConfig(tp=tp, pp=pp, dp=dp), tok_mb, recompute=recompute,
                                     cad=dp * pp > 1, comm_buffer_gb=comm_buffer_gb,
                                     microbatches_in_flight=min(M, pp) if pp > 1 else 1)
            row["memory_gb"] = round(est["total"], 1)
            row["fits"] = bool(est["total"] <= capacity_gb * 0.97)
            rows.append(row)
    # layouts that fit first, fastest first
    rows.sort(key=lambda r: (not r["fits"], min(r["step_ms_local_attention"], r["step_ms_cad"])))
    return {"model": cfg.name, "gpus": gpus, "tokens_per_sequence": tokens, "sequences_per_step": seqs, "dist": dist,
            "recompute": recompute, "tp_transport": tp_transport, "capacity_gb": capacity_gb, "layouts": rows,
            "note": "time: predicted from the attention table, the per-token linear time and the link bandwidth of the "
                    "B200 time model, calibrated on one measured step; memory: the pre-flight estimate of "
                    "utils/guards.py (keep_attn is counted like full recompute: kept attention outputs go to "
                    "whatever HBM is left, then to host memory)"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("tool", choices=["buffer", "compare", "layouts"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=131072)
    ap.add_argument("--dist", default="mixture")
    ap.add_argument("--iterations", type=int, default=20)
    ap.add_argument("--tolerance", type=float, default=0.02)
    ap.add_argument("--seqs-per-step", type=int, default=None, help="layouts: packed sequences per step (default: one per GPU)")
    ap.add_argument("--microbatches", type=int, default=None, help="layouts: micro-batches per step of the pipelined layouts")
    ap.add_argument("--recompute", default="keep_attn", choices=["none", "full", "keep_attn"])
    ap.add_argument("--comm-buffer-gb", type=float, default=4.0)
    ap.add_argument("--capacity-gb", type=float, default=180.0, help="layouts: HBM per GPU")
    ap.add_argument("--tp-transport", default="gather", choices=["gather", "tile", "nccl"],
                    help="layouts: how a tensor-parallel all-gather reaches its GEMM (gather = --tp-transport p2p)")
    ap.add_argument("--sweep-file", default=None,
                    help="layouts: `kernel_bench --kernel attn_sweep` output of the target machine for the attention table")
    ap.add_argument("--net-file", default=None,
                    help="layouts: `python -m distca_b200.utils.net_bench` output of the target machine for the collectives")
    a = ap.parse_args()
    if a.tool == "layouts":
        tm = net = None
        if a.sweep_file:
            from . import time_model_from_sweep
            tm = time_model_from_sweep(a.sweep_file)
        if a.net_file:
            from . import NetworkModel
            net = NetworkModel.from_sweep(a.net_file)
        print(json.dumps(search_layouts(a.model, a.world, a.tokens, a.dist, a.iterations, a.tolerance,
                                        microbatches=a.microbatches, seqs_per_step=a.seqs_per_step,
                                        recompute=a.recompute, tp_transport=a.tp_transport,
                                        comm_buffer_gb=a.comm_buffer_gb, capacity_gb=a.capacity_gb, time_model=tm,
                                        network=net)))
        return
    f = {"buffer": recommend_buffer_gb, "compare": compare_policies}[a.tool]
    print(json.dumps(f(a.model, a.world, a.tokens, a.dist, a.iterations, a.tolerance)))


if __name__ == "__main__":
    main()
