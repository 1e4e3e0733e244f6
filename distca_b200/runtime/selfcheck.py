"""Multi-rank self-checks, run under torchrun:

    torchrun --nproc-per-node 2 -m distca_b200.runtime.selfcheck cad --model small-128 --tokens 8192
    torchrun --nproc-per-node 4 -m distca_b200.runtime.selfcheck cad --tp 2 --pp 2 --microbatches 2

``cad``: training steps with core-attention disaggregation against the same steps with local
attention (same seed, same batches): the losses and every rank's local gradients must agree to
bf16 accuracy. With ``--pp`` > 1 the pipeline trainer is used and idle pipeline slots serve
attention. ``dp`` / ``tp``: the peer-memory transports against NCCL. ``percp``: the per-document CP baseline
against CAD. ``span``: documents spanning ranks against the per-document CP baseline. This is the multi-GPU analogue of the reference's layer / end-to-end tests that compare
the plain path with the CAD path (tests/test_megatron_layer.py:149-252,
tests/test_megatron_e2e_pipeline.py:389-414).
Exit code 0 on success; rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
import torch.distributed as dist

from ..models.config import ParallelConfig, TrainConfig, get_model_config
from .trainer import BatchSource, Trainer, init_distributed


def _DEV() -> torch.device:
    """Where the ranks' tensors live: the current GPU, or the CPU (gloo ranks: ``cad``, ``percp`` and ``span`` run
    there too, on the CPU restatements of the kernels; ``dp`` and ``tp`` compare GPU transports)."""
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def _free() -> None:
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


LOSS_RTOL = 2e-3        # relative difference of a step's loss between the two paths
TENSOR_RTOL = 2e-2      # largest element-wise difference of a named gradient, relative to that tensor's largest entry


def check_cad(a) -> int:
    rank, world, _ = init_distributed()
    cfg = get_model_config(a.model, a.layers)
    par = ParallelConfig(tp=a.tp, pp=a.pp, dp=world // (a.tp * a.pp))
    results, grads = {}, {}
    for mode in ("local", "cad"):
        tc = TrainConfig(cad=(mode == "cad"), recompute=a.recompute if mode == "cad" else "full",
                         grad_dtype="fp32" if a.pp > 1 else "bf16")
        if mode == "cad":
            tc.extra["nano_batches"] = a.nano
            tc.extra["fuse_ticks"] = a.fuse_ticks
        if a.pp > 1:
            from ..parallel.pipeline import PipelineTrainer
            tr = PipelineTrainer(cfg, par, tc, num_microbatch=a.microbatches, seed=1)
            seqs = a.microbatches
        else:
            tr = Trainer(cfg, par, tc, seed=1)
            seqs = 1
        src = BatchSource(cfg, par, a.tokens, a.dist, seed=a.seed, seqs_per_rank=seqs)
        losses = []
        for _ in range(a.steps):
            losses.append(tr.train_step(src.next(tr.dp_rank)))
        tr.check_device_status()
        results[mode] = losses
        grads[mode] = tr.model.store.grad.float().clone()
        offsets = dict(tr.model.store.offsets)
        if mode == "cad":
            results["plan"] = {k: v for k, v in tr.cad.plan_stats.items() if k != "send_bytes"}
        tr.close()
        del tr
        _free()
    g0, g1 = grads["local"], grads["cad"]
    err = (g0 - g1).abs().max().item()
    scale = g0.abs().max().item() + 1e-12
    cos = torch.nn.functional.cosine_similarity(g0, g1, dim=0).item()
    # every named tensor on its own scale (the reference asserts rtol = atol = 1.1e-3 on one named gradient,
    # tests/test_megatron_e2e_pipeline.py:414; bf16 kernels with different summation orders need a little more)
    worst_name, worst_rel = None, 0.0
    for name, (o, n) in offsets.items():
        a0, a1 = g0[o:o + n], g1[o:o + n]
        rel = (a0 - a1).abs().max().item() / (a0.abs().max().item() + 1e-12)
        if rel > worst_rel:
            worst_name, worst_rel = name, rel
    ok = (all(abs(x - y) <= LOSS_RTOL * abs(x) for x, y in zip(results["local"], results["cad"]))
          and worst_rel <= TENSOR_RTOL and cos > 0.9995)
    flags = torch.tensor([1 if ok else 0], device=_DEV())
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"check": "cad", "ok": bool(flags.item()), "parallel": par.describe(),
                          "loss_local": results["local"], "loss_cad": results["cad"], "grad_max_err": err,
                          "grad_scale": scale, "grad_cosine": cos, "worst_tensor": worst_name,
                          "worst_tensor_rel_err": worst_rel, "plan": results.get("plan")}))
    dist.barrier()
    return 0 if flags.item() else 1


def check_dp(a) -> int:
    """Peer-memory reduce-scatter + Adam-with-all-gather against NCCL reduce-scatter / all-gather:
    after the same steps the parameters must agree to bf16 accuracy and the losses must match."""
    rank, world, _ = init_distributed()
    cfg = get_model_config(a.model, a.layers)
    par = ParallelConfig(tp=1, pp=1, dp=world)
    out = {}
    for transport in ("nccl", "p2p"):
        tc = TrainConfig(cad=False, recompute="full", lr=1e-3)
        tc.extra["dp_transport"] = transport
        tr = Trainer(cfg, par, tc, seed=1)
        src = BatchSource(cfg, par, a.tokens, a.dist, seed=a.seed)
        losses = [tr.train_step(src.next(tr.dp_rank)) for _ in range(a.steps)]
        tr.check_device_status()
        out[transport] = (losses, tr.model.store.flat.float().clone(), float(tr.opt.last_grad_norm))
        tr.close()
        del tr
        _free()
    p0, p1 = out["nccl"][1], out["p2p"][1]
    err = (p0 - p1).abs().max().item()
    ok = err <= TENSOR_RTOL * p0.abs().max().item() and all(abs(x - y) <= LOSS_RTOL * abs(x) for x, y in zip(out["nccl"][0], out["p2p"][0]))
    flags = torch.tensor([1 if ok else 0], device=_DEV())
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"check": "dp", "ok": bool(flags.item()), "loss_nccl": out["nccl"][0], "loss_p2p": out["p2p"][0],
                          "param_max_diff": err, "grad_norm": [out["nccl"][2], out["p2p"][2]]}))
    dist.barrier()
    return 0 if flags.item() else 1


def check_percp(a) -> int:
    """The per-document context-parallel baseline (all-gather K/V, NCCL) against core-attention
    disaggregation on the same global batches: different token layouts, same model, so the losses of a few
    optimizer steps and the weights they produce must agree to bf16 accuracy."""
    rank, world, _ = init_distributed()
    cfg = get_model_config(a.model, a.layers)
    par = ParallelConfig(tp=1, pp=1, dp=world)
    out = {}
    for mode in ("cad", "percp"):
        tc = TrainConfig(cad=(mode == "cad"), recompute=a.recompute, lr=1e-3)
        tc.extra["baseline_mode"] = a.baseline if mode == "percp" else "none"
        tc.extra["cp_seq_len"] = a.tokens
        tr = Trainer(cfg, par, tc, seed=1)
        src = BatchSource(cfg, par, a.tokens, a.dist, seed=a.seed)
        losses = []
        for _ in range(a.steps):
            losses.append(tr.train_step(src.next_global() if mode == "percp" else src.next(tr.dp_rank)))
        tr.check_device_status()
        out[mode] = (losses, tr.model.store.flat.float().clone())
        tr.close()
        del tr
        _free()
    p0, p1 = out["cad"][1], out["percp"][1]
    err = (p0 - p1).abs().max().item()
    ok = (err <= TENSOR_RTOL * p0.abs().max().item()
          and all(abs(x - y) <= LOSS_RTOL * abs(x) for x, y in zip(out["cad"][0], out["percp"][0])))
    flags = torch.tensor([1 if ok else 0], device=_DEV())
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"check": "percp", "ok": bool(flags.item()), "loss_cad": out["cad"][0],
                          "loss_percp": out["percp"][0], "param_max_diff": err}))
    dist.barrier()
    return 0 if flags.item() else 1


def check_tp(a) -> int:
    """All-gather -> GEMM and GEMM -> reduce-scatter fused into the tcgen05 GEMM over peer memory against
    the NCCL collectives + plain GEMM: same losses and gradients to bf16 accuracy."""
    rank, world, _ = init_distributed()
    cfg = get_model_config(a.model, a.layers)
    par = ParallelConfig(tp=world, pp=1, dp=1)
    out = {}
    for transport in ("nccl", "p2p", "p2p-tile"):
        tc = TrainConfig(cad=False, recompute="full")
        tc.extra["tp_transport"] = transport
        tc.extra["tp_max_rows_local"] = a.tokens // world
        tr = Trainer(cfg, par, tc, seed=1)
        src = BatchSource(cfg, par, a.tokens, a.dist, seed=a.seed)
        losses = [tr.train_step(src.next(tr.dp_rank)) for _ in range(a.steps)]
        tr.check_device_status()
        out[transport] = (losses, tr.model.store.grad.float().clone(), tr.model.tp.fused is not None,
                          tr.model.tp.nccl_row_collectives // a.steps)
        if tr.model.tp.fused is not None:
            tr.model.tp.fused.close()
        tr.close()
        del tr
        _free()
    g0 = out["nccl"][1]
    cos = {t: torch.nn.functional.cosine_similarity(g0, out[t][1], dim=0).item() for t in ("p2p", "p2p-tile")}
    ok = all(c > 0.9995 for c in cos.values()) and all(
        abs(x - y) <= LOSS_RTOL * abs(x) for t in ("p2p", "p2p-tile") for x, y in zip(out["nccl"][0], out[t][0]))
    flags = torch.tensor([1 if ok else 0], device=_DEV())
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"check": "tp", "ok": bool(flags.item()), "loss_nccl": out["nccl"][0], "loss_p2p": out["p2p"][0],
                          "loss_p2p_tile": out["p2p-tile"][0],
                          "fused": out["p2p"][2] and out["p2p-tile"][2] and not out["nccl"][2],
                          "nccl_row_collectives_per_step": {t: out[t][3] for t in out},
                          "grad_cosine": cos["p2p"], "grad_cosine_p2p_tile": cos["p2p-tile"],
                          "grad_max_err": (g0 - out["p2p"][1]).abs().max().item()}))
    dist.barrier()
    return 0 if flags.item() else 1


def check_span(a) -> int:
    """Documents that span ranks (the planner lays one global batch out over the ranks by sequential fill, a
    long document is held as head / tail pieces by several ranks and its attention is disaggregated) against
    the per-document context-parallel baseline on the same global batches: two different token layouts and two
    different attention schemes of the same model, so the losses of a few optimizer steps and the weights they
    produce must agree to bf16 accuracy."""
    import numpy as np
    from .trainer import make_span_batch
    rank, world, _ = init_distributed()
    cfg = get_model_config(a.model, a.layers)
    par = ParallelConfig(tp=1, pp=1, dp=world)
    out = {}
    for mode in ("percp", "span"):
        tc = TrainConfig(cad=(mode == "span"), recompute=a.recompute, lr=1e-3)
        tc.extra["baseline_mode"] = "percp" if mode == "percp" else "none"
        tr = Trainer(cfg, par, tc, seed=1)
        losses, longest = [], 0
        for step in range(a.steps):
            hb = make_span_batch(np.random.default_rng(a.seed * 1009 + step), world, a.tokens, cfg.vocab,
                                 max_doc_len=world * a.tokens, min_doc_len=a.tokens // 2)
            longest = max(longest, max(hb.doc_lens))
            losses.append(tr.train_step(hb))
        tr.check_device_status()
        out[mode] = (losses, tr.model.store.flat.float().clone())
        tr.close()
        del tr
        _free()
    p0, p1 = out["percp"][1], out["span"][1]
    err = (p0 - p1).abs().max().item()
    ok = (err <= TENSOR_RTOL * p0.abs().max().item()
          and all(abs(x - y) <= LOSS_RTOL * abs(x) for x, y in zip(out["percp"][0], out["span"][0])))
    flags = torch.tensor([1 if ok else 0], device=_DEV())
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"check": "span", "ok": bool(flags.item()), "loss_percp": out["percp"][0],
                          "loss_span": out["span"][0], "param_max_diff": err, "longest_document": longest,
                          "tokens_per_rank": a.tokens}))
    dist.barrier()
    return 0 if flags.item() else 1


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("check", choices=["cad", "dp", "tp", "percp", "span"])
    ap.add_argument("--model", default="small-128")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--dist", default="mixture")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--microbatches", type=int, default=2)
    ap.add_argument("--nano", type=int, default=1, choices=[1, 2], help="ping-pong nano-batches in the CAD run")
    ap.add_argument("--baseline", default="percp", choices=["percp", "perseq"],
                    help="percp check: per-document or per-sequence context parallelism as the baseline arm")
    ap.add_argument("--fuse-ticks", action="store_true", help="with --nano 2: the next layer's pre-attention half per nano-batch right after this layer's post-attention half")
    ap.add_argument("--recompute", default="full", choices=["full", "keep_attn"],
                    help="activation policy of the CAD run (the local run always recomputes fully)")
    a = ap.parse_args()
    rc = {"cad": check_cad, "dp": check_dp, "tp": check_tp, "percp": check_percp, "span": check_span}[a.check](a)
    if dist.is_initialized():
        dist.destroy_process_group()
    sys.exit(rc)


if __name__ == "__main__":
    main()
