"""Headline benchmark: Llama-3-8B training at 128K tokens per sequence, whole-box tokens/s.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 3 --warmup 3

Every GPU holds one packed 128K-token sequence per step (weak scaling, data-parallel size = number
of GPUs); with more than one GPU core attention is disaggregated across all of them (CAD), the
gradients are reduce-scattered and AdamW runs on parameter shards. A step is forward + backward +
gradient reduction + optimizer update of the full 32-layer model. Activation policy: only each layer's
input and its core-attention output are kept (``--recompute keep_attn``: HBM or pinned host memory,
reported in ``config``); everything else of a layer is recomputed in backward (``--recompute full``
recomputes attention too).

Two timed regions after the warm-up, each of exactly ``--steps`` steps, bracketed by a barrier and
a device synchronise on both sides, maximum over ranks:
  * ``value``  – CUDA events; the batches are already on the device and the losses are read after
                 the region (device time of the training step itself);
  * ``e2e``    – wall clock through the public call ``Trainer.train_step(host_batch)``: every step
                 copies its inputs from pinned host memory and reads its loss back.
Documents are synthetic (80 % log-uniform [128, 8192], 20 % log-uniform [32768, 131072] tokens,
packed to 128K), weights random-init N(0, 0.02). Working sets are far larger than L2 (hundreds of
MB to GBs per kernel), so no explicit L2 flush is needed between steps.

``--impl reference`` reports why the reference's own training path cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


# The fixed layouts of the contract's other configurations (8 GPUs each).
NAMED_CONFIGS = {
    "tp8_64k": {"what": "Llama-3-8B, TP=8, 8 packed sequences of 64K tokens per step, documents log-uniform [128, 65536]",
                "model": "llama3-8b", "tp": 8, "pp": 1, "dp": 1, "seq_len": 65536, "seqs_per_rank": 8, "microbatches": 1,
                "dist": "loguniform", "recompute": "keep_attn"},
    "4d_128k": {"what": "Llama-3-8B, TP=2 x PP=2 x DP=2 with CAD, 128K-token sequences, long/short mixture",
                "model": "llama3-8b", "tp": 2, "pp": 2, "dp": 2, "seq_len": 131072, "seqs_per_rank": 1, "microbatches": 2,
                "dist": "mixture", "recompute": "keep_attn"},
    "34b_256k": {"what": "CodeLlama-34B shape, TP=4 x PP=2 with CAD, 256K-token sequences, full activation recompute",
                 "model": "codellama-34b", "tp": 4, "pp": 2, "dp": 1, "seq_len": 262144, "seqs_per_rank": 1, "microbatches": 2,
                 "dist": "mixture", "recompute": "full"},
}


def _args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq-len", type=int, default=None, help="tokens per packed sequence (headline: 131072; --config: its own)")
    ap.add_argument("--num-layers", type=int, default=None, help="debug only; the headline uses all layers")
    ap.add_argument("--dist", default="mixture")
    ap.add_argument("--no-cad", action="store_true")
    ap.add_argument("--comm-buffer-gb", type=float, default=6.0)
    ap.add_argument("--tolerance", type=float, default=0.02, help="CAD planner balance tolerance")
    ap.add_argument("--attention-policy", default="cad", choices=["cad", "cp", "water_fill"],
                    help="cp: per-document context-parallel baseline (every long document cut over all ranks, no balancer)")
    ap.add_argument("--nano-batches", type=int, default=1, choices=[1, 2],
                    help="2: ping-pong schedule over two nano-batches per rank")
    ap.add_argument("--no-fuse-qkv-rope", action="store_true",
                    help="separate RoPE / dispatch kernel instead of the QKV GEMM epilogue (for A/B timing)")
    ap.add_argument("--config", default="headline", choices=["headline", *NAMED_CONFIGS],
                    help="headline: the dp{N} + CAD scaling benchmark (default); the others are fixed 8-GPU layouts: "
                         + "; ".join(f"{k}: {v['what']}" for k, v in NAMED_CONFIGS.items()))
    ap.add_argument("--baseline-mode", default="none", choices=["none", "percp", "perseq"],
                    help="percp: the no-CAD per-document context-parallel baseline on the same documents (all-gather K/V; "
                         "with --config: tensor parallel x context parallel over the remaining ranks; on the headline "
                         "layout: context parallel over all GPUs); perseq: the same with packed sequences cut over the "
                         "ranks instead of documents (per-sequence context parallelism)")
    ap.add_argument("--microbatches", type=int, default=None, help="micro-batches per step of a pipelined --config")
    ap.add_argument("--phase-timers", action="store_true",
                    help="CUDA-event phase timers in the device-timed region; the JSON line gains phases_ms_per_step")
    ap.add_argument("--recompute", default=None, choices=["full", "keep_attn"],
                    help="keep_attn: recompute every layer in backward except core attention, whose output is kept "
                         "(HBM or pinned host memory); falls back to full when neither has room")
    return ap.parse_args()


def reference_arm(a) -> None:
    """The reference trains through Megatron-LM + TransformerEngine (+ omegaconf); none of them is present
    offline, so its public entry point cannot start. Its own communication layer does build and run here: that
    arm is ``python -m distca_b200.utils.fa2a_bench --impl reference``."""
    why = None
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "distca")):
        why = "reference package not installed under baseline/_ref"
    else:
        missing = []
        for mod in ("megatron.core", "transformer_engine", "omegaconf"):
            try:
                __import__(mod)
            except Exception:
                missing.append(mod)
        if missing:
            why = ("the reference's training entry point imports " + ", ".join(missing) + ", absent offline (its package "
                   "installs and its NVSHMEM library builds for sm_100a: the communication arm runs, "
                   "python -m distca_b200.utils.fa2a_bench --impl reference)")
        else:
            why = "reference dependencies present but its launcher is not wired on this box"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))


class ClockSampler:
    """nvidia-smi clocks/throttle reasons every 200 ms while the timed regions run (rank 0 only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc, self.path = None, f"/tmp/bench_clocks_{os.getpid()}.csv"
        try:
            self.f = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.f.close()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1])); mx.append(float(p[2])); power.append(float(p[3]))
                except ValueError:
                    continue
                for n, v in zip(names, p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if sm:
            busy = [s for s, w in zip(sm, power) if w > 300] or sm
            out = {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "power_w_max": max(power), "samples": len(sm)}
        return out


def run_named_config(a) -> None:
    """One of the fixed 8-GPU layouts (``--config``): every step goes through the public ``train_step`` call
    (pinned host batch in, loss out); timed with CUDA events around each step and with the wall clock around
    all of them, maximum over ranks. ``--baseline-mode percp`` runs the per-document context-parallel baseline
    on the same global batches instead (TP unchanged, the other ranks form one context-parallel group)."""
    import torch
    import torch.distributed as dist
    from distca_b200.models.config import ParallelConfig, TrainConfig, get_model_config
    from distca_b200.runtime.trainer import BatchSource, Trainer, init_distributed
    from distca_b200.utils import timers

    spec = dict(NAMED_CONFIGS[a.config])
    rank, world, local = init_distributed()
    tp, pp, dp = spec["tp"], spec["pp"], spec["dp"]
    M = a.microbatches or spec["microbatches"]
    seq_len = a.seq_len or spec["seq_len"]
    percp = a.baseline_mode in ("percp", "perseq")       # perseq: chunks of packed sequences instead of documents
    seqs_per_step = dp * spec["seqs_per_rank"] * (M if pp > 1 else 1)
    if percp:
        # same global batch; pipeline and data-parallel ranks become one context-parallel group
        dp, pp = dp * pp, 1
    assert world == tp * pp * dp, f"--config {a.config} needs {tp * pp * dp} GPUs, WORLD_SIZE={world}"
    # --model other than the default replaces the layout's model (debugging a layout on a small model)
    cfg = get_model_config(spec["model"] if a.model == "llama3-8b" else a.model, a.num_layers)
    par = ParallelConfig(tp=tp, pp=pp, dp=dp)
    recompute = a.recompute or spec["recompute"]
    tc = TrainConfig(cad=not (a.no_cad or percp), recompute=recompute, comm_buffer_gb=a.comm_buffer_gb)
    tc.extra.update(tolerance=a.tolerance, attention_policy=a.attention_policy, fuse_qkv_rope=not a.no_fuse_qkv_rope,
                    baseline_mode=a.baseline_mode, cp_seq_len=seq_len)
    if pp > 1 and tc.cad:
        tc.extra["nano_batches"] = a.nano_batches     # ping-pong nano-batches inside the pipeline stages
    if pp > 1:
        from distca_b200.parallel.pipeline import PipelineTrainer
        trainer = PipelineTrainer(cfg, par, tc, num_microbatch=M, seed=0)
        seqs_per_rank = M * spec["seqs_per_rank"]
    else:
        trainer = Trainer(cfg, par, tc, seed=0)
        seqs_per_rank = seqs_per_step // dp
    dev = trainer.device

    def source(seed):
        if percp:
            # one stream of seqs_per_step sequences; every rank takes the whole batch and cuts its chunks
            return BatchSource(cfg, ParallelConfig(tp=1, pp=1, dp=seqs_per_step), seq_len, spec["dist"], seed=seed)
        return BatchSource(cfg, par, seq_len, spec["dist"], seed=seed, seqs_per_rank=seqs_per_rank)

    def draw(src):
        return src.next_global() if percp else src.next(trainer.dp_rank)

    def barrier():
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)

    warm_src, src = source(99), source(1234)
    losses = [trainer.train_step(draw(warm_src)) for _ in range(a.warmup)]
    batches = [draw(src) for _ in range(a.steps)]
    sampler = ClockSampler(local) if rank == 0 else None
    from distca_b200.ops import _lib
    torch.cuda.reset_peak_memory_stats(dev)
    barrier()
    timers.enable(True)
    launches0 = _lib.LAUNCHES
    events = []
    t0 = time.perf_counter()
    for i, hb in enumerate(batches):
        if i + 1 < len(batches) and hasattr(trainer, "prefetch_plan") and not percp:
            trainer.prefetch_plan(batches[i + 1])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        losses.append(trainer.train_step(hb))
        e1.record()
        events.append((e0, e1))
    barrier()
    ms_e2e = (time.perf_counter() - t0) * 1e3
    ms_dev = sum(x.elapsed_time(y) for x, y in events)
    launches = _lib.LAUNCHES - launches0
    phases = timers.GLOBAL.summary()
    timers.enable(False)
    clocks = sampler.stop() if sampler is not None else None
    exposed = sum(v for k, v in phases.items() if k.removeprefix("re_").startswith("cad_wait")
                  or k.removeprefix("re_") in ("cad_dispatch", "cad_return")) / a.steps
    attn_ms = sum(v for k, v in phases.items() if k.removeprefix("re_") in ("cad_attn_fwd", "cad_attn_bwd")) / a.steps
    free, total_mem = torch.cuda.mem_get_info(dev)
    t = torch.tensor([ms_dev, ms_e2e, exposed, attn_ms, (total_mem - free) / 2**30], dtype=torch.float64, device=dev)
    tsum = torch.tensor([attn_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    ms_dev, ms_e2e, exposed, attn_max, mem_gb = (float(x) for x in t)
    attn_mean = float(tsum[0]) / world
    tokens = seq_len * seqs_per_step * a.steps
    if percp:
        docs_of = lambda hb: [hb.doc_lens]
        h2d = batches[0].tokens.numel() // dp * 20
    else:
        docs_of = lambda hb: hb.all_doc_lens
        h2d = batches[0].nbytes()
    lin_flop = 3.0 * cfg.flops_per_token_linear() * tokens
    attn_flop = sum(3.0 * 2.0 * float(L) * L * cfg.head_dim * cfg.heads_q * cfg.num_layers
                    for hb in batches for docs in docs_of(hb) for L in docs)
    if rank == 0:
        cad_rt = getattr(trainer, "cad", None)
        out = {
            "metric": f"{cfg.name}_{a.config}_tokens_per_sec_box", "value": tokens / (ms_dev / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_dev / a.steps,
            "higher_is_better": True, "scaling": "fixed 8-GPU layout", "vs_baseline": None, "dtype": "bf16",
            "data": f"synthetic packed documents ({spec['dist']}), random-init weights",
            "config": {"model": cfg.name, "layers": cfg.num_layers, "global_batch": seqs_per_step, "seq_len": seq_len,
                       "parallelism": f"tp{tp}-" + (f"cp{dp}-{a.baseline_mode}" if percp else f"pp{pp}-dp{dp}" + ("-cad" if cad_rt is not None else "")),
                       "microbatches": M if pp > 1 else 1, "recompute": recompute,
                       "nano_batches": int(tc.extra.get("nano_batches", 1)),
                       "grad_dtype": str(trainer.model.store.grad.dtype).replace("torch.", ""),
                       "tp_transport": "p2p" if (tp > 1 and getattr(trainer.model.tp, "use_p2p", False)) else ("nccl" if tp > 1 else None),
                       "dp_transport": "p2p" if getattr(trainer, "p2p", None) is not None else ("nccl" if dp > 1 else None),
                       "l2": "working set of every kernel exceeds L2 (inputs larger than L2)"},
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            "model_flops": {"linear_pflop_per_step": lin_flop / a.steps / 1e15,
                            "attention_pflop_per_step": attn_flop / a.steps / 1e15,
                            "achieved_pflops_per_gpu": (lin_flop + attn_flop) / (ms_dev / 1e3) / 1e15 / world},
            "memory_gb_max_over_ranks": mem_gb, "clocks": clocks, "loss_first_last": [losses[0], losses[-1]],
            "impl": "ours",
        }
        if getattr(trainer, "last_schedule", None):
            out["pipeline"] = trainer.last_schedule
        if cad_rt is not None:
            out["cad"] = {"planned_imbalance_after": cad_rt.plan_stats.get("imbalance_after"),
                          "planned_cost_imbalance_after": cad_rt.plan_stats.get("cost_imbalance_after"),
                          "server_speed": cad_rt.plan_stats.get("speed"),
                          "exposed_dispatch_ms_per_step": exposed,
                          "attention_ms_per_step_max_over_ranks": attn_max,
                          "attention_time_imbalance_max_over_mean": (attn_max / attn_mean) if attn_mean > 0 else None,
                          "tolerance": a.tolerance}
        if percp:
            out["percp"] = {"kv_bytes_received_per_layer_and_rank": trainer.percp.bytes_per_layer}
        if a.phase_timers:
            out["phases_ms_per_step"] = {k: round(v / a.steps, 2) for k, v in sorted(phases.items())}
        print(json.dumps(out))
    trainer.close()
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    a = _args()
    if a.impl == "reference":
        reference_arm(a)
        return
    if a.config != "headline":
        run_named_config(a)
        return
    if a.baseline_mode in ("percp", "perseq"):
        # the headline layout (one 128K pack per GPU) under per-document context parallelism instead of CAD:
        # the like-for-like arm of the two attention schemes (same documents, same GPUs, TP = PP = 1)
        NAMED_CONFIGS["headline_layout"] = {
            "what": "headline layout", "model": a.model, "tp": 1, "pp": 1, "dp": a.gpus, "seq_len": a.seq_len or 131072,
            "seqs_per_rank": 1, "microbatches": 1, "dist": a.dist, "recompute": a.recompute or "keep_attn"}
        a.config = "headline_layout"
        run_named_config(a)
        return
    import torch
    import torch.distributed as dist
    from distca_b200.models.config import ParallelConfig, TrainConfig, get_model_config
    from distca_b200.ops import _lib
    from distca_b200.runtime.trainer import BatchSource, Trainer, init_distributed

    rank, world, local = init_distributed()
    assert world == a.gpus, f"--gpus {a.gpus} but WORLD_SIZE={world}"
    a.seq_len = a.seq_len or 131072
    a.recompute = a.recompute or "keep_attn"
    cfg = get_model_config(a.model, a.num_layers)
    par = ParallelConfig(tp=1, pp=1, dp=world)
    tc = TrainConfig(cad=not a.no_cad, recompute=a.recompute, comm_buffer_gb=a.comm_buffer_gb)
    tc.extra["tolerance"] = a.tolerance
    tc.extra["attention_policy"] = a.attention_policy
    tc.extra["nano_batches"] = a.nano_batches
    tc.extra["fuse_qkv_rope"] = not a.no_fuse_qkv_rope
    trainer = Trainer(cfg, par, tc, seed=0)
    # warm-up and timed steps draw from separate streams, so the timed documents do not depend on --warmup
    warm_src = BatchSource(cfg, par, a.seq_len, a.dist, seed=99)
    src = BatchSource(cfg, par, a.seq_len, a.dist, seed=1234)
    dev = trainer.device

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    losses = []
    for _ in range(a.warmup):
        losses.append(trainer.train_step(warm_src.next(trainer.dp_rank)))
    trainer.check_device_status()

    sampler = ClockSampler(local) if rank == 0 else None
    # ---- region A: device-timed, inputs resident on the device ----
    staged = []
    for _ in range(a.steps):
        hb = src.next(trainer.dp_rank)
        if a.nano_batches == 2:
            from distca_b200.runtime.trainer import split_nano
            nano = split_nano(hb)
            staged.append((hb, (nano, [trainer.to_device(n) if n.ids.numel() else None for n in nano])))
        else:
            staged.append((hb, trainer.to_device(hb)))
    barrier()
    from distca_b200.utils import timers
    timers.enable(trainer.cad is not None or a.phase_timers)   # CUDA-event phase timers (no host sync)
    launches0 = _lib.LAUNCHES
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    dev_losses = []
    for hb, batch in staged:
        if a.nano_batches == 2:
            trainer.plan_attention_nano(batch[0])
            dev_losses.append(trainer.train_step_prepared(batch[1], hb))
        else:
            trainer.plan_attention(hb)
            dev_losses.append(trainer.train_step_prepared(batch, hb))
    e1.record()
    barrier()
    launches = _lib.LAUNCHES - launches0
    ms_dev = e0.elapsed_time(e1)
    phases = timers.GLOBAL.summary()
    timers.enable(False)
    exposed = sum(v for k, v in phases.items() if k.removeprefix("re_").startswith("cad_wait")
                  or k.removeprefix("re_") in ("cad_dispatch", "cad_return")) / a.steps
    attn_ms = sum(v for k, v in phases.items() if k.removeprefix("re_") in ("cad_attn_fwd", "cad_attn_bwd")) / a.steps
    losses += [float(x.item()) for x in dev_losses]
    # ---- region B: end to end through Trainer.train_step (H2D of inputs + D2H of the loss per step),
    #      on the same documents as region A so the two numbers differ only by the host traffic ----
    host_batches = [hb for hb, _ in staged]
    del staged
    h2d = host_batches[0].nbytes()
    barrier()
    t0 = time.perf_counter()
    for i, hb in enumerate(host_batches):
        if i + 1 < len(host_batches):
            trainer.prefetch_plan(host_batches[i + 1])   # the planner works on step i+1 while step i runs
        losses.append(trainer.train_step(hb))
    barrier()
    ms_e2e = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if sampler is not None else None
    trainer.check_device_status()

    t = torch.tensor([ms_dev, ms_e2e, exposed, attn_ms], dtype=torch.float64, device=dev)
    tsum = torch.tensor([attn_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    ms_dev, ms_e2e, exposed, attn_max = float(t[0]), float(t[1]), float(t[2]), float(t[3])
    attn_mean = float(tsum[0]) / world
    tokens = a.seq_len * world * a.steps
    # model FLOPs of the timed steps (no recompute counted): 6 * weights * tokens for the GEMMs and
    # 3 x the causal forward 2 * L^2 * head_dim * heads_q per document and layer for core attention
    lin_flop = 3.0 * cfg.flops_per_token_linear() * tokens
    attn_flop = sum(3.0 * 2.0 * float(L) * L * cfg.head_dim * cfg.heads_q * cfg.num_layers
                    for hb in host_batches for docs in hb.all_doc_lens for L in docs)
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    full = a.num_layers is None and a.model == "llama3-8b" and a.seq_len == 131072
    store = trainer.model._store
    store_where = store.placement if store is not None else None
    if rank == 0:
        out = {
            "metric": "llama3_8b_128k_tokens_per_sec_box" if full else f"{cfg.name}_{a.seq_len}_tokens_per_sec_box",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": ms_dev / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic packed documents (mixture of log-uniform lengths), random-init weights",
            "config": {"model": cfg.name, "layers": cfg.num_layers, "global_batch": world, "seq_len": a.seq_len,
                       "parallelism": (f"dp{world}-{a.attention_policy}" if trainer.cad is not None else f"dp{world}"),
                       "recompute": trainer.model.recompute, "nano_batches": a.nano_batches,
                       "grad_dtype": str(trainer.model.store.grad.dtype).replace("torch.", ""),
                       "dp_transport": "p2p" if trainer.p2p is not None else ("nccl" if world > 1 else None), "attention_outputs_kept_in": store_where, "optimizer": "sharded AdamW, fp32 master weights (bf16 + 16-bit remainder)",
                       "l2": "working set of every kernel exceeds L2 (inputs larger than L2)"},
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "activation_offload_bytes_per_step_each_way": (
                        store.where.count("host") * a.seq_len * cfg.q_dim * 2 if store is not None else 0)},
            "gpu_launches": launches,
            "model_flops": {"linear_pflop_per_step": lin_flop / a.steps / 1e15, "attention_pflop_per_step": attn_flop / a.steps / 1e15,
                            "achieved_pflops_per_gpu": (lin_flop + attn_flop) / (ms_dev / 1e3) / 1e15 / world,
                            "note": "model FLOPs (recompute not counted); attention share varies with the documents drawn"},
            "clocks": clocks,
            "loss_first_last": [losses[0], losses[-1]],
            "impl": "ours",
        }
        if a.phase_timers:
            out["phases_ms_per_step"] = {k: round(v / a.steps, 2) for k, v in sorted(phases.items())}
        if trainer.cad is not None:
            # achieved / roofline of the fused compute + communication paths (rank 0's traffic of the last plan)
            from distca_b200.utils.observability import fused_path_rooflines
            peaks = {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "link_gbs": 770.0, "source": "fallback"}
            pk = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
            if os.path.exists(pk):
                with open(pk) as f:
                    mp = json.load(f)
                if "bf16_tflops_sustained" in mp and "hbm_gbs" in mp:
                    peaks.update(bf16_tflops=mp["bf16_tflops_sustained"], hbm_gbs=mp["hbm_gbs"],
                                 source="measured (sustained GEMM)")
            try:
                sb = list(trainer.cad.plan_stats.get("send_bytes", [0] * world))
                remote = float(sum(sb) - (sb[trainer.cad.me] if trainer.cad.me < len(sb) else 0))
                q_share = cfg.q_dim / (cfg.q_dim + 2.0 * cfg.kv_dim)    # the return trip carries O (forward) / dQ + copies (backward)
                nparam = trainer.model.store.numel
                gb = trainer.model.store.grad.element_size()
                out["roofline"] = {"peaks": peaks, "paths": fused_path_rooflines(
                    phases, a.steps, tokens_per_rank=a.seq_len, hidden=cfg.hidden, qkv_dim=cfg.qkv_dim, layers=cfg.num_layers,
                    passes_qkv=2, attn_flops_fwd_per_rank=attn_flop / 3.0 / a.steps / world, remote_dispatch_bytes=remote,
                    remote_return_bytes=remote * q_share, grad_bytes_in=nparam * gb * (world - 1) / world,
                    param_bytes_out=nparam * 2 * (world - 1) / world,
                    optimizer_hbm_bytes=nparam / world * (gb * world + 2 + 2 + 16 + 2 * world), peaks=peaks)}
            except Exception as e:   # a diagnostic block must never cost the measurement its output line
                out["roofline"] = {"peaks": peaks, "error": repr(e)}
            out["cad"] = {"planned_imbalance_after": trainer.cad.plan_stats.get("imbalance_after"),
                          "planned_imbalance_before": trainer.cad.plan_stats.get("imbalance_before"),
                          "planned_cost_imbalance_after": trainer.cad.plan_stats.get("cost_imbalance_after"),
                          "server_speed": trainer.cad.plan_stats.get("speed"),
                          "exposed_dispatch_ms_per_step": exposed,
                          "attention_ms_per_step_max_over_ranks": attn_max,
                          "attention_time_imbalance_max_over_mean": (attn_max / attn_mean) if attn_mean > 0 else None,
                          "tolerance": a.tolerance}
        print(json.dumps(out))
    trainer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
