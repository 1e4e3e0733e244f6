"""Training entry point with the argument surface of the reference's ``pretrain_llama.py``
(pretrain_llama.py:871-943 there) plus explicit switches for what the reference hides in
environment variables: the CAD toggle, the communication-buffer size, recompute policy,
baseline mode and Megatron-layout checkpoints.

    torchrun --nnodes 1 --nproc-per-node 8 pretrain_llama.py --model llama3-8b --num-tokens 131072 \
        --tp-size 1 --pp-size 1 --dp-size 8 --num-batches 1 --max-sample-id 10 --cad --comm-buffer-gb 6

    python pretrain_llama.py --model tiny-128 --num-tokens 1024 --num-layers 1 --max-sample-id 1   # smoke

World size must equal ``tp * pp * dp`` (``--cp-size`` is accepted as the reference's name for the
data-parallel degree). Every step: sample documents, pack ``--num-batches`` sequences of
``--num-tokens`` tokens per data-parallel rank, plan core attention, forward/backward, reduce
gradients, AdamW update. Artifacts (``config.json``, ``benchmark.raw.jsonl``, ``benchmark.json``,
``plan_inspect.jsonl``, ``mem.rank*.jsonl``, ``logs/``) go to ``--output-dir``.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import numpy as np

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    # --- reference flags ---
    ap.add_argument("--num-tokens", type=int, default=1024, help="tokens per packed sequence")
    ap.add_argument("--num-batches", type=int, default=1, help="packed sequences per data-parallel rank and step")
    ap.add_argument("--cp-size", type=int, default=None, help="reference name of the data-parallel degree")
    ap.add_argument("--dp-size", type=int, default=None)
    ap.add_argument("--num-seqs", type=int, default=None, help="unused; kept for command-line compatibility")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--num-nodes", type=int, default=1)
    ap.add_argument("--num-gpus-per-node", type=int, default=None)
    ap.add_argument("--tp-size", type=int, default=1)
    ap.add_argument("--pp-size", type=int, default=1)
    ap.add_argument("--num-microbatch", type=int, default=1)
    ap.add_argument("--use-planner", action="store_true", default=True)
    # shaping of the wlbllm / prolong length distributions and of local corpora, with the reference's defaults
    # (pretrain_llama.py:887-901): documents below the threshold are kept with probability filter-ratio, longer
    # ones count up-sample-factor times, lengths are stretched by elongate-factor
    ap.add_argument("--up-sample-factor", type=int, default=4)
    ap.add_argument("--elongate-factor", type=int, default=1)
    ap.add_argument("--filter-threshold", type=int, default=65536)
    ap.add_argument("--filter-ratio", type=float, default=0.50)
    ap.add_argument("--sample-name", default="mixture",
                    choices=["wlbllm", "prolong", "mixture", "loguniform", "loguniform64", "full",
                             "bookcorpus", "wikitext", "openwebtext", "c4"])
    ap.add_argument("--check-for-nan-in-loss", dest="check_nan", action="store_true", default=True)
    ap.add_argument("--no-check-for-nan-in-loss", dest="check_nan", action="store_false")
    ap.add_argument("--check-for-spiky-loss", type=float, default=0.0, metavar="FACTOR",
                    help="stop when the loss exceeds FACTOR x the largest loss seen so far (0 = off)")
    ap.add_argument("--check-for-large-grads", type=float, default=0.0, metavar="FACTOR",
                    help="stop when the gradient norm exceeds FACTOR x the largest seen so far (0 = off)")
    ap.add_argument("--quit-if-maybe-oom", action="store_true",
                    help="estimate the per-GPU memory of the configuration first and refuse to start if it does not fit")
    ap.add_argument("--torch-profile-step", type=int, default=-1, help="write a torch.profiler chrome trace of this step")
    ap.add_argument("--cost-model-file", default=None,
                    help="output of `python -m distca_b200.utils.kernel_bench --kernel attn_sweep` on this machine: the "
                         "planner's attention cost model is fitted to it instead of the built-in B200 constants")
    ap.add_argument("--bind-cpus", action="store_true",
                    help="bind every rank to its own contiguous slice of the host's CPUs and write the per-rank "
                         "environment record (<output-dir>/envs/)")
    ap.add_argument("--check-finite", action="store_true",
                    help="debug: test every layer's output and input gradient for NaN / Inf and name the first one "
                         "(one device synchronisation per layer pass; non-pipelined, one nano-batch)")
    ap.add_argument("--record-memory-history", action="store_true",
                    help="record the caching allocator's history: memory.rank{r}.pickle after the second step and "
                         "oom.rank{r}.pickle when an allocation fails (PyTorch memory visualiser format)")
    ap.add_argument("--trace-calls-step", type=int,
                    default=0 if os.environ.get("EXPERIMENT_PYTHON_DEBUG_TRACE_CALLS", "0") == "1" else -1,
                    help="log every Python call of this package during this step to <output-dir>/calls.rank{r}.log "
                         "(which rank is stuck where; heavy)")
    ap.add_argument("--span-documents", action="store_true",
                    help="lay the documents of a global batch out over the ranks by sequential fill, so a document "
                         "may be longer than one rank's tokens (--max-total-tokens bounds its length); needs --cad, no pipeline")
    ap.add_argument("--data-path", default=None, help="local .txt / .jsonl corpus instead of synthetic documents")
    ap.add_argument("--tokenizer-path", default=None, help="local Hugging Face tokenizer directory (default: UTF-8 bytes)")
    ap.add_argument("--change-long-doc-ratio", type=float, default=0.0)
    ap.add_argument("--packing", default="sequential", choices=["sequential", "wlb"],
                    help="wlb: workload-balanced packing of every global batch (WLB-LLM: documents longest first to the "
                         "pack with the least (l/B)^2 + l/B work, equal tokens per pack) instead of packing in order")
    ap.add_argument("--max-total-tokens", type=int, default=None)
    ap.add_argument("--model-path", default=None, help="HuggingFace config.json (or its directory)")
    ap.add_argument("--num-layers", type=int, default=None)
    ap.add_argument("--max-sample-id", type=int, default=3, help="number of training steps")
    ap.add_argument("--should-add-debug-cases", action="store_true",
                    help="start the stream with packs of one full-length document each (heaviest balanced case)")
    ap.add_argument("--val-every-n-steps", type=int, default=0)
    ap.add_argument("--ckpt-every-n-steps", type=int, default=0)
    ap.add_argument("--output-dir", default=None)
    ap.add_argument("--enable-wandb", action="store_true")
    ap.add_argument("--wandb-project", default="distca_b200")
    ap.add_argument("--wandb-run-name", default=None)
    ap.add_argument("--allow-all-ranks-loss", action="store_true", help="every rank logs its step lines")
    # --- switches the reference keeps in the environment or in test scripts ---
    ap.add_argument("--model", default="tiny-128", help="preset: tiny | tiny-128 | small-128 | llama3-8b | codellama-34b")
    ap.add_argument("--cad", dest="cad", action="store_true", default=True)
    ap.add_argument("--no-cad", dest="cad", action="store_false")
    ap.add_argument("--comm-buffer-gb", type=float, default=float(os.environ.get("EXPERIMENT_NVSHMEM_BUFFER_SIZE_GB", 2.0)))
    ap.add_argument("--recompute", default=None, choices=["none", "selective", "full", "keep_attn"],
                    help="keep_attn (default without pipeline stages; with them: full): recompute every layer in backward except core attention, whose output is kept in HBM or pinned host memory; full: recompute whole layers; none: keep all activations")
    ap.add_argument("--baseline-mode", default="none", choices=["none", "percp", "perseq"],
                    help="percp: no core-attention disaggregation; the data-parallel ranks form a per-document "
                         "context-parallel group instead (every document cut over all of them, K/V all-gathered, "
                         "dK/dV reduce-scattered with NCCL): the comparison point of the reference's --mode wlbllm; "
                         "perseq: the same with every packed SEQUENCE cut over the ranks wherever its documents end "
                         "(per-sequence context parallelism: balanced tokens, unbalanced attention work)")
    ap.add_argument("--tp-transport", default="p2p", choices=["p2p", "p2p-tile", "nccl"],
                    help="tensor-parallel collectives: p2p = shards gathered once by peer stores + reduce-scatter in the "
                         "GEMM epilogue; p2p-tile = all-gather in the GEMM's operand load as well (every CTA loads the "
                         "remote tiles it needs); nccl = NCCL collectives")
    ap.add_argument("--dp-transport", default="p2p", choices=["p2p", "nccl"],
                    help="gradient reduce-scatter / parameter all-gather: fused kernels over peer memory, or NCCL")
    ap.add_argument("--attention-policy", default="cad", choices=["cad", "cp", "water_fill"],
                    help="cad: balanced core-attention disaggregation; cp: per-document context-parallel baseline")
    ap.add_argument("--tolerance", type=float, default=float(os.environ.get("MIN_TOLERANCE_FACTOR", 0.1)))
    ap.add_argument("--pingpong", dest="pingpong", action="store_true", default=False,
                    help="two nano-batches per rank and step, interleaved layer by layer (the reference's ping-pong "
                         "schedule); off by default, like bench.py: on one stream it measured the same speed")
    ap.add_argument("--no-pingpong", dest="pingpong", action="store_false")
    ap.add_argument("--fuse-ticks", action="store_true",
                    help="with --pingpong: per nano-batch, run the next layer's pre-attention half (and its Q/K/V "
                         "dispatch) right after this layer's post-attention half, as the reference's fused ticks do")
    ap.add_argument("--save", default=None, help="checkpoint directory (Megatron layout)")
    ap.add_argument("--load", default=None)
    ap.add_argument("--save-interval", type=int, default=0)
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--weight-decay", type=float, default=0.01)
    ap.add_argument("--clip-grad", type=float, default=1.0)
    ap.add_argument("--grad-dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--log-memory", action="store_true", default=os.environ.get("EXPERIMENT_LOG_MEMORY_USAGE", "0") == "1")
    ap.add_argument("--phase-timers", action="store_true")
    ap.add_argument("--wait-report-ms", type=float, default=(float(os.environ["DISTCA_WAIT_REPORT_MS"])
                                                              if os.environ.get("DISTCA_WAIT_REPORT_MS") else None),
                    help="record every signal wait of the attention servers that kept the stream idle for longer than "
                         "this many milliseconds (which wait, which layer, how long) in the step records")
    ap.add_argument("--nvtx", action="store_true", help="NVTX ranges per step, tick, layer pass and phase")
    return ap.parse_args(argv)


def main(argv=None) -> int:
    a = parse_args(argv)
    import torch
    import torch.distributed as dist
    from distca_b200.models.config import ParallelConfig, TrainConfig, get_model_config
    from distca_b200.runtime.trainer import BatchSource, Trainer, init_distributed
    from distca_b200.utils import timers
    from distca_b200.utils.checkpoint import load_checkpoint, save_checkpoint
    from distca_b200.utils.observability import MemoryLog, RunArtifacts, get_logger, inspect_plan, nvtx_range

    rank, world, local = init_distributed()
    if os.environ.get("EXPERIMENT_PYTHON_BETTER_TRACEBACK", "1") == "1":
        from distca_b200.utils.profiler import install_rank_excepthook
        install_rank_excepthook(rank)
    dp = a.dp_size or a.cp_size or max(1, world // (a.tp_size * a.pp_size))
    par = ParallelConfig(tp=a.tp_size, pp=a.pp_size, dp=dp)
    if par.world != world:
        raise SystemExit(f"world size {world} != tp {a.tp_size} x pp {a.pp_size} x dp {dp}")
    if a.num_gpus_per_node is not None and a.num_nodes * a.num_gpus_per_node != world:
        raise SystemExit(f"world size {world} != --num-nodes {a.num_nodes} x --num-gpus-per-node {a.num_gpus_per_node}")
    if a.pp_size > 1 and a.num_microbatch < a.pp_size:
        raise SystemExit("--num-microbatch must be at least --pp-size")
    cfg = get_model_config(a.model_path or a.model, a.num_layers)
    if a.recompute is None:
        # pipeline stages keep the attention outputs of every micro-batch in flight in HBM: opt-in there
        a.recompute = "keep_attn" if a.pp_size == 1 else "full"
    recompute = {"full": "full", "selective": "full", "keep_attn": "keep_attn", "none": "none"}[a.recompute]
    cad = a.cad and a.baseline_mode == "none"
    tc = TrainConfig(lr=a.lr, weight_decay=a.weight_decay, clip_grad=a.clip_grad, recompute=recompute,
                     grad_dtype=a.grad_dtype, cad=cad, pingpong=a.pingpong, comm_buffer_gb=a.comm_buffer_gb)
    tc.extra["tolerance"] = a.tolerance
    tc.extra["attention_policy"] = a.attention_policy
    tc.extra["baseline_mode"] = a.baseline_mode
    tc.extra["cp_seq_len"] = a.num_tokens          # per-sequence CP cuts every packed sequence over the ranks
    tc.extra["tp_transport"] = a.tp_transport
    tc.extra["dp_transport"] = a.dp_transport
    if a.wait_report_ms is not None:
        tc.extra["wait_report_ms"] = a.wait_report_ms
    tc.extra["check_finite"] = a.check_finite
    tc.extra["fuse_ticks"] = a.fuse_ticks
    if a.cost_model_file:
        tc.extra["cost_model_file"] = a.cost_model_file
    if a.baseline_mode in ("percp", "perseq") and a.pp_size > 1:
        raise SystemExit(f"--baseline-mode {a.baseline_mode} has no pipeline stages: use --pp-size 1")
    # ping-pong nano-batches: in the non-pipelined trainer and inside pipeline stages alike
    tc.extra["nano_batches"] = 2 if (a.pingpong and cad and dp * a.pp_size > 1 and not a.span_documents) else 1
    if a.quit_if_maybe_oom:
        import torch as _t
        from distca_b200.utils.guards import estimate_memory_gb, quit_if_maybe_oom
        cap = _t.cuda.get_device_properties(local).total_memory / 1e9 if _t.cuda.is_available() else 180.0
        quit_if_maybe_oom(estimate_memory_gb(cfg, par, a.num_tokens * a.num_batches, recompute=recompute, cad=cad,
                                             comm_buffer_gb=a.comm_buffer_gb, nano_batches=tc.extra["nano_batches"],
                                             microbatches_in_flight=min(a.num_microbatch, a.pp_size) if a.pp_size > 1 else 1),
                          cap)
    if a.allow_all_ranks_loss or os.environ.get("ALLOW_ALL_RANKS_LOSS", "0") == "1":
        os.environ["DISTCA_LOG_ALL_RANKS"] = "1"          # every rank prints its step lines, not only rank 0
    log = get_logger(rank=rank, out_dir=a.output_dir)
    if a.bind_cpus:
        from distca_b200.utils import affinity
        affinity.bind(local, int(os.environ.get("LOCAL_WORLD_SIZE", a.num_gpus_per_node or world)), logger=log)
        if a.output_dir:
            affinity.dump_environment(a.output_dir, rank, local)
    art = RunArtifacts(a.output_dir, rank)
    art.write_config({"args": vars(a), "model": cfg.__dict__, "parallel": par.__dict__, "world": world})
    mem = MemoryLog(a.output_dir, rank, enabled=a.log_memory)
    mem_hist = None
    if a.record_memory_history:
        from distca_b200.utils.observability import MemoryHistory
        mem_hist = MemoryHistory(a.output_dir or ".", rank).start()
    from distca_b200.utils.observability import MetricsSink
    sink = MetricsSink(a.enable_wandb, rank, a.wandb_project, a.wandb_run_name, vars(a), a.output_dir)
    # with CAD the phase timers are always on: they give the exposed dispatch time and the attention time per
    # server of every step (CUDA events only: no host synchronisation inside the step)
    timers.enable(a.phase_timers or (cad and world > 1 and torch.cuda.is_available()))
    timers.enable_nvtx(a.nvtx)

    if par.pp > 1:
        from distca_b200.parallel.pipeline import PipelineTrainer
        trainer = PipelineTrainer(cfg, par, tc, num_microbatch=a.num_microbatch, seed=a.seed)
    else:
        trainer = Trainer(cfg, par, tc, seed=a.seed)
    start_it = 0
    if a.load:
        start_it = load_checkpoint(a.load, trainer.model, trainer.opt, cfg, tp_rank=trainer.tp_rank, tp_size=par.tp,
                                   pp_rank=trainer.pp_rank, pp_size=par.pp, dp_rank=trainer.dp_rank)
        log.info("resumed from %s at iteration %d", a.load, start_it)
    max_len = a.num_tokens * a.elongate_factor if a.max_total_tokens is None else a.max_total_tokens
    seqs_per_rank = a.num_batches * (a.num_microbatch if par.pp > 1 else 1)
    stream = None
    if a.data_path:
        from distca_b200.data.text import TextBatches
        stream = TextBatches(a.data_path, a.num_tokens, par.dp * seqs_per_rank, cfg.vocab, a.tokenizer_path, a.seed,
                             a.elongate_factor, a.up_sample_factor, a.filter_threshold, a.filter_ratio)
    src = BatchSource(cfg, par, a.num_tokens, a.sample_name if a.sample_name in
                      ("wlbllm", "prolong", "mixture", "loguniform", "loguniform64", "full") else "wlbllm",
                      seed=a.seed, seqs_per_rank=seqs_per_rank, stream=stream,
                      shape=dict(up_sample_factor=a.up_sample_factor, filter_threshold=a.filter_threshold,
                                 filter_ratio=a.filter_ratio, elongate_factor=a.elongate_factor,
                                 change_long_doc_ratio=a.change_long_doc_ratio),
                      debug_packs=1200 if a.should_add_debug_cases else 0, packing=a.packing)
    src.stream.max_doc_len = min(max_len, a.num_tokens)
    log.info("model %s (%.2fB params) world %d = tp%d x pp%d x dp%d, cad=%s recompute=%s", cfg.name,
             cfg.num_params() / 1e9, world, par.tp, par.pp, par.dp, cad, recompute)
    mem.log("after_init")

    tokens_per_step = a.num_tokens * seqs_per_rank * par.dp
    save_dir = a.save or (os.path.join(a.output_dir, "checkpoints") if a.output_dir and a.ckpt_every_n_steps else None)
    save_every = a.save_interval or a.ckpt_every_n_steps
    from distca_b200.utils.guards import TrainingGuards
    from distca_b200.utils.profiler import ProfilerCtx
    guards = TrainingGuards(a.check_nan, a.check_for_spiky_loss, a.check_for_large_grads)
    percp = a.baseline_mode in ("percp", "perseq") and par.dp > 1
    draw = (lambda: src.next_global()) if percp else (lambda: src.next(trainer.dp_rank))
    for _ in range(start_it):
        draw()                        # resume: the data stream continues where the saved run stopped
    hb_next = draw()
    for it in range(start_it, start_it + a.max_sample_id):
        hb, hb_next = hb_next, draw()
        if a.span_documents:
            from distca_b200.runtime.trainer import make_span_batch
            hb = make_span_batch(np.random.default_rng(a.seed * 100003 + it), par.dp, a.num_tokens * a.num_batches,
                                 cfg.vocab, max_doc_len=max_len)
        elif hasattr(trainer, "prefetch_plan") and not percp:
            trainer.prefetch_plan(hb_next)   # core attention of step it+1 is planned while step it runs
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        calls = None
        if it == a.trace_calls_step:
            from distca_b200.utils.profiler import TraceFunctions
            os.makedirs(a.output_dir or ".", exist_ok=True)
            calls = TraceFunctions(out=open(os.path.join(a.output_dir or ".", f"calls.rank{rank}.log"), "w"))
            calls.__enter__()
        try:
            with nvtx_range(f"sample_{it}"), ProfilerCtx(a.output_dir, rank, enabled=(it == a.torch_profile_step)):
                loss = trainer.train_step(hb)
        finally:
            if calls is not None:
                calls.__exit__(None, None, None)
                calls.out.close()
        guards.check(it, loss, float(trainer.opt.last_grad_norm) if trainer.opt.last_grad_norm is not None else None)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        rec = {"step": it, "loss": loss, "step_ms": ms, "tokens_per_s": tokens_per_step / (ms / 1e3),
               "grad_norm": float(trainer.opt.last_grad_norm) if trainer.opt.last_grad_norm is not None else None}
        cad_rt = getattr(trainer, "cad", None)
        if cad_rt is not None:
            rec["attn_imbalance"] = cad_rt.plan_stats.get("imbalance_after")
            rec["attn_time_imbalance_measured"] = cad_rt.plan_stats.get("attention_time_imbalance")
            ph = timers.GLOBAL.summary(reset=not a.phase_timers) if timers.GLOBAL.enabled else {}
            rec["exposed_dispatch_ms"] = (sum(v for k, v in ph.items() if k.removeprefix("re_").startswith("cad_wait") or
                                              k.removeprefix("re_") in ("cad_dispatch", "cad_return")) if ph else None)
            if getattr(cad_rt, "wait_report_ms", None) is not None:
                rec["blocking_waits"] = [e for e in cad_rt.blocking_events if e["step"] == cad_rt._steps_seen]
            if cad_rt.last_plan is not None:
                art.plan({"step": it, **inspect_plan(cad_rt.last_plan, cad_rt.W)})
        if a.phase_timers:
            rec["phases_ms"] = timers.GLOBAL.summary()
        art.step(rec)
        sink.log(rec)
        mem.log(f"step_{it}")
        if mem_hist is not None and it == start_it + 1:
            log.info("allocator history written to %s", mem_hist.dump())
        log.info("step %d loss %.4f %.1f ms %.0f tok/s%s", it, loss, ms, rec["tokens_per_s"],
                 f" imbalance {rec['attn_imbalance']:.3f}" if rec.get("attn_imbalance") else "")
        if a.val_every_n_steps and (it + 1) % a.val_every_n_steps == 0 and not percp:
            log.info("step %d validation loss %.4f", it, trainer.eval_step(hb_next))
        if save_dir and save_every and (it + 1) % save_every == 0:
            d = save_checkpoint(save_dir, it + 1, trainer.model, trainer.opt, cfg, tp_rank=trainer.tp_rank,
                                tp_size=par.tp, pp_rank=trainer.pp_rank, pp_size=par.pp, dp_rank=trainer.dp_rank,
                                args=vars(a))
            log.info("saved checkpoint %s", d)
    trainer.check_device_status()
    summary = art.finish(warmup=1 if a.max_sample_id > 1 else 0)
    if rank == 0 and summary:
        log.info("summary %s", summary)
    sink.close()
    trainer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
