"""Pipeline parallelism: a tick-synchronous 1F1B schedule whose idle slots serve attention.

Stage ``p`` of ``pp`` runs the forward of micro-batch ``f - p`` in forward slot ``f`` and the backward of
micro-batch ``b - (pp - 1 - p)`` in backward slot ``b`` (real if that index is in ``[0, M)``, else a dummy).
There are ``M + pp - 1`` forward slots and as many backward slots, laid out as the reference does
(distca/runtime/megatron/forward_backward_func.py:217-223, 279-300, 365-470):

    warm-up    pp - 1 ticks   forward slot only      (slots f = 0 .. pp-2)
    steady     M ticks        forward + backward     (f = pp-1+i, b = i)
    cool-down  pp - 1 ticks   backward slot only     (b = M .. M+pp-2)

so the last stage runs the backward of a micro-batch in the tick of its forward, and a gradient reaches
stage p one tick per stage later. With core-attention disaggregation every dp x pp rank is an attention
server in every slot: a stage whose slot is a dummy owns no tokens there but still runs the attention tasks
the planner gives it, layer by layer, in lock-step with the stages that do real work. Each slot has its own
CAD plan over all ranks (the reference's per-tick planning, distca/utils/test_util.py:481-556, 582-795);
all plans of a step (and of the next step, :meth:`PipelineTrainer.prefetch_plan`) are built on a planning
thread while the GPU works.

Activations and activation gradients travel between stages with NCCL point-to-point, tensors of shape
[tokens / tp, hidden]: the exchange of a slot is started as soon as the slot's kernels are queued and is
waited for only where the received tensor is consumed (the next tick), so the transfer overlaps the other
slot's compute.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import ModelConfig, ParallelConfig, TrainConfig
from ..models.llama import Batch, LlamaModel, LocalCoreAttention
from ..ops import _lib
from ..ops.attention import AttnPlan, AttnTasks
from .groups import build_groups
from .optimizer import ShardedAdam


def slot_schedule(M: int, pp: int) -> list[tuple[int | None, int | None]]:
    """``(forward slot index or None, backward slot index or None)`` of every tick of a step:
    ``pp - 1`` forward-only ticks, ``M`` ticks with both slots, ``pp - 1`` backward-only ticks."""
    ticks = []
    for t in range(M + 2 * (pp - 1)):
        f = t if t < M + pp - 1 else None
        b = t - (pp - 1) if t >= pp - 1 else None
        ticks.append((f, b))
    return ticks


class PipelineTrainer:
    def __init__(self, model_cfg: ModelConfig, par: ParallelConfig, train_cfg: TrainConfig, *, num_microbatch: int,
                 device=None, seed: int = 0):
        assert par.pp > 1 and model_cfg.num_layers % par.pp == 0
        assert num_microbatch >= 1
        # tied input / output embeddings live on different stages: their values and gradients would have to be
        # kept equal across the first and the last stage, which this engine does not do
        assert not model_cfg.tie_embeddings, "tie_embeddings is not supported with pipeline stages"
        self.model_cfg, self.par, self.cfg, self.M = model_cfg, par, train_cfg, num_microbatch
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        assert self.world == par.world
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        on_gpu = self.device.type == "cuda"
        self.tp_rank, self.dp_rank, self.pp_rank = par.coords(self.rank)
        self.groups = build_groups(par, self.rank)
        tp = None
        if par.tp > 1:
            from .tensor_parallel import TensorParallel
            # default on GPUs: all-gather / reduce-scatter fused into the GEMMs over peer memory
            tp = TensorParallel(self.groups.tp_group, par.tp, self.tp_rank, self.device,
                                use_p2p=train_cfg.extra.get("tp_transport", "p2p") in ("p2p", "p2p-tile"),
                                tile_loads=train_cfg.extra.get("tp_transport", "p2p") == "p2p-tile",
                                max_cols=model_cfg.hidden)
        per = model_cfg.num_layers // par.pp
        self.first, self.last = self.pp_rank == 0, self.pp_rank == par.pp - 1
        grad_dtype = {"bf16": None, "fp32": torch.float32}[train_cfg.grad_dtype]
        if num_microbatch > 1 and grad_dtype is None and on_gpu:
            grad_dtype = torch.float32  # several micro-batches accumulate into the gradient buffer
        self.p2p = None
        buffers = None
        if par.dp > 1 and on_gpu and train_cfg.extra.get("dp_transport", "p2p") == "p2p":
            # parameters and gradients in peer-mapped memory: reduce-scatter and parameter all-gather run in
            # this repository's kernels over NVLink (fp32 gradients when micro-batches accumulate)
            from .dp_p2p import PeerDataParallel

            def buffers(numel):
                self.p2p = PeerDataParallel(self.groups.dp_group, self.device, numel,
                                            grad_dtype=grad_dtype or torch.bfloat16)
                return self.p2p.flat, self.p2p.grad
        self.model = LlamaModel(model_cfg, self.device, tp=tp, layer_range=(self.pp_rank * per, (self.pp_rank + 1) * per),
                                first_stage=self.first, last_stage=self.last, grad_dtype=grad_dtype, seed=seed,
                                recompute=train_cfg.recompute, lm_head_chunk=train_cfg.lm_head_chunk,
                                pad_params_to=par.dp, param_buffers=buffers)
        for layer in self.model.layers:
            layer.fuse_rope = bool(train_cfg.extra.get("fuse_qkv_rope", True))
        self.model.fuse_ticks = bool(train_cfg.extra.get("fuse_ticks", False))
        self.local_attn = LocalCoreAttention(model_cfg, par.tp)
        self.cad = None
        if train_cfg.cad and par.dp * par.pp > 1 and on_gpu:
            from .cad import CadRuntime
            self.cad = CadRuntime(model_cfg, par, train_cfg, self.groups, self.device,
                                  tolerance=float(train_cfg.extra.get("tolerance", 0.1)))
        elif train_cfg.cad and par.dp * par.pp > 1:
            from .cad_cpu import GlooCadRuntime
            self.cad = GlooCadRuntime(model_cfg, self.groups.attn_group, self.groups.attn_ranks, par.tp,
                                      tolerance=float(train_cfg.extra.get("tolerance", 0.1)), dtype=self.model.dtype)
        # ping-pong inside the stages: every micro-batch is cut into two nano-batches, each with its own
        # core-attention runtime (own arena, signals and per-slot plans), interleaved layer by layer
        self.nano = int(train_cfg.extra.get("nano_batches", 1))
        assert self.nano in (1, 2)
        assert self.nano == 1 or self.cad is not None, "nano-batches in pipeline stages need core-attention disaggregation"
        self.cads = [self.cad] if self.cad is not None else []
        if self.nano == 2:
            if on_gpu:
                from .cad import CadRuntime
                self.cads.append(CadRuntime(model_cfg, par, train_cfg, self.groups, self.device,
                                            tolerance=float(train_cfg.extra.get("tolerance", 0.1))))
            else:
                from .cad_cpu import GlooCadRuntime
                self.cads.append(GlooCadRuntime(model_cfg, self.groups.attn_group, self.groups.attn_ranks, par.tp,
                                                tolerance=float(train_cfg.extra.get("tolerance", 0.1)),
                                                dtype=self.model.dtype))
        repl = tuple(n for n, _ in self.model.store.shapes if n.endswith("norm_weight") or n.endswith("layernorm.weight"))
        self.opt = ShardedAdam(self.model.store, train_cfg, dp_group=self.groups.dp_group if par.dp > 1 else None,
                               norm_group=self.groups.world_group, replicated_names=repl if par.tp > 1 else (),
                               tp_rank=self.tp_rank, p2p=self.p2p)
        if self.opt.bucketed:
            self.model.grad_ready_hook = self.opt.bucket_ready
        self.prev = par.rank_of(self.tp_rank, self.dp_rank, self.pp_rank - 1) if not self.first else None
        self.next = par.rank_of(self.tp_rank, self.dp_rank, self.pp_rank + 1) if not self.last else None
        self.act_dtype = self.model.dtype
        self.step_idx = 0
        from ..utils.watchdog import StepGuard
        self.guard = StepGuard.for_process_group()     # heartbeat check before, watchdog around every step
        self._plan_pool = None
        self._plans_ahead = None         # (document table of the step, {(which, slot): Future})
        self.last_schedule = None        # what the last step ran: ticks, slots, bubble fraction

    # ------------------------------------------------------------------------------------------
    # stage-to-stage exchange: started when the slot's kernels are queued, waited for where consumed
    def _start_exchange(self, send: torch.Tensor | None, send_to, recv_shape, recv_from):
        ops, recv = [], None
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), send_to))
        if recv_shape is not None:
            recv = torch.empty(recv_shape, dtype=self.act_dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, recv, recv_from))
        works = dist.batch_isend_irecv(ops) if ops else []
        return works, recv, send      # the sent tensor is kept alive until the exchange was waited for

    @staticmethod
    def _finish_exchange(pending):
        if pending is None:
            return None
        works, recv, _sent = pending
        for w in works:
            w.wait()
        return recv

    # ------------------------------------------------------------------------------------------
    # per-slot core-attention plans
    def _slot_docs(self, all_mb_docs, which: str, slot: int):
        """Documents every rank of the attention group owns in a slot, in attention-group rank order
        (pp-major, dp-minor: the order build_groups uses)."""
        pp, dp, M = self.par.pp, self.par.dp, len(all_mb_docs)
        out = []
        for p in range(pp):
            mb = slot - p if which == "fwd" else slot - (pp - 1 - p)
            for d in range(dp):
                out.append(list(all_mb_docs[mb][d]) if 0 <= mb < M else [])
        return out

    def _submit_plans(self, all_mb_docs) -> dict:
        """Queue the host work (C++ plan + address tables) of every slot of a step on the planning thread, in
        the order the slots run. The first plan of a run sizes the arena, which is a collective: it is made
        by the caller, synchronously, before this is used."""
        if self._plan_pool is None:
            from concurrent.futures import ThreadPoolExecutor
            self._plan_pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="cad-planner")
        futs = {}

        def work(docs, cad):
            plan = cad.make_plan(docs)
            return plan, (cad.make_tables(plan) if plan.fits else None)
        per_nano = self._nano_docs(all_mb_docs)
        for f, b in slot_schedule(len(all_mb_docs), self.par.pp):
            for which, slot in (("fwd", f), ("bwd", b)):
                if slot is not None:
                    for k, cad in enumerate(self.cads):
                        futs[(which, slot, k)] = self._plan_pool.submit(work, self._slot_docs(per_nano[k], which, slot), cad)
        return futs

    def _arenas_ready(self) -> bool:
        """Sizing an arena is a collective: plans are only made on the planning thread once every runtime has one."""
        return all(getattr(c, "arena", None) is not None for c in self.cads)

    def _nano_docs(self, all_mb_docs):
        """``[nano-batch][micro-batch][dp rank]`` document lists: with two nano-batches every rank's documents of
        a micro-batch are cut at the document boundary nearest to half its tokens (the rule of
        ``runtime.trainer.nano_cut``, applied by every rank to every rank's list, so all agree)."""
        if self.nano == 1:
            return [all_mb_docs]
        from ..runtime.trainer import nano_cut
        halves = ([], [])
        for mb in all_mb_docs:
            cuts = [nano_cut(d) for d in mb]
            halves[0].append([list(d[:c]) for d, c in zip(mb, cuts)])
            halves[1].append([list(d[c:]) for d, c in zip(mb, cuts)])
        return list(halves)

    def prefetch_plan(self, hb_next) -> None:
        """Plan every slot of the NEXT step on the planning thread while the current step runs."""
        if self.cad is None or not hasattr(self.cad, "make_tables") or not self._arenas_ready():
            return
        _, all_mb_docs = self._microbatch_docs(hb_next)
        self._plans_ahead = (all_mb_docs, self._submit_plans(all_mb_docs))

    def _set_attention(self, all_mb_docs, plans, which, slot, mb):
        if self.cad is not None:
            per_nano = self._nano_docs(all_mb_docs)
            for k, cad in enumerate(self.cads):
                docs = self._slot_docs(per_nano[k], which, slot)
                fut = plans.get((which, slot, k)) if plans else None
                if fut is not None:
                    plan, tables = fut.result()
                    cad.plan_step(docs, plan=plan, tables=tables)
                else:
                    cad.plan_step(docs)
            return self.cad
        if 0 <= mb < self.M:
            self.local_attn.set_batch(AttnPlan(AttnTasks.from_doc_lens(all_mb_docs[mb][self.dp_rank]), self.device))
        return self.local_attn

    # ------------------------------------------------------------------------------------------
    def train_step(self, hb) -> float:
        """``hb``: HostBatch whose tensors hold ``M`` micro-batches of equal length back to back;
        ``hb.all_doc_lens[d]`` lists rank d's documents of all micro-batches in order. A lost peer raises on
        the host before anything is launched; the step runs under the watchdog."""
        self.guard.check()
        with self.guard.watch("pipeline step"):
            return self._train_step(hb)

    def _train_step(self, hb) -> float:
        from ..utils import timers
        from ..utils.observability import nvtx_range
        M, pp, p = self.M, self.par.pp, self.pp_rank
        self.model.store.zero_grad()
        self.opt.begin_step()
        T, all_mb_docs, batches = self._split_microbatches(hb)
        if self.par.tp > 1:
            self.model.tp.ensure_fused(T // self.par.tp)
        Tl = T // self.par.tp
        H = self.model_cfg.hidden
        nano_batches = self._split_nano_batches(all_mb_docs, batches) if self.nano == 2 else None
        if self.nano == 2:
            for cad in self.cads:
                if hasattr(cad, "capacity_hint"):
                    cad.capacity_hint = max(cad.capacity_hint, T)     # a nano-batch can be the whole micro-batch
        plans = None
        if self.cad is not None and hasattr(self.cad, "make_tables"):
            if self._plans_ahead is not None and self._plans_ahead[0] == all_mb_docs:
                plans = self._plans_ahead[1]
            elif self._arenas_ready():
                plans = self._submit_plans(all_mb_docs)
            self._plans_ahead = None
        saved = {}
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        n_layers = len(self.model.layers)
        pend_x = pend_dy = None           # exchanges in flight: next forward input / next backward gradient
        ticks = slot_schedule(M, pp)
        real = 0
        for tick, (f, b) in enumerate(ticks):
            # ---------------- forward slot ----------------
            if f is not None:
                f_mb = f - p
                with nvtx_range(f"tick{tick}.fwd.mb{f_mb if 0 <= f_mb < M else 'dummy'}"):
                    x_in = self._finish_exchange(pend_x)
                    pend_x = None
                    ca = self._set_attention(all_mb_docs, plans, "fwd", f, f_mb)
                    if plans is None and self.cad is not None and hasattr(self.cad, "make_tables") and tick == 0:
                        plans = self._submit_plans(all_mb_docs)      # the arena exists now: plan the rest ahead
                        for k in range(len(self.cads)):
                            plans.pop(("fwd", f, k), None)
                    x_out = None
                    if 0 <= f_mb < M and self.nano == 2:
                        real += 1
                        nb, rows = nano_batches[f_mb]
                        x_outs, saved[f_mb] = self.model.stage_forward_nano(nb, self.cads, self._split_rows(x_in, rows))
                        x_out = self._join_rows(x_outs) if not self.last else None
                    elif 0 <= f_mb < M:
                        real += 1
                        x_out, saved[f_mb] = self.model.stage_forward(batches[f_mb], ca, x_in,
                                                                      keep_last=self.last and self.cad is None)
                    elif self.cad is not None:
                        for _ in range(n_layers):
                            for cad in self.cads:
                                cad.dummy_forward()
                    nf = f_mb + 1          # what this stage runs in its next forward slot
                    more = f + 1 < M + pp - 1
                    pend_x = self._start_exchange(
                        x_out if (x_out is not None and not self.last) else None, self.next,
                        (Tl, H) if (more and not self.first and 0 <= nf < M) else None, self.prev)
            # ---------------- backward slot ----------------
            if b is not None:
                b_mb = b - (pp - 1 - p)
                with nvtx_range(f"tick{tick}.bwd.mb{b_mb if 0 <= b_mb < M else 'dummy'}"):
                    dy_in = self._finish_exchange(pend_dy)
                    pend_dy = None
                    ca = self._set_attention(all_mb_docs, plans, "bwd", b, b_mb)
                    dx = None
                    if 0 <= b_mb < M and self.nano == 2:
                        real += 1
                        nb, rows = nano_batches[b_mb]
                        loss, dxs = self.model.stage_backward_nano(nb, self.cads, saved.pop(b_mb),
                                                                   self._split_rows(dy_in, rows), grads_final=(b_mb == M - 1))
                        dx = self._join_rows(dxs) if dxs is not None else None
                        if loss is not None:
                            loss_sum += loss
                    elif 0 <= b_mb < M:
                        real += 1
                        loss, dx = self.model.stage_backward(batches[b_mb], ca, saved.pop(b_mb), dy_in,
                                                             grads_final=(b_mb == M - 1))
                        if loss is not None:
                            loss_sum += loss
                    elif self.cad is not None:
                        for li in range(n_layers):
                            # same order of calls per runtime as a stage that runs a real micro-batch
                            for cad in self.cads:
                                if self.model.recompute == "keep_attn":
                                    # the recompute half only re-dispatches Q/K/V (nothing to send from here), no attention runs
                                    cad.no_tokens_dispatch()
                                    cad.restore_no_tokens(li)
                                else:
                                    cad.dummy_forward()    # the recompute half of a backward slot
                            for cad in self.cads:
                                cad.dummy_backward()
                    nb = b_mb + 1
                    more = b + 1 < M + pp - 1
                    pend_dy = self._start_exchange(
                        dx if (dx is not None and not self.first) else None, self.prev,
                        (Tl, H) if (more and not self.last and 0 <= nb < M) else None, self.next)
        self._finish_exchange(pend_x)
        self._finish_exchange(pend_dy)
        slots = 2 * (M + pp - 1)
        self.last_schedule = {"ticks": len(ticks), "forward_slots": M + pp - 1, "backward_slots": M + pp - 1,
                              "real_slots_this_stage": real, "bubble_fraction": 1.0 - real / slots}
        if self.par.tp > 1:
            self.model.tp.sync_replicated_grads(self.model.store)
        with timers.phase("optimizer"):
            self.opt.step()
        # the loss lives on the last stage: share it with everybody (sum over dp, max trick over pp)
        dist.all_reduce(loss_sum, group=self.groups.world_group)
        loss_sum /= self.par.tp
        self.step_idx += 1
        value = float(loss_sum.item())
        for cad in self.cads:
            if hasattr(cad, "end_of_step_feedback"):
                cad.end_of_step_feedback()
        self.check_device_status()      # raises when a kernel of this step reported a failed wait / bounds check
        return value

    def _split_nano_batches(self, all_mb_docs, batches):
        """Per micro-batch: ([Batch or None per nano-batch], [sequence-parallel rows per nano-batch]) of THIS rank."""
        from ..runtime.trainer import nano_cut
        out = []
        for mb, b in zip(all_mb_docs, batches):
            docs = mb[self.dp_rank]
            t0 = sum(docs[:nano_cut(docs)])
            T = int(b.ids.numel())
            assert t0 % self.par.tp == 0 and (T - t0) % self.par.tp == 0, "nano-batch rows must divide by the tensor-parallel size"
            parts = []
            for lo, hi in ((0, t0), (t0, T)):
                parts.append(Batch(b.ids[lo:hi], b.labels[lo:hi], b.pos[lo:hi], b.num_valid_global) if hi > lo else None)
            out.append((parts, [t0 // self.par.tp, (T - t0) // self.par.tp]))
        return out

    @staticmethod
    def _split_rows(x, rows):
        """The stage input (or gradient) of a micro-batch as one tensor per nano-batch (``None`` where empty)."""
        if x is None:
            return [None] * len(rows)
        out, lo = [], 0
        for r in rows:
            out.append(x[lo:lo + r] if r else None)
            lo += r
        return out

    @staticmethod
    def _join_rows(parts):
        parts = [t for t in parts if t is not None]
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)

    def _microbatch_docs(self, hb):
        """(tokens per micro-batch, documents [micro-batch][dp rank]) of a host batch."""
        M = self.M
        T = hb.ids.numel() // M
        all_mb_docs = [[[] for _ in range(self.par.dp)] for _ in range(M)]
        for d, docs in enumerate(hb.all_doc_lens):
            acc, mb = 0, 0
            for L in docs:
                all_mb_docs[mb][d].append(L)
                acc += L
                if acc == T:
                    acc, mb = 0, mb + 1
        return T, all_mb_docs

    def _split_microbatches(self, hb):
        self.model.ensure_positions(max(hb.doc_lens, default=0))
        T, all_mb_docs = self._microbatch_docs(hb)
        M = self.M
        ids, labels, pos = (t.to(self.device, non_blocking=True) for t in (hb.ids, hb.labels, hb.pos))
        batches = [Batch(ids[i * T:(i + 1) * T], labels[i * T:(i + 1) * T], pos[i * T:(i + 1) * T], hb.num_valid_global)
                   for i in range(M)]
        return T, all_mb_docs, batches

    def eval_step(self, hb) -> float:
        """Forward-only pipeline pass (no gradients, no update): M + pp - 1 ticks of forward slots; idle
        stages still serve attention. Returns the loss of the global batch on every rank."""
        M, pp, p = self.M, self.par.pp, self.pp_rank
        T, all_mb_docs, batches = self._split_microbatches(hb)
        Tl, H = T // self.par.tp, self.model_cfg.hidden
        n_layers = len(self.model.layers)
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        x_in = None
        keep_policy, self.model.recompute = self.model.recompute, "full"     # nothing is kept for a backward
        keep_nano, keep_cads = self.nano, self.cads
        self.nano, self.cads = 1, self.cads[:1]                              # evaluation runs whole micro-batches
        try:
            for tick in range(M + pp - 1):
                f_mb = tick - p
                # the plan of a forward slot covers the micro-batches every stage runs in this tick
                ca = self._set_attention(all_mb_docs, None, "fwd", tick, f_mb)
                x_out = None
                if 0 <= f_mb < M:
                    x_out, _ = self.model.stage_forward(batches[f_mb], ca, x_in)
                    if self.last:
                        loss, _ = self.model.head_loss_and_grad(x_out, batches[f_mb].labels,
                                                                batches[f_mb].num_valid_global, need_grad=False)
                        loss_sum += loss
                elif self.cad is not None:
                    for _ in range(n_layers):
                        self.cad.dummy_forward()
                nf = f_mb + 1
                x_in = self._finish_exchange(self._start_exchange(
                    x_out if (x_out is not None and not self.last) else None, self.next,
                    (Tl, H) if (not self.first and 0 <= nf < M) else None, self.prev))
        finally:
            self.model.recompute = keep_policy
            self.nano, self.cads = keep_nano, keep_cads
        dist.all_reduce(loss_sum, group=self.groups.world_group)
        loss_sum /= self.par.tp
        return float(loss_sum.item())

    def check_device_status(self) -> None:
        if self.device.type == "cuda":
            _lib.check_status(self.device, "pipeline step")

    def close(self) -> None:
        """Release peer-mapped arenas (collective: every rank of the groups must call it)."""
        if self._plan_pool is not None:
            self._plan_pool.shutdown(wait=True)
            self._plan_pool = None
        self.guard.close()
        for cad in self.cads:
            cad.close()
        self.cads, self.cad = [], None
        if self.par.tp > 1 and getattr(self.model.tp, "fused", None) is not None:
            self.model.tp.fused.close()
            self.model.tp.fused = None
        if self.p2p is not None:
            self.model = None
            self.opt = None
            self.p2p.close()
            self.p2p = None
