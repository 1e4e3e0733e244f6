"""Pipeline parallelism: a tick-synchronous 1F1B schedule whose idle slots serve attention.

Tick ``t`` has a forward slot and a backward slot on EVERY stage:

    forward  slot of stage p : micro-batch  t - p                  (real if 0 <= . < M, else dummy)
    backward slot of stage p : micro-batch  t - 2(pp-1) + p        (real if 0 <= . < M, else dummy)

so the last stage runs the backward of a micro-batch in the tick of its forward, gradients reach
stage p one tick per stage later, and there are ``M + 2(pp-1)`` ticks. With core-attention
disaggregation every dp x pp rank is an attention server in every slot: a stage whose slot is a
dummy owns no tokens there but still runs the attention tasks the planner gives it, layer by layer,
in lock-step with the stages that do real work. Each slot has its own CAD plan over all ranks
(forward slots: the documents each stage is running forward; backward slots likewise), which is
the reference's per-tick planning (distca/utils/test_util.py:481-556, 582-795) with its
dummy forward / dummy backward (distca/runtime/megatron/forward_backward_func.py:283-300, 365-380,
427-470). Activations and activation gradients travel between stages with NCCL point-to-point
(``batch_isend_irecv``), tensors of shape [tokens / tp, hidden].
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


class PipelineTrainer:
    def __init__(self, model_cfg: ModelConfig, par: ParallelConfig, train_cfg: TrainConfig, *, num_microbatch: int,
                 device=None, seed: int = 0):
        assert par.pp > 1 and model_cfg.num_layers % par.pp == 0
        assert num_microbatch >= 1
        self.model_cfg, self.par, self.cfg, self.M = model_cfg, par, train_cfg, num_microbatch
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        assert self.world == par.world
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.tp_rank, self.dp_rank, self.pp_rank = par.coords(self.rank)
        self.groups = build_groups(par, self.rank)
        tp = None
        if par.tp > 1:
            from .tensor_parallel import TensorParallel
            tp = TensorParallel(self.groups.tp_group, par.tp, self.tp_rank, self.device)
        per = model_cfg.num_layers // par.pp
        self.first, self.last = self.pp_rank == 0, self.pp_rank == par.pp - 1
        grad_dtype = {"bf16": None, "fp32": torch.float32}[train_cfg.grad_dtype]
        if num_microbatch > 1 and grad_dtype is None and self.device.type == "cuda":
            grad_dtype = torch.float32  # several micro-batches accumulate into the gradient buffer
        self.model = LlamaModel(model_cfg, self.device, tp=tp, layer_range=(self.pp_rank * per, (self.pp_rank + 1) * per),
                                first_stage=self.first, last_stage=self.last, grad_dtype=grad_dtype, seed=seed,
                                recompute=train_cfg.recompute, lm_head_chunk=train_cfg.lm_head_chunk,
                                pad_params_to=par.dp)
        self.local_attn = LocalCoreAttention(model_cfg, par.tp)
        self.cad = None
        if train_cfg.cad and par.dp * par.pp > 1 and self.device.type == "cuda":
            from .cad import CadRuntime
            self.cad = CadRuntime(model_cfg, par, train_cfg, self.groups, self.device,
                                  tolerance=float(train_cfg.extra.get("tolerance", 0.1)))
        elif train_cfg.cad and par.dp * par.pp > 1:
            from .cad_cpu import GlooCadRuntime
            self.cad = GlooCadRuntime(model_cfg, self.groups.attn_group, self.groups.attn_ranks, par.tp,
                                      tolerance=float(train_cfg.extra.get("tolerance", 0.1)), dtype=self.model.dtype)
        repl = tuple(n for n, _ in self.model.store.shapes if n.endswith("norm_weight") or n.endswith("layernorm.weight"))
        self.opt = ShardedAdam(self.model.store, train_cfg, dp_group=self.groups.dp_group if par.dp > 1 else None,
                               norm_group=self.groups.world_group, replicated_names=repl if par.tp > 1 else (),
                               tp_rank=self.tp_rank)
        self.prev = par.rank_of(self.tp_rank, self.dp_rank, self.pp_rank - 1) if not self.first else None
        self.next = par.rank_of(self.tp_rank, self.dp_rank, self.pp_rank + 1) if not self.last else None
        self.act_dtype = self.model.dtype
        self.step_idx = 0
        from ..utils.watchdog import StepGuard
        self.guard = StepGuard.for_process_group()     # heartbeat check before, watchdog around every step

    # ------------------------------------------------------------------------------------------
    def _exchange(self, send_next=None, send_prev=None, recv_prev_shape=None, recv_next_shape=None):
        ops, rp, rn = [], None, None
        if send_next is not None:
            ops.append(dist.P2POp(dist.isend, send_next.contiguous(), self.next))
        if send_prev is not None:
            ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), self.prev))
        if recv_prev_shape is not None:
            rp = torch.empty(recv_prev_shape, dtype=self.act_dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, rp, self.prev))
        if recv_next_shape is not None:
            rn = torch.empty(recv_next_shape, dtype=self.act_dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, rn, self.next))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return rp, rn

    def _slot_docs(self, all_mb_docs, which: str, tick: int):
        """Documents every rank of the attention group owns in a slot, in attention-group rank order
        (pp-major, dp-minor: the order build_groups uses)."""
        pp, dp = self.par.pp, self.par.dp
        out = []
        for p in range(pp):
            mb = tick - p if which == "fwd" else tick - 2 * (pp - 1) + p
            for d in range(dp):
                out.append(list(all_mb_docs[mb][d]) if 0 <= mb < self.M else [])
        return out

    def _set_attention(self, all_mb_docs, which, tick, mb):
        if self.cad is not None:
            self.cad.plan_step(self._slot_docs(all_mb_docs, which, tick))
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
        M, pp, p = self.M, self.par.pp, self.pp_rank
        self.model.store.zero_grad()
        T, all_mb_docs, batches = self._split_microbatches(hb)
        Tl = T // self.par.tp
        H = self.model_cfg.hidden
        saved = {}
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        x_in, dy_in = None, None
        n_layers = len(self.model.layers)
        for tick in range(M + 2 * (pp - 1)):
            f_mb = tick - p
            b_mb = tick - 2 * (pp - 1) + p
            # ---------------- forward slot ----------------
            ca = self._set_attention(all_mb_docs, "fwd", tick, f_mb)
            x_out = None
            if 0 <= f_mb < M:
                x_out, saved[f_mb] = self.model.stage_forward(batches[f_mb], ca, x_in,
                                                              keep_last=self.last and self.cad is None)
            elif self.cad is not None:
                for _ in range(n_layers):
                    self.cad.dummy_forward()
            # ---------------- backward slot ----------------
            ca = self._set_attention(all_mb_docs, "bwd", tick, b_mb)
            dx = None
            if 0 <= b_mb < M:
                loss, dx = self.model.stage_backward(batches[b_mb], ca, saved.pop(b_mb), dy_in)
                if loss is not None:
                    loss_sum += loss
            elif self.cad is not None:
                for li in range(n_layers):
                    if self.model.recompute == "keep_attn":
                        # the recompute half only re-dispatches Q/K/V (nothing to send from here), no attention runs
                        self.cad.no_tokens_dispatch()
                        self.cad.restore_no_tokens(li)
                    else:
                        self.cad.dummy_forward()    # the recompute half of a backward slot
                    self.cad.dummy_backward()
            # ---------------- hand activations / gradients to the neighbours ----------------
            nf, nb = f_mb + 1, b_mb + 1       # what this stage runs in the next tick
            x_in, dy_in = self._exchange(
                send_next=x_out if (x_out is not None and not self.last) else None,
                send_prev=dx if (dx is not None and not self.first) else None,
                recv_prev_shape=(Tl, H) if (not self.first and 0 <= nf < M) else None,
                recv_next_shape=(Tl, H) if (not self.last and 0 <= nb < M) else None)
        if self.par.tp > 1:
            self.model.tp.sync_replicated_grads(self.model.store)
        self.opt.step()
        # the loss lives on the last stage: share it with everybody (sum over dp, max trick over pp)
        dist.all_reduce(loss_sum, group=self.groups.world_group)
        loss_sum /= self.par.tp
        self.step_idx += 1
        value = float(loss_sum.item())
        if self.cad is not None and hasattr(self.cad, "end_of_step_feedback"):
            self.cad.end_of_step_feedback()
        self.check_device_status()      # raises when a kernel of this step reported a failed wait / bounds check
        return value

    def _split_microbatches(self, hb):
        M = self.M
        T = hb.ids.numel() // M
        self.model.ensure_positions(max(hb.doc_lens, default=0))
        all_mb_docs = [[[] for _ in range(self.par.dp)] for _ in range(M)]
        for d, docs in enumerate(hb.all_doc_lens):
            acc, mb = 0, 0
            for L in docs:
                all_mb_docs[mb][d].append(L)
                acc += L
                if acc == T:
                    acc, mb = 0, mb + 1
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
        try:
            for tick in range(M + pp - 1):
                f_mb = tick - p
                # the plan of a forward slot covers the micro-batches every stage runs in this tick
                ca = self._set_attention(all_mb_docs, "fwd", tick, f_mb)
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
                x_in, _ = self._exchange(send_next=x_out if (x_out is not None and not self.last) else None,
                                         recv_prev_shape=(Tl, H) if (not self.first and 0 <= nf < M) else None)
        finally:
            self.model.recompute = keep_policy
        dist.all_reduce(loss_sum, group=self.groups.world_group)
        loss_sum /= self.par.tp
        return float(loss_sum.item())

    def check_device_status(self) -> None:
        if self.device.type == "cuda":
            _lib.check_status(self.device, "pipeline step")

    def close(self) -> None:
        self.guard.close()
        if self.cad is not None:
            self.cad.close()
            self.cad = None
