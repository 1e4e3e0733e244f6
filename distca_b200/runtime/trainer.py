"""Training driver: builds the model, the core-attention runtime, the optimizer and the data
stream for one rank, and runs steps.

``Trainer.train_step`` is the public call: it takes the step's host batch (pinned CPU tensors),
copies it to the device, plans core attention, runs forward/backward, reduces gradients, updates
the weights and returns the loss as a Python float (a device-to-host read).

The reference's counterpart is ``MegatronE2eWorker.forward_backward_batch`` driven by the loop in
``pretrain_llama.py:709-863`` (which, unlike this driver, never steps the optimizer).
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from ..data.synthetic import SyntheticBatches
from ..models.config import ModelConfig, ParallelConfig, TrainConfig
from ..models.llama import Batch, LlamaModel, LocalCoreAttention
from ..ops import _lib
from ..ops.attention import AttnPlan, AttnTasks
from ..parallel.optimizer import ShardedAdam


@dataclass
class HostBatch:
    """One rank's share of a global batch, on the host.

    ``ids``/``labels``: int64 [T]; ``pos``: int32 [T]; ``doc_lens``: this rank's documents in order;
    ``all_doc_lens``: documents of every data-parallel rank (the CAD planner needs the whole picture);
    ``num_valid_global``: non-ignored labels in the global batch.
    """
    ids: torch.Tensor
    labels: torch.Tensor
    pos: torch.Tensor
    doc_lens: list[int]
    all_doc_lens: list[list[int]]
    num_valid_global: int

    def nbytes(self) -> int:
        return self.ids.numel() * 8 + self.labels.numel() * 8 + self.pos.numel() * 4


@dataclass
class SpanHostBatch:
    """A global batch whose documents are NOT pre-assigned to ranks: the planner lays them out over the
    ranks by sequential fill, so a document longer than one rank's share spans several ranks (each
    holding a head and a tail piece). Every rank holds the same object; its own tokens are cut out
    once the layout is known. ``tokens``: int64, all documents back to back."""
    doc_lens: list[int]
    tokens: torch.Tensor

    @property
    def num_valid_global(self) -> int:
        return int(self.tokens.numel()) - len(self.doc_lens)      # the last token of a document predicts nothing

    def materialise(self, layout, tokens_per_rank: int, pinned: bool = False):
        """ids / labels / positions of one rank from its layout segments (doc, a, b, row0)."""
        starts = np.concatenate([[0], np.cumsum(self.doc_lens)])
        ids = torch.zeros(tokens_per_rank, dtype=torch.int64)
        labels = torch.full((tokens_per_rank,), -100, dtype=torch.int64)
        pos = torch.zeros(tokens_per_rank, dtype=torch.int32)
        for doc, a, b, row0 in layout:
            doc, a, b, row0 = int(doc), int(a), int(b), int(row0)
            o, L = int(starts[doc]), self.doc_lens[doc]
            ids[row0:row0 + b - a] = self.tokens[o + a:o + b]
            nb = min(b, L - 1)                                     # labels exist up to the document's second-to-last token
            if nb > a:
                labels[row0:row0 + nb - a] = self.tokens[o + a + 1:o + nb + 1]
            pos[row0:row0 + b - a] = torch.arange(a, b, dtype=torch.int32)
        if pinned:
            ids, labels, pos = ids.pin_memory(), labels.pin_memory(), pos.pin_memory()
        return ids, labels, pos


def make_span_batch(rng: np.random.Generator, world: int, tokens_per_rank: int, vocab: int, max_doc_len: int,
                    min_doc_len: int = 128, multiple_of: int = 16) -> SpanHostBatch:
    """Synthetic global batch of ``world * tokens_per_rank`` tokens with log-uniform document lengths up
    to ``max_doc_len`` (which may exceed ``tokens_per_rank``)."""
    total, docs = world * tokens_per_rank, []
    while total > 0:
        L = int(np.exp(rng.uniform(np.log(min_doc_len), np.log(max_doc_len))))
        L = min(total, max(multiple_of, L // multiple_of * multiple_of))
        docs.append(L)
        total -= L
    toks = torch.from_numpy(rng.integers(0, vocab, size=world * tokens_per_rank, dtype=np.int64))
    return SpanHostBatch(docs, toks)


def nano_cut(docs: list[int]) -> int:
    """Number of leading documents of ``docs`` that form the first nano-batch: the document boundary closest
    to half the tokens (0 or ``len(docs)`` when one document holds more than half of them)."""
    total, best, run, k = sum(docs), None, 0, 0
    for i in range(len(docs) + 1):
        d = abs(2 * run - total)
        if best is None or d < best:
            best, k = d, i
        if i < len(docs):
            run += docs[i]
    return k


def split_nano(hb: HostBatch) -> list[HostBatch]:
    """Cut one rank's batch into two nano-batches at the document boundary closest to half its
    tokens (every rank applies the same rule to every rank's document list, so all agree on who owns
    what in each nano-batch). A nano-batch may be empty (one document filling the whole sequence)."""
    cut = nano_cut
    per_rank = [(d[:cut(d)], d[cut(d):]) for d in hb.all_doc_lens]
    k = cut(hb.doc_lens)
    t0 = sum(hb.doc_lens[:k])
    out = []
    for n, sl in enumerate((slice(0, t0), slice(t0, None))):
        out.append(HostBatch(hb.ids[sl], hb.labels[sl], hb.pos[sl], list(hb.doc_lens[:k] if n == 0 else hb.doc_lens[k:]),
                             [list(p[n]) for p in per_rank], hb.num_valid_global))
    return out


def init_distributed() -> tuple[int, int, int]:
    """(rank, world, local_rank) from the torchrun environment; single process when unset."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        # collective timeout in seconds (the reference's EXPERIMENT_TORCH_DIST_TIMEOUT, distca/utils/test_util.py:93-104):
        # a rank that never joins ends the others' next collective with an error instead of a silent hang
        import datetime
        kw = {}
        if os.environ.get("EXPERIMENT_TORCH_DIST_TIMEOUT"):
            kw["timeout"] = datetime.timedelta(seconds=float(os.environ["EXPERIMENT_TORCH_DIST_TIMEOUT"]))
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world,
                                    device_id=torch.device("cuda", local), **kw)
        else:
            dist.init_process_group("gloo", rank=rank, world_size=world, **kw)
    elif torch.cuda.is_available():
        torch.cuda.set_device(local)
    return rank, world, local


class Trainer:
    def __init__(self, model_cfg: ModelConfig, par: ParallelConfig, train_cfg: TrainConfig, *,
                 device=None, seed: int = 0):
        self.model_cfg, self.par, self.cfg = model_cfg, par, train_cfg
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        assert self.world == par.world, f"world {self.world} != tp*pp*dp {par.world}"
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.tp_rank, self.dp_rank, self.pp_rank = par.coords(self.rank)
        from ..parallel.groups import build_groups
        self.groups = build_groups(par, self.rank) if self.world > 1 else None
        tp = None
        if par.tp > 1:
            from ..parallel.tensor_parallel import TensorParallel
            # default on GPUs: all-gather / reduce-scatter fused into the GEMMs over peer memory
            # (--tp-transport nccl keeps the NCCL collectives); the arena is sized at the first step
            tp = TensorParallel(self.groups.tp_group, par.tp, self.tp_rank, self.device,
                                use_p2p=train_cfg.extra.get("tp_transport", "p2p") in ("p2p", "p2p-tile"),
                                tile_loads=train_cfg.extra.get("tp_transport", "p2p") == "p2p-tile",
                                max_rows_local=int(train_cfg.extra.get("tp_max_rows_local", 0)),
                                max_cols=max(model_cfg.hidden, 0))
        grad_dtype = {"bf16": None, "fp32": torch.float32}[train_cfg.grad_dtype]
        assert par.pp == 1, "pipeline stages are built by parallel.pipeline.PipelineTrainer"
        self.p2p = None
        buffers = None
        if (par.dp > 1 and self.device.type == "cuda"
                and train_cfg.extra.get("dp_transport", "p2p") == "p2p"):
            # parameters and gradients live in peer-mapped memory so that the gradient reduce-scatter
            # and the parameter all-gather run inside our own kernels over NVLink
            from ..parallel.dp_p2p import PeerDataParallel

            def buffers(numel):
                self.p2p = PeerDataParallel(self.groups.dp_group, self.device, numel,
                                            grad_dtype=grad_dtype or torch.bfloat16)
                return self.p2p.flat, self.p2p.grad
        self.model = LlamaModel(model_cfg, self.device, tp=tp, grad_dtype=grad_dtype, seed=seed,
                                recompute=train_cfg.recompute, lm_head_chunk=train_cfg.lm_head_chunk,
                                pad_params_to=par.dp, param_buffers=buffers)
        for layer in self.model.layers:
            layer.fuse_rope = bool(train_cfg.extra.get("fuse_qkv_rope", True))
        self.model.nano_streams = bool(train_cfg.extra.get("nano_streams", True))
        self.model.check_finite = bool(train_cfg.extra.get("check_finite", False))
        self.model.fuse_ticks = bool(train_cfg.extra.get("fuse_ticks", False))
        if self.groups is not None and self.device.type == "cuda":
            self.model.store_sync_group = self.groups.world_group
        self.core_attn = LocalCoreAttention(model_cfg, par.tp)
        self.cad = None
        if train_cfg.cad and par.dp * par.pp > 1 and self.device.type == "cuda":
            from ..parallel.cad import CadRuntime
            self.cad = CadRuntime(model_cfg, par, train_cfg, self.groups, self.device,
                                  tolerance=float(train_cfg.extra.get("tolerance", 0.1)))
            self.core_attn = self.cad
        elif train_cfg.cad and par.dp * par.pp > 1:
            from ..parallel.cad_cpu import GlooCadRuntime
            self.cad = GlooCadRuntime(model_cfg, self.groups.attn_group, self.groups.attn_ranks, par.tp,
                                      tolerance=float(train_cfg.extra.get("tolerance", 0.1)), dtype=self.model.dtype)
            self.core_attn = self.cad
        # baseline: per-document context parallelism over the same ranks, no disaggregation (all-gather K/V)
        self.percp = None
        if train_cfg.extra.get("baseline_mode", "none") in ("percp", "perseq") and par.dp * par.pp > 1:
            assert self.cad is None and par.pp == 1, "the context-parallel baselines replace CAD and have no pipeline stages"
            from ..parallel.percp import PerDocCPAttention
            seq_len = None
            if train_cfg.extra["baseline_mode"] == "perseq":       # per-sequence CP: chunks of packed sequences
                seq_len = int(train_cfg.extra["cp_seq_len"])
            self.percp = PerDocCPAttention(model_cfg, self.groups.attn_group, len(self.groups.attn_ranks),
                                           self.groups.attn_ranks.index(self.rank), self.device, par.tp, seq_len=seq_len)
            self.core_attn = self.percp
        # ping-pong: a second core-attention module (own arena, own plan) for the second nano-batch
        self.nano = int(train_cfg.extra.get("nano_batches", 1))
        assert self.nano in (1, 2)
        self.core_attns = [self.core_attn]
        if self.nano == 2:
            if self.cad is not None and self.device.type == "cuda":
                from ..parallel.cad import CadRuntime
                second = CadRuntime(model_cfg, par, train_cfg, self.groups, self.device,
                                    tolerance=float(train_cfg.extra.get("tolerance", 0.1)))
            elif self.cad is not None:
                from ..parallel.cad_cpu import GlooCadRuntime
                second = GlooCadRuntime(model_cfg, self.groups.attn_group, self.groups.attn_ranks, par.tp,
                                        tolerance=float(train_cfg.extra.get("tolerance", 0.1)), dtype=self.model.dtype)
            else:
                second = LocalCoreAttention(model_cfg, par.tp)
            self.core_attns.append(second)
        repl = tuple(n for n, _ in self.model.store.shapes if n.endswith("norm_weight") or n.endswith("layernorm.weight"))
        self.opt = ShardedAdam(self.model.store, train_cfg,
                               dp_group=self.groups.dp_group if self.groups and par.dp > 1 else None,
                               norm_group=self.groups.world_group if self.groups else None,
                               replicated_names=repl if par.tp > 1 else (), tp_rank=self.tp_rank, p2p=self.p2p)
        if self.opt.bucketed:
            self.model.grad_ready_hook = self.opt.bucket_ready
        self.step_idx = 0
        self.timers: dict[str, float] = {}
        from ..utils.watchdog import StepGuard
        self.guard = StepGuard.for_process_group()     # heartbeat check before, watchdog around every step
        self._plan_pool = None       # worker thread that plans the next step's core attention
        self._plan_ahead = None      # (document lists, Future of the plan)

    # ------------------------------------------------------------------------------------
    def to_device(self, hb: HostBatch) -> Batch:
        ids = hb.ids.to(self.device, non_blocking=True)
        labels = hb.labels.to(self.device, non_blocking=True)
        pos = hb.pos.to(self.device, non_blocking=True)
        return Batch(ids, labels, pos, hb.num_valid_global)

    def prefetch_plan(self, hb_next: HostBatch) -> None:
        """Start planning core attention for the NEXT step on a worker thread while the current step
        runs on the GPU (the C++ planner releases the GIL). ``train_step`` picks the plan up when it is
        given the same documents; otherwise it plans synchronously. The reference plans step N+1
        inside its data loader for the same reason (distca/planner/planner.py:411-507)."""
        if isinstance(hb_next, SpanHostBatch) or (self.cad is not None and not hasattr(self.cad, "make_tables")):
            return
        if self.cad is not None and any(ca.arena is None for ca in self.core_attns):
            return                   # the first plan sizes the arena: a collective, done in plan_step
        if self._plan_pool is None:
            from concurrent.futures import ThreadPoolExecutor
            self._plan_pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="cad-planner")
        if self.nano == 2:
            if self.cad is None:
                return
            # ping-pong: one plan per nano-batch, each for its own core-attention module
            docs2 = [[list(d) for d in n.all_doc_lens] for n in split_nano(hb_next)]

            def work2(cas=list(self.core_attns), docs2=docs2):
                out = []
                for ca, docs in zip(cas, docs2):
                    plan = ca.make_plan(docs)
                    out.append((plan, ca.make_tables(plan) if plan.fits else None))
                return out
            self._plan_ahead = (docs2, self._plan_pool.submit(work2))
            return
        if self.cad is None:
            # local attention: the work lists of the next step are built on the worker thread
            mine = list(hb_next.doc_lens)
            self._plan_ahead = (mine, self._plan_pool.submit(
                lambda: AttnPlan(AttnTasks.from_doc_lens(mine), self.device, upload=False)))
            return
        docs = [list(d) for d in hb_next.all_doc_lens]

        def work(cad=self.cad, docs=docs):
            plan = cad.make_plan(docs)
            return plan, (cad.make_tables(plan) if plan.fits else None)     # all host work of the next step
        self._plan_ahead = (docs, self._plan_pool.submit(work))

    def plan_attention(self, hb: HostBatch) -> None:
        if self.cad is not None:
            plan = tables = None
            if self._plan_ahead is not None:
                docs, fut = self._plan_ahead
                self._plan_ahead = None
                if docs == [list(d) for d in hb.all_doc_lens]:
                    plan, tables = fut.result()
            if plan is not None:
                self.cad.plan_step(hb.all_doc_lens, self.dp_rank, plan=plan, tables=tables)
            else:
                self.cad.plan_step(hb.all_doc_lens, self.dp_rank)
        else:
            plan = None
            if self._plan_ahead is not None:
                mine, fut = self._plan_ahead
                self._plan_ahead = None
                if mine == list(hb.doc_lens):
                    plan = fut.result()
                    plan.upload()
            if plan is None:
                plan = AttnPlan(AttnTasks.from_doc_lens(hb.doc_lens), self.device)
            self.core_attn.set_batch(plan)

    def plan_attention_nano(self, nano: list[HostBatch]) -> None:
        """One plan per nano-batch, each on its own core-attention module."""
        whole = max(sum(a) + sum(b) for a, b in zip(nano[0].all_doc_lens, nano[1].all_doc_lens))
        ahead = [None, None]
        if self._plan_ahead is not None:
            docs2, fut = self._plan_ahead
            self._plan_ahead = None
            if docs2 == [[list(d) for d in n.all_doc_lens] for n in nano]:
                ahead = fut.result()
        for k, (ca, hb) in enumerate(zip(self.core_attns, nano)):
            if self.cad is not None:
                if hasattr(ca, "capacity_hint"):
                    # a nano-batch can be as large as the whole sequence (one long document)
                    ca.capacity_hint = max(ca.capacity_hint, whole)
                if ahead[k] is not None:
                    ca.plan_step(hb.all_doc_lens, self.dp_rank, plan=ahead[k][0], tables=ahead[k][1])
                else:
                    ca.plan_step(hb.all_doc_lens, self.dp_rank)
            else:
                ca.set_batch(AttnPlan(AttnTasks.from_doc_lens(hb.doc_lens), self.device))

    def train_step(self, hb) -> float:
        """One optimizer step on ``hb`` (host tensors); returns the loss. Before anything is launched the
        peers' heartbeats are checked (a lost rank raises on the host), and the step runs under a watchdog."""
        self.guard.check()
        with self.guard.watch():
            return self._train_step(hb)

    def _train_step(self, hb) -> float:
        from ..utils import timers
        with timers.phase("zero_grad"):
            self.model.store.zero_grad()
            self.opt.begin_step()
        self.model.ensure_positions(max(hb.doc_lens, default=0))
        assert self.percp is None or isinstance(hb, SpanHostBatch), \
            "the per-document CP baseline takes the global batch (BatchSource.next_global)"
        if self.par.tp > 1 and not isinstance(hb, SpanHostBatch):
            self.model.tp.ensure_fused(hb.ids.numel() // self.par.tp)
        if isinstance(hb, SpanHostBatch) and self.percp is not None:
            # baseline: every rank holds a head and a tail chunk of every document of the global batch
            W = self.percp.W
            if self.par.tp > 1:
                self.model.tp.ensure_fused(int(hb.tokens.numel()) // W // self.par.tp)
            with timers.phase("plan"):
                ids, labels, pos = hb.materialise(self.percp.layout(hb.doc_lens),
                                                  int(hb.tokens.numel()) // W, pinned=self.device.type == "cuda")
                self.percp.set_batch(hb.doc_lens)
            batch = Batch(ids.to(self.device, non_blocking=True), labels.to(self.device, non_blocking=True),
                          pos.to(self.device, non_blocking=True), hb.num_valid_global)
            loss, _ = self.model.forward_backward(batch, self.core_attn)
            return self._finish_step(loss)
        if isinstance(hb, SpanHostBatch):
            # documents may span ranks: the planner decides the layout, then this rank cuts out its tokens
            assert self.cad is not None and self.nano == 1, "spanning documents need core-attention disaggregation"
            with timers.phase("plan"):
                plan = self.cad.make_plan_span([hb.doc_lens])
                rp = plan.rank(self.cad.me)
                ids, labels, pos = hb.materialise(rp.layout, int(rp.num_tokens), pinned=self.device.type == "cuda")
                self.cad.plan_step(None, self.dp_rank, plan=plan)
            batch = Batch(ids.to(self.device, non_blocking=True), labels.to(self.device, non_blocking=True),
                          pos.to(self.device, non_blocking=True), hb.num_valid_global)
            loss, _ = self.model.forward_backward(batch, self.core_attn)
            return self._finish_step(loss)
        if self.nano == 2:
            nano = split_nano(hb)
            batches = [self.to_device(n) if n.ids.numel() else None for n in nano]
            with timers.phase("plan"):
                self.plan_attention_nano(nano)
            loss, _ = self.model.forward_backward_nano(batches, self.core_attns)
            return self._finish_step(loss)
        batch = self.to_device(hb)
        with timers.phase("plan"):
            self.plan_attention(hb)
        loss, _ = self.model.forward_backward(batch, self.core_attn)
        return self._finish_step(loss)

    def _finish_step(self, loss) -> float:
        from ..utils import timers
        if self.par.tp > 1:
            self.model.tp.sync_replicated_grads(self.model.store)
        with timers.phase("optimizer"):
            self.opt.step()
        if self.groups is not None and self.par.dp > 1:
            dist.all_reduce(loss, group=self.groups.dp_group)
        self.step_idx += 1
        value = float(loss.item())
        for ca in self.core_attns:
            if hasattr(ca, "end_of_step_feedback"):
                ca.end_of_step_feedback()       # measured attention time of this step steers the next plans
        # the read above synchronised: a wait that ran out or a failed bounds check in this step raises here,
        # before the caller logs the loss, checkpoints or starts another step (the Adam kernels of such a
        # step have already skipped their update)
        self.check_device_status()
        return value

    def train_step_prepared(self, batch: Batch, hb: HostBatch) -> torch.Tensor:
        """Same step with the batch already on the device and the plan built; returns the loss as a
        device tensor (no host synchronisation). Used for device-only timing."""
        self.model.store.zero_grad()
        self.opt.begin_step()
        self.model.ensure_positions(max(hb.doc_lens, default=0))
        if self.par.tp > 1:
            self.model.tp.ensure_fused(hb.ids.numel() // self.par.tp)
        if self.nano == 2:
            loss, _ = self.model.forward_backward_nano(batch, self.core_attns)   # batch: list of nano-batches
        else:
            loss, _ = self.model.forward_backward(batch, self.core_attn)
        if self.par.tp > 1:
            self.model.tp.sync_replicated_grads(self.model.store)
        self.opt.step()
        self.step_idx += 1
        return loss

    def eval_step(self, hb: HostBatch) -> float:
        self.model.ensure_positions(max(hb.doc_lens, default=0))
        if self.par.tp > 1:
            self.model.tp.ensure_fused(hb.ids.numel() // self.par.tp)
        batch = self.to_device(hb)
        self.plan_attention(hb)
        loss = self.model.forward_loss(batch, self.core_attn)
        if self.groups is not None and self.par.dp > 1:
            dist.all_reduce(loss, group=self.groups.dp_group)
        return float(loss.item())

    def check_device_status(self) -> None:
        if self.device.type == "cuda":
            _lib.check_status(self.device, "training step")

    def close(self) -> None:
        """Release peer-mapped arenas (collective: every rank of the groups must call it)."""
        if self._plan_pool is not None:
            self._plan_pool.shutdown(wait=True)
            self._plan_pool = None
        self.guard.close()
        if self.cad is not None:
            for ca in self.core_attns:
                ca.close()
            self.cad = None
        if self.par.tp > 1 and getattr(self.model.tp, "fused", None) is not None:
            self.model.tp.fused.close()
            self.model.tp.fused = None
        if self.p2p is not None:
            self.model = None
            self.opt = None
            self.p2p.close()
            self.p2p = None


class BatchSource:
    """Turns the synthetic global batch into per-rank :class:`HostBatch` objects.

    Every rank draws the same global batch from the same seed (no broadcast needed) and keeps the
    pack with its data-parallel index; the reference has rank 0 sample and broadcast the
    document lengths instead (distca/utils/test_util.py:455-473).
    """

    def __init__(self, model_cfg: ModelConfig, par: ParallelConfig, tokens_per_seq: int, dist_name: str,
                 seed: int, seqs_per_rank: int = 1, pinned: bool = True, stream=None, shape: dict | None = None,
                 debug_packs: int = 0, packing: str = "sequential"):
        """``stream``: any object with ``next_doc_lens()`` / ``next_tokens(packs)`` (e.g.
        :class:`~distca_b200.data.text.TextBatches`); default: synthetic documents of ``dist_name``."""
        self.par = par
        self.stream = stream or SyntheticBatches(tokens_per_seq, par.dp * seqs_per_rank, dist_name, seed, model_cfg.vocab,
                                                 shape=shape, debug_packs=debug_packs, packing=packing)
        self.seqs_per_rank = seqs_per_rank
        self.pinned = pinned and torch.cuda.is_available()

    def next_global(self) -> SpanHostBatch:
        """The same global batch as :meth:`next`, whole, on every rank: all documents in order with all their
        tokens (layouts that cut every document over the ranks, e.g. the per-document CP baseline)."""
        packs = self.stream.next_doc_lens()
        ids, _labels, _pos = self.stream.next_tokens(packs)
        return SpanHostBatch([L for p in packs for L in p], ids.reshape(-1).clone())

    def next(self, dp_rank: int) -> HostBatch:
        packs = self.stream.next_doc_lens()
        ids, labels, pos = self.stream.next_tokens(packs)
        n_valid = int((labels >= 0).sum())
        s = self.seqs_per_rank
        sl = slice(dp_rank * s, (dp_rank + 1) * s)
        my_ids, my_labels, my_pos = ids[sl].reshape(-1), labels[sl].reshape(-1), pos[sl].reshape(-1)
        if self.pinned:
            my_ids, my_labels, my_pos = my_ids.pin_memory(), my_labels.pin_memory(), my_pos.pin_memory()
        per_rank = [sum(packs[r * s:(r + 1) * s], []) for r in range(self.par.dp)]
        return HostBatch(my_ids, my_labels, my_pos, per_rank[dp_rank], per_rank, n_valid)
