"""Core-attention disaggregation runtime: the ``core_attn`` object a model uses when its attention
runs on attention servers instead of on the rank that owns the tokens.

Per layer and direction the data path is

  forward   owner : RoPE kernel rotates Q/K and stores Q, K, V rows straight into the servers'
                    arenas (K/V rows fan out to every server that holds a later shard of the
                    document)                                   -> signal "qkv"
            server: wait "qkv"; tcgen05 attention over its task list, O rows stored straight into
                    the owners' arenas, log-sum-exp kept locally   -> signal "out"
            owner : wait "out"; out-projection reads O from its arena
  backward  owner : delta = rowsum(dO o O); dO and delta rows stored into the servers' arenas
                                                                -> signal "dout"
            server: wait "dout"; tcgen05 attention backward on the still-resident Q/K/V;
                    dQ rows and per-copy dK/dV rows stored into the owners' arenas -> signal "dqkv"
            owner : wait "dqkv"; sum of the dK/dV copies; RoPE backward; QKV dgrad/wgrad

All stores are plain peer stores over NVLink from inside the kernels; signals are monotonic
counters with bounded waits (:mod:`distca_b200.parallel.p2p`). Because every rank signals every
rank in each phase, "I have my results back" implies "every server has finished reading its
inputs", so arena regions are reused layer after layer without a credit protocol.

A rank may own no tokens in a slot (a pipeline stage in a bubble): it then calls
``dummy_forward`` / ``dummy_backward`` once per layer and only serves attention, which is how
pipeline bubbles are filled with other ranks' attention work (the reference's dummy forward /
backward, distca/runtime/megatron/forward_backward_func.py:283-300, 365-380, 427-470).

A server keeps nothing of a layer beyond the Q/K/V rows in its arena, and those only from the
dispatch that precedes the call: the log-sum-exp rows go home with the output rows, and the backward
ships dO plus 12 bytes per head (delta, log-sum-exp) after the recompute pass has dispatched Q/K/V
again, instead of the reference's (dO | O | LSE | Q), K, V resend
(distca/runtime/megatron/ops/fused_comm_attn.py:407-461). Forward and backward of a micro-batch may
therefore run under different plans (different pipeline ticks); this needs a recompute policy that
re-runs the QKV projection in backward (``full`` or ``keep_attn``).

Reference counterparts: dispatch/all-to-all/unpack autograd ops (distca/runtime/dispatch_fn.py:29-216),
``FusedCommAttn`` (distca/runtime/megatron/ops/fused_comm_attn.py:282-461).
"""
from __future__ import annotations

import os

import numpy as np
import torch

from ..models.config import ModelConfig, ParallelConfig, TrainConfig
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..planner import Planner, PlannerConfig, default_cost_model
from ..utils import timers
from .p2p import PeerArena, SignalBoard, scatter_rows, sum_slots

SIG_QKV, SIG_OUT, SIG_DOUT, SIG_DQKV = 0, 1, 2, 3


class CadRuntime:
    def __init__(self, model_cfg: ModelConfig, par: ParallelConfig, train_cfg: TrainConfig, groups, device,
                 tolerance: float = 0.1, group=None, group_ranks=None):
        assert train_cfg.recompute in ("full", "keep_attn"), \
            "CAD keeps server state only across recompute+backward of one layer"
        self.cfg, self.par, self.tcfg = model_cfg, par, train_cfg
        self.device = torch.device(device)
        self.group = group if group_ranks is not None else groups.attn_group
        ranks = group_ranks if group_ranks is not None else groups.attn_ranks
        self.W = len(ranks)
        self.me = ranks.index(groups.rank)
        tp = par.tp
        self.hq, self.hkv, self.D = model_cfg.heads_q // tp, model_cfg.heads_kv // tp, model_cfg.head_dim
        self.qd, self.kd = self.hq * self.D, self.hkv * self.D
        self.qkvd = self.qd + 2 * self.kd
        self.q_bytes, self.kv_bytes = self.qd * 2, self.kd * 2
        self.tolerance = tolerance
        self.arena: PeerArena | None = None
        self.T = 0        # capacity: most tokens any rank owns in a slot
        self.Tcur = 0     # tokens this rank owns in the current slot
        self.scratch = attn_ops.BwdScratch()
        self.plan_stats: dict = {}
        self.last_plan = None
        self.capacity_hint = 0      # tokens per rank to size the arena for (nano-batches vary in size)
        # time-model balancing: the planner balances predicted milliseconds (tile-granular cost of this
        # repository's attention kernels) and gives every server a share in proportion to its measured speed
        self.use_cost_model = bool(train_cfg.extra.get("cost_model", True))
        self.speed_feedback = bool(train_cfg.extra.get("speed_feedback", True))
        import threading
        self._plan_lock = threading.Lock()
        self._pending_speed = None
        self.speed = None                   # relative speed per server after the last feedback
        self._attn_events: list = []        # (start, end) CUDA events of this step's attention calls
        self._wait_events: list = []        # ... and of its signal waits (time this rank stood idle), with the wait's name
        # waits longer than this many milliseconds are kept as "blocking events" (the reference's TickSync blocking
        # detection, distca/runtime/megatron/ops/stream_sync_fn.py:24-77); None: off
        thr = train_cfg.extra.get("wait_report_ms", os.environ.get("DISTCA_WAIT_REPORT_MS"))
        self.wait_report_ms = float(thr) if thr not in (None, "") else None
        self.blocking_events: list = []     # dicts {step, wait, index, ms}, newest last, at most 4096 kept
        self._steps_seen = 0
        self._predicted_ms = 0.0            # what the cost model predicted for them
        self.predicted_ms = 0.0             # cost-model milliseconds (forward + backward) of the current plan on this server

    # ------------------------------------------------------------------------------------------
    def _setup(self, T: int) -> None:
        """Allocate and carve the arena for ``T`` tokens per rank (collective over the group)."""
        self.T = T
        W = self.W
        buf_bytes = int(self.tcfg.comm_buffer_gb * (1 << 30))
        self.max_q = 2 * T
        kv_room = max(buf_bytes - self.max_q * self.q_bytes, 2 * T * 2 * self.kv_bytes)
        self.max_kv = min(max(2 * T, kv_room // (2 * self.kv_bytes)), W * T)
        self.C = W
        sizes = {
            "Qr": self.max_q * self.q_bytes, "Kr": self.max_kv * self.kv_bytes, "Vr": self.max_kv * self.kv_bytes,
            "dOr": self.max_q * self.q_bytes, "DELTAr": self.max_q * self.hq * 4, "LSE": self.max_q * self.hq * 4,
            "AO": T * self.q_bytes, "LSEo": T * self.hq * 4, "DQKV": T * self.qkvd * 2,
            "SLOTS": self.C * T * 2 * self.kv_bytes,
        }
        total = sum(sizes.values()) + 16 * 1024 * len(sizes) + 4096
        self.arena = PeerArena(total, self.group, self.device)
        self.sig = SignalBoard(self.arena, 4)
        self.off = {k: self.arena.alloc(v) for k, v in sizes.items()}
        a = self.arena
        self.Qr = a.view(self.off["Qr"], (self.max_q, self.hq, self.D), torch.bfloat16)
        self.Kr = a.view(self.off["Kr"], (self.max_kv, self.hkv, self.D), torch.bfloat16)
        self.Vr = a.view(self.off["Vr"], (self.max_kv, self.hkv, self.D), torch.bfloat16)
        self.dOr = a.view(self.off["dOr"], (self.max_q, self.hq, self.D), torch.bfloat16)
        self.DELTAr = a.view(self.off["DELTAr"], (self.max_q, self.hq), torch.float32)
        self.LSE = a.view(self.off["LSE"], (self.max_q, self.hq), torch.float32)
        self.AO = a.view(self.off["AO"], (T, self.qd), torch.bfloat16)
        self.LSEo = a.view(self.off["LSEo"], (T, self.hq), torch.float32)   # log-sum-exp of this rank's own tokens
        self.DQKV = a.view(self.off["DQKV"], (T, self.qkvd), torch.bfloat16)
        self.SLOTS = a.view(self.off["SLOTS"], (self.C, T, 2 * self.kd), torch.bfloat16)
        self.planner = Planner(PlannerConfig(world=W, tokens_per_rank=T, tolerance=self.tolerance,
                                             q_row_bytes=self.q_bytes, kv_row_bytes=self.kv_bytes,
                                             max_q_rows=self.max_q, max_kv_rows=self.max_kv,
                                             cost_model=self._cost_model() if self.use_cost_model else None))

    def _cost_model(self) -> dict:
        """The balancer's cost model: fitted to a measured sweep when ``extra["cost_model_file"]`` names one
        (``kernel_bench --kernel attn_sweep`` output of this machine), else the built-in B200 constants."""
        path = self.tcfg.extra.get("cost_model_file")
        if path:
            from ..planner import cost_model_from_sweep
            cm = cost_model_from_sweep(path, heads_q=self.hq)
            return {k: cm[k] for k in ("tile", "ms_per_tile_pair", "ms_per_q_tile", "ms_per_task")}
        return default_cost_model(self.hq)

    # ------------------------------------------------------------------------------------------
    def make_plan(self, docs_per_rank: list[list[int]]):
        """Host-only part of planning (callable ahead of time / from another thread)."""
        cap = max(max((sum(d) for d in docs_per_rank), default=0), self.capacity_hint if self.arena is None else 0)
        if self.arena is None:
            self._setup(cap)
        assert cap <= self.T, "tokens per rank grew beyond the arena capacity"
        policy = self.tcfg.extra.get("attention_policy", "cad")
        with self._plan_lock:       # the planning thread and the step's thread never plan at the same time
            if self._pending_speed is not None:
                self.planner.set_speed(self._pending_speed)
                self._pending_speed = None
            if policy == "cp":
                return self.planner.plan_fixed_cp(docs_per_rank)   # baseline: per-document context parallelism
            if policy == "water_fill":
                return self.planner.plan_fixed_water_fill(docs_per_rank)   # legacy: only the longest document moves
            return self.planner.plan_fixed(docs_per_rank)

    def make_tables(self, plan) -> dict:
        """Host-only: this rank's address tables and attention work lists for ``plan`` as numpy arrays
        (no CUDA call, no change of this object: callable from the planning thread)."""
        rp = plan.rank(self.me)
        T = int(rp.num_tokens)
        base = np.asarray(self.arena.base, dtype=np.int64)
        # ---- owner-side tables ----
        qr, qrow = rp.q_dst_rank.astype(np.int64), rp.q_dst_row.astype(np.int64)
        C = max(1, int(rp.max_copies))
        kr = rp.kv_dst_rank.reshape(T, C).astype(np.int64)
        krow = rp.kv_dst_row.reshape(T, C).astype(np.int64)
        t = {"T": T, "copies": C,
             "q_dst": base[qr] + self.off["Qr"] + qrow * self.q_bytes,
             "delta_dst": base[qr] + self.off["DELTAr"] + qrow * (self.hq * 4),
             "lse_dst": base[qr] + self.off["LSE"] + qrow * (self.hq * 4),
             "kv_dst": np.ascontiguousarray(np.where(kr >= 0, base[np.maximum(kr, 0)] + self.off["Kr"] + krow * self.kv_bytes, 0)),
             "kv_valid": np.ascontiguousarray(rp.kv_dst_rank.reshape(T, C))}
        # ---- server-side tables ----
        tasks = rp.tasks  # [n, 8]: doc, q_a, q_b, q_row0, k_row0, kv_len, owner, owner_row0
        t["q_rows"], t["kv_rows"] = int(rp.q_rows), int(rp.kv_rows)
        if len(tasks):
            qlen = (tasks[:, 2] - tasks[:, 1]).astype(np.int64)
            at = attn_ops.AttnTasks(tasks[:, 3].astype(np.int64), qlen, tasks[:, 4].astype(np.int64),
                                    tasks[:, 5].astype(np.int64))
            owner = np.repeat(tasks[:, 6].astype(np.int64), qlen)
            orow = np.repeat(tasks[:, 7].astype(np.int64), qlen) + (np.arange(qlen.sum()) - np.repeat(np.cumsum(qlen) - qlen, qlen))
            row_out = base[owner] + self.off["AO"] + orow * self.q_bytes
            lse_out = base[owner] + self.off["LSEo"] + orow * (self.hq * 4)
            q_ret = base[owner] + self.off["DQKV"] + orow * (self.qkvd * 2)
        else:
            at = attn_ops.AttnTasks.from_lists([])
            row_out = lse_out = q_ret = np.zeros(0, dtype=np.int64)
        t["attn_plan"] = attn_ops.AttnPlan(at, self.device, upload=False)
        w = t["attn_plan"].fwd_host.copy()
        if len(w):
            w["out_ptr"] = row_out[w["q_row0"]].astype(np.uint64)
            w["lse_ptr"] = lse_out[w["q_row0"]].astype(np.uint64)   # statistics go home with the output rows
        t["fwd_work"] = w
        t["q_ret"] = q_ret
        kv_ret = np.zeros(t["kv_rows"], dtype=np.int64)
        slot_bytes = self.T * 2 * self.kv_bytes
        for k0, n, own, orow0, slot in rp.ctx_segments:
            kv_ret[k0:k0 + n] = (base[own] + self.off["SLOTS"] + int(slot) * slot_bytes
                                 + (int(orow0) + np.arange(n, dtype=np.int64)) * (2 * self.kv_bytes))
        t["kv_ret"] = kv_ret
        flops = np.asarray(plan.flops_after)
        cost = np.asarray(plan.cost_after)
        t["predicted_ms"] = float(cost[self.me]) if self.use_cost_model else 0.0
        t["stats"] = {"imbalance_before": plan.imbalance_before, "imbalance_after": plan.imbalance_after,
                      "cost_imbalance_after": plan.cost_imbalance_after,
                      "tolerance": plan.tolerance_used, "q_rows": t["q_rows"], "kv_rows": t["kv_rows"],
                      "tasks": int(len(tasks)), "send_bytes": rp.send_bytes.tolist(),
                      "my_flops_share": float(flops[self.me] / max(flops.sum(), 1.0))}
        return t

    def make_plan_span(self, batches: list[list[int]]):
        """Plan for documents laid out over the ranks by sequential fill (a document longer than a rank's
        share spans consecutive ranks as head / tail pieces, distca/planner/planner.py:243-267):
        ``batches`` = document lengths per sequence of the global batch. Host only."""
        cap = sum(sum(b) for b in batches) // self.W
        if self.arena is None:
            self._setup(max(cap, self.capacity_hint))
        assert cap <= self.T, "tokens per rank grew beyond the arena capacity"
        with self._plan_lock:
            if self._pending_speed is not None:
                self.planner.set_speed(self._pending_speed)
                self._pending_speed = None
            return self.planner.plan(batches)

    def plan_step(self, docs_per_rank: list[list[int]], dp_rank: int | None = None, plan=None, tables=None) -> None:
        """Plan core attention for this slot's documents (``docs_per_rank[r]`` may be empty) and put
        this rank's tables on the device. ``plan`` / ``tables`` may come from :meth:`make_plan` /
        :meth:`make_tables` run ahead of time."""
        if plan is None:
            plan = self.make_plan(docs_per_rank)
        if not plan.fits:
            raise RuntimeError("core-attention plan does not fit the communication arena; raise --comm-buffer-gb")
        if tables is None:
            tables = self.make_tables(plan)
        self.last_plan = plan
        dev = self.device
        self.Tcur, self.copies = tables["T"], tables["copies"]
        self.q_dst = torch.from_numpy(tables["q_dst"]).to(dev)
        self.delta_dst = torch.from_numpy(tables["delta_dst"]).to(dev)
        self.lse_dst = torch.from_numpy(tables["lse_dst"]).to(dev)
        self.kv_dst = torch.from_numpy(tables["kv_dst"]).to(dev)
        self.kv_valid = torch.from_numpy(tables["kv_valid"]).to(dev)
        self.q_rows, self.kv_rows = tables["q_rows"], tables["kv_rows"]
        self.attn_plan = tables["attn_plan"]
        self.attn_plan.upload()
        w = tables["fwd_work"]
        self.fwd_work = attn_ops._to_device(w, dev) if len(w) else torch.zeros(0, dtype=torch.uint8, device=dev)
        self.q_ret = torch.from_numpy(tables["q_ret"]).to(dev)
        self.kv_ret = torch.from_numpy(tables["kv_ret"]).to(dev)
        self.plan_stats = tables["stats"]
        self.predicted_ms = tables.get("predicted_ms", 0.0)

    # ------------------------------------------------------------------------------------------
    # measured-speed feedback into the planner
    _FWD_SHARE = 0.23      # forward share of the cost model's forward + backward milliseconds
    MIN_FEEDBACK_MS = 20.0 # mean attention time per step below which the measurements are not fed back

    def _timed_attention(self, share: float):
        """Context manager: CUDA events around one attention call (read back at the end of the step)."""
        rt = self

        class _T:
            def __enter__(self_inner):
                if rt.speed_feedback and rt.use_cost_model:
                    self_inner.a = torch.cuda.Event(enable_timing=True)
                    self_inner.a.record()
                return self_inner

            def __exit__(self_inner, *exc):
                if rt.speed_feedback and rt.use_cost_model:
                    b = torch.cuda.Event(enable_timing=True)
                    b.record()
                    rt._attn_events.append((self_inner.a, b))
                    rt._predicted_ms += rt.predicted_ms * share
                return False
        return _T()

    def _timed_wait(self, what: str = ""):
        """Context manager: CUDA events around one signal wait (how long this rank stood idle). ``what`` names the
        wait in the blocking report."""
        rt = self

        class _T:
            def __enter__(self_inner):
                if rt.speed_feedback and rt.use_cost_model:
                    self_inner.a = torch.cuda.Event(enable_timing=True)
                    self_inner.a.record()
                return self_inner

            def __exit__(self_inner, *exc):
                if rt.speed_feedback and rt.use_cost_model:
                    b = torch.cuda.Event(enable_timing=True)
                    b.record()
                    rt._wait_events.append((self_inner.a, b, what))
                return False
        return _T()

    def end_of_step_feedback(self, smoothing: float = 0.5, wait_gain: float = 0.5) -> None:
        """Collective over the attention group, called once per step after the device was synchronised.
        Every server reports (attention time measured, attention time predicted, time spent idle in signal
        waits); the planner's next plans give server ``r`` the share of the attention work that would have
        made all servers equally busy: its measured rate (predicted work per millisecond of attention: GPUs
        under a power cap do not run at one clock, and the cost model is not exact) times the attention time
        it can afford, i.e. what it had plus ``wait_gain`` of its idle time above the group's mean (a rank
        whose GEMMs run slower idles less and gets less attention work). The reference balances predicted
        FLOPs only."""
        if not (self.speed_feedback and self.use_cost_model) or self.arena is None:
            return
        measured = sum(a.elapsed_time(b) for a, b in self._attn_events)
        waits = [(w, a.elapsed_time(b)) for a, b, w in self._wait_events]
        waited = sum(ms for _, ms in waits)
        self._steps_seen += 1
        if self.wait_report_ms is not None:
            self.blocking_events = (self.blocking_events
                                    + self.blocking_report(waits, self.wait_report_ms, self._steps_seen))[-4096:]
        predicted, self._attn_events, self._wait_events, self._predicted_ms = self._predicted_ms, [], [], 0.0
        import torch.distributed as dist
        mine = torch.tensor([measured, predicted, waited], dtype=torch.float32, device=self.device)
        allv = torch.empty(self.W * 3, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(allv, mine, group=self.group)
        allv = allv.view(self.W, 3).cpu().numpy().astype(np.float64)
        if (allv[:, :2] <= 0).any():
            return                       # a server without work this step: keep the current shares
        self.last_measured = allv
        self.plan_stats["attention_ms_per_server"] = [round(float(v), 2) for v in allv[:, 0]]
        self.plan_stats["attention_time_imbalance"] = float(allv[:, 0].max() / allv[:, 0].mean())
        if allv[:, 0].mean() < self.MIN_FEEDBACK_MS:
            return                       # a step this short measures launch overheads, not the servers' speed
        share = self.feedback_shares(allv[:, 0], allv[:, 1], allv[:, 2], wait_gain)
        prev = self.speed if self.speed is not None else np.ones(self.W)
        speed = smoothing * share + (1.0 - smoothing) * prev
        speed = np.clip(speed, prev * 0.95, prev * 1.05)          # at most 5 % per step: one odd step cannot swing the plan
        self.speed = speed / speed.mean()
        self.plan_stats["idle_ms_per_server"] = [round(float(v), 2) for v in allv[:, 2]]
        self._pending_speed = self.speed.tolist()
        self.plan_stats["speed"] = [round(float(v), 4) for v in self.speed]
    # ------------------------------------------------------------------------------------------
    # server halves (every rank of the group runs them once per layer and direction)
    @staticmethod
    def blocking_report(waits, threshold_ms: float, step: int = 0) -> list:
        """``waits``: (name, milliseconds) of one step's signal waits in launch order. Returns one record per wait
        that kept the stream idle for longer than ``threshold_ms``: which wait, its index among the step's waits of
        that name (= the layer, in forward order for the forward waits and in backward order for the others) and
        how long."""
        seen: dict = {}
        out = []
        for name, ms in waits:
            k = seen.get(name, 0)
            seen[name] = k + 1
            if ms > threshold_ms:
                out.append({"step": step, "wait": name, "index": k, "ms": round(float(ms), 3)})
        return out

    @staticmethod
    def feedback_shares(attn_ms, predicted, idle_ms, wait_gain: float = 0.5):
        """Relative share of the attention work per server (mean 1) from one step's measurements."""
        attn_ms, predicted, idle_ms = (np.asarray(x, dtype=np.float64) for x in (attn_ms, predicted, idle_ms))
        rate = predicted / attn_ms                                   # work per millisecond of attention
        afford = attn_ms + wait_gain * (idle_ms - idle_ms.mean())    # attention time that evens out the idle time
        afford = np.maximum(afford, 0.5 * attn_ms)
        want = rate * afford
        return np.clip(want / want.mean(), 0.75, 1.3)

    def _serve_forward(self) -> None:
        self._serve_forward_begin()
        self._serve_forward_end()

    def _serve_forward_begin(self) -> None:
        with timers.phase("cad_wait_qkv"), self._timed_wait("qkv"):
            self.sig.wait(SIG_QKV)
        with timers.phase("cad_attn_fwd"), self._timed_attention(self._FWD_SHARE):
            attn_ops.flash_fwd(self.Qr, self.Kr, self.Vr, self.attn_plan, out=self.AO.unflatten(1, (self.hq, self.D)),
                               lse=self.LSE, work_dev=self.fwd_work)
        self.sig.signal(SIG_OUT)

    def _serve_forward_end(self) -> None:
        with timers.phase("cad_wait_out"), self._timed_wait("out"):
            self.sig.wait(SIG_OUT)

    def _serve_backward(self, layer: int | None = None) -> None:
        self._serve_backward_begin(layer)
        self._serve_backward_end()

    def _serve_backward_begin(self, layer: int | None = None) -> None:
        with timers.phase("cad_wait_dout"), self._timed_wait("dout"):
            self.sig.wait(SIG_DOUT)   # also covers this layer's Q/K/V rows: every owner sends them first
        nq, nk = max(self.q_rows, 1), max(self.kv_rows, 1)
        lse = self.LSE[:nq]    # sent by the owners together with dO and delta
        fused = bool(self.tcfg.extra.get("fuse_grad_return", True))
        with timers.phase("cad_attn_bwd"), self._timed_attention(1.0 - self._FWD_SHARE):
            if self.q_rows and fused:
                # the backward kernels store every dQ row and every dK / dV row straight into its owner's arena
                # (DQKV rows / copy slots, peer stores over NVLink) from their epilogues: nothing is staged
                # on the server and no scatter pass follows
                attn_ops.flash_bwd(self.Qr[:nq], self.Kr[:nk], self.Vr[:nk], None, lse, self.dOr[:nq],
                                   self.attn_plan, scratch=self.scratch, delta_rows=self.DELTAr[:nq],
                                   dq_row_ptr=self.q_ret, dkv_row_ptr=self.kv_ret, dv_off_bytes=self.kv_bytes)
            elif self.q_rows:
                dq = torch.empty(nq, self.hq, self.D, dtype=torch.bfloat16, device=self.device)
                dk = torch.empty(nk, self.hkv, self.D, dtype=torch.bfloat16, device=self.device)
                dv = torch.empty(nk, self.hkv, self.D, dtype=torch.bfloat16, device=self.device)
                attn_ops.flash_bwd(self.Qr[:nq], self.Kr[:nk], self.Vr[:nk], None, lse, self.dOr[:nq],
                                   self.attn_plan, dq=dq, dk=dk, dv=dv, scratch=self.scratch,
                                   delta_rows=self.DELTAr[:nq])
        with timers.phase("cad_return"):
            if self.q_rows and not fused:
                scatter_rows(dq.flatten(1)[:self.q_rows], self.q_bytes, self.q_ret)
                if self.kv_rows:
                    scatter_rows(dk.flatten(1)[:self.kv_rows], self.kv_bytes, self.kv_ret)
                    scatter_rows(dv.flatten(1)[:self.kv_rows], self.kv_bytes, self.kv_ret, self.kv_bytes)
            self.sig.signal(SIG_DQKV)

    def _serve_backward_end(self) -> None:
        with timers.phase("cad_wait_dqkv"), self._timed_wait("dqkv"):
            self.sig.wait(SIG_DQKV)

    # ------------------------------------------------------------------------------------------
    # the model-facing interface (same as LocalCoreAttention)
    def apply_rope(self, qkv, pos, table) -> None:
        """RoPE fused with the Q/K/V dispatch: rotated rows go to the servers, nothing is written back."""
        with timers.phase("cad_dispatch"):
            ew.rope_(qkv, pos, table, self.hq, self.hkv, self.D, q_dst=self.q_dst, kv_dst=self.kv_dst,
                     max_copies=self.copies, v_off_bytes=self.off["Vr"] - self.off["Kr"], write_inplace=False)
            self.sig.signal(SIG_QKV)

    def qkv_epilogue(self):
        """The QKV GEMM's epilogue rotates the heads and stores the rows straight into the servers'
        arenas (same tables as :meth:`apply_rope`); nothing is written locally."""
        if self.Tcur == 0:
            return None
        return {"write_local": False, "q_dst": self.q_dst, "kv_dst": self.kv_dst, "max_copies": self.copies,
                "v_off_bytes": self.off["Vr"] - self.off["Kr"]}

    def qkv_dispatched(self) -> None:
        self.sig.signal(SIG_QKV)

    def forward(self, qkv: torch.Tensor, layer: int = 0):
        self.forward_begin(qkv, layer)
        return self.forward_end()

    # The two halves let a ping-pong schedule put another nano-batch's work between "my server has
    # finished and signalled" and "every server has delivered my rows".
    def forward_begin(self, qkv, layer: int = 0) -> None:
        self._serve_forward_begin()

    def forward_end(self):
        """(attention output rows, log-sum-exp rows) of this rank's own tokens: both were written into this
        rank's arena by the servers, which keep nothing between forward and backward."""
        self._serve_forward_end()
        return self.AO[:self.Tcur], None

    def pack_saved(self, attn_out: torch.Tensor, ctx=None) -> torch.Tensor:
        """What ``keep_attn`` stores per layer: O and the statistics side by side, [T, qd + 2 hq] bf16."""
        T = attn_out.shape[0]
        return torch.cat([attn_out, self.LSEo[:T].view(torch.bfloat16)], dim=1)

    def restore(self, qkv: torch.Tensor, saved: torch.Tensor, layer: int = 0):
        """Recompute under ``keep_attn``: the Q/K/V rows were dispatched again by the QKV epilogue; the
        attention output and its statistics come from the owner's store, so no attention kernel and no
        wait runs here."""
        o = saved[:, :self.qd]
        lse = saved[:, self.qd:].contiguous().view(torch.float32)
        return o, (o, lse)

    def backward(self, ctx, dattn: torch.Tensor, layer: int = 0) -> torch.Tensor:
        self.backward_begin(ctx, dattn, layer)
        return self.backward_end()

    def backward_begin(self, ctx, dattn, layer: int = 0) -> None:
        self.backward_dispatch(ctx, dattn, layer)
        self.backward_serve(layer)

    def backward_dispatch(self, ctx, dattn, layer: int = 0) -> None:
        """Owner half: dO and delta rows go to the servers of this rank's queries."""
        T = self.Tcur
        if T:
            o, lse = ctx if ctx is not None else (self.AO[:T], self.LSEo[:T])
            with timers.phase("cad_dispatch"):
                if self.tcfg.extra.get("fuse_dout_dispatch", True) and lse.stride(1) == 1:
                    # one kernel: delta = rowsum(dO o O), then dO / delta / LSE rows stored at the servers
                    attn_ops.dispatch_dout(o.unflatten(1, (self.hq, self.D)), dattn.unflatten(1, (self.hq, self.D)), lse,
                                           self.q_dst, self.off["dOr"] - self.off["Qr"], self.delta_dst, self.lse_dst)
                else:
                    delta = attn_ops.attn_delta_rows(o.unflatten(1, (self.hq, self.D)),
                                                     dattn.unflatten(1, (self.hq, self.D)))
                    scatter_rows(dattn, self.q_bytes, self.q_dst, self.off["dOr"] - self.off["Qr"])
                    scatter_rows(delta, self.hq * 4, self.delta_dst)
                    scatter_rows(lse, self.hq * 4, self.lse_dst)
        self.sig.signal(SIG_DOUT)

    def backward_serve(self, layer: int = 0) -> None:
        """Server half: attention backward for the tasks planned onto this rank, gradients sent home."""
        self._serve_backward_begin(layer)

    def backward_end(self):
        self._serve_backward_end()
        T = self.Tcur
        if not T:
            return None
        with timers.phase("cad_return"):
            sum_slots(self.SLOTS[:self.copies, :T], self.kv_valid, self.DQKV[:T, self.qd:])
        return self.DQKV[:T]

    def no_tokens_dispatch(self) -> None:
        """Stand-in for ``apply_rope`` on a rank that owns no tokens in this slot."""
        self.sig.signal(SIG_QKV)

    def restore_no_tokens(self, layer: int = 0) -> None:
        pass

    def dummy_forward(self) -> None:
        """One layer's forward for a rank that owns no tokens in this slot: serve only."""
        self.sig.signal(SIG_QKV)
        self._serve_forward()

    def dummy_backward(self) -> None:
        """One layer's backward (after its ``dummy_forward`` recompute twin) for a rank without tokens."""
        self.sig.signal(SIG_DOUT)
        self._serve_backward()

    def close(self) -> None:
        if self.arena is not None:
            self.arena.close()
            self.arena = None
