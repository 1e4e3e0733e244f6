"""Data-parallel gradient reduction + sharded AdamW (ZeRO-1 style distributed optimizer).

Every data-parallel rank owns one contiguous slice of the flat parameter buffer. A step is

  1. reduce-scatter of the flat gradient buffer -> this rank's gradient slice (mean over ranks),
  2. global gradient norm (sum of squares on the slice, all-reduce of one float) -> clip factor that
     stays on the device,
  3. AdamW on the slice with split fp32 masters (bf16 parameter + 16-bit remainder),
  4. all-gather of the updated bf16 slices into every rank's flat parameter buffer.

Step 1 uses either NCCL (``reduce_scatter_tensor``) or the peer-memory kernel of
:mod:`distca_b200.parallel.p2p` that pulls the peers' slices over NVLink, sums in fp32 and feeds
Adam directly. The reference delegates all of this to Megatron's DistributedOptimizer with
``grad_reduce_in_fp32`` (distca/utils/megatron_test_utils.py:235-258, worker.py:49-66, 246-251).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import TrainConfig
from ..models.llama import ParamStore
from ..ops import elementwise as ew


class ShardedAdam:
    def __init__(self, store: ParamStore, cfg: TrainConfig, dp_group=None, norm_group=None,
                 replicated_names: tuple[str, ...] = (), tp_rank: int = 0, p2p=None):
        self.store, self.cfg = store, cfg
        self.dp_group = dp_group
        self.norm_group = norm_group          # every rank whose parameters enter the global norm
        self.dp = dist.get_world_size(dp_group) if dp_group is not None else 1
        self.dp_rank = dist.get_rank(dp_group) if dp_group is not None else 0
        assert store.numel % (self.dp * ParamStore.ALIGN) == 0, "pad the parameter buffer to dp * ALIGN"
        self.shard = store.numel // self.dp
        self.lo, self.hi = self.dp_rank * self.shard, (self.dp_rank + 1) * self.shard
        dev = store.flat.device
        self.on_gpu = dev.type == "cuda"
        self.m = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.shard, dtype=torch.float32, device=dev)
        self.lo16 = torch.zeros(self.shard, dtype=torch.int16, device=dev) if self.on_gpu else None
        self.master = None if self.on_gpu else store.flat[self.lo:self.hi].float().clone()
        self.step_count = 0
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.gscale = torch.ones(1, dtype=torch.float32, device=dev)
        self.p2p = p2p
        # parameters that every tensor-parallel rank holds a full copy of count once in the norm
        self._dup_ranges = []
        if tp_rank != 0:
            for n in replicated_names:
                o, k = store.offsets[n]
                self._dup_ranges.append((o, o + k))
        self.last_grad_norm = None
        # gradient reduce-scatter in buckets while backward still runs (peer transport only)
        # (not with tensor parallelism: the replicated norm-weight gradients are first summed over the
        # tensor-parallel group at the end of backward, and the data-parallel reduction has to follow that)
        self.bucketed = (self.p2p is not None and self.dp > 1 and not replicated_names
                         and bool(cfg.extra.get("dp_buckets", True)))
        self._reduced: list[tuple[int, int]] = []      # [lo, hi) ranges of this step already reduced
        if self.dp > 1 and store.grad.dtype != torch.float32 and self.p2p is None:
            self._rs_out = torch.empty(self.shard, dtype=store.grad.dtype, device=dev)
        else:
            self._rs_out = None

    # -- 1 --
    def reduce_gradients(self) -> torch.Tensor:
        g = self.store.grad
        if self.dp == 1:
            return g
        out = self._rs_out if self._rs_out is not None else torch.empty(self.shard, dtype=g.dtype, device=g.device)
        # the loss is already divided by the number of valid tokens of the GLOBAL batch, so the
        # gradient of the global batch is the plain sum over data-parallel ranks
        if g.device.type == "cuda":
            dist.reduce_scatter_tensor(out, g, op=dist.ReduceOp.SUM, group=self.dp_group)
        else:
            tmp = g.clone()
            dist.all_reduce(tmp, group=self.dp_group)
            out.copy_(tmp[self.lo:self.hi])
        return out

    # -- 2 --
    def _clip_factor(self, gshard: torch.Tensor) -> None:
        self.sumsq.zero_()
        ew.sumsq_(gshard, self.sumsq)
        for a, b in self._dup_ranges:  # remove this rank's copy of replicated parameters
            a2, b2 = max(a, self.lo) - self.lo, min(b, self.hi) - self.lo
            if b2 > a2:
                self.sumsq -= gshard[a2:b2].float().pow(2).sum()
        if self.norm_group is not None and dist.get_world_size(self.norm_group) > 1:
            dist.all_reduce(self.sumsq, group=self.norm_group)
        norm = self.sumsq.sqrt()
        self.last_grad_norm = norm
        if self.cfg.clip_grad and self.cfg.clip_grad > 0:
            torch.clamp(self.cfg.clip_grad / (norm + 1e-6), max=1.0, out=self.gscale)
        else:
            self.gscale.fill_(1.0)

    def begin_step(self) -> None:
        """Call once per step before any gradient is produced (next to ``zero_grad``)."""
        if self.bucketed:
            self.sumsq.zero_()
            self._reduced = []

    def bucket_ready(self, names) -> None:
        """The gradients of the parameters ``names`` (one layer: a contiguous range of the flat buffer) are
        final for this step: their part of this rank's shard is reduce-scattered now, on a side stream, while
        the backward pass goes on (the reference leaves this to Megatron's DistributedOptimizer with
        ``overlap_grad_reduce`` off, distca/utils/megatron_test_utils.py:235-258). Every rank calls it for the
        same buckets in the same order."""
        if not self.bucketed:
            return
        lo = min(self.store.offsets[n][0] for n in names)
        hi = max(self.store.offsets[n][0] + self.store.offsets[n][1] for n in names)
        hi = (hi + ParamStore.ALIGN - 1) // ParamStore.ALIGN * ParamStore.ALIGN
        a, b = max(lo, self.lo), min(hi, self.hi)
        ranges = []
        if b > a:
            ranges.append((a, b - a))
            self._reduced.append((a, b))
        self.p2p.bucket_ready(ranges, self.sumsq)

    def _remaining(self) -> list[tuple[int, int]]:
        """Parts of this rank's shard that no bucket has reduced yet, as (lo, n)."""
        out, cur = [], self.lo
        for a, b in sorted(self._reduced):
            if a > cur:
                out.append((cur, a - cur))
            cur = max(cur, b)
        if cur < self.hi:
            out.append((cur, self.hi - cur))
        return out

    def _step_peer(self) -> None:
        """Steps 1-4 on peer memory: reduce-scatter fused with the norm partial, Adam fused with the
        parameter all-gather (see :mod:`distca_b200.parallel.dp_p2p`)."""
        c = self.cfg
        if self.bucketed:
            # the layers were reduced as backward produced them; what is left (embedding, final norm, LM head)
            # follows here, after every rank's backward has ended
            self.p2p.join_buckets()
            rest = self._remaining()
            self._reduced = []
            self.p2p.sig.signal(0)
            self.p2p.sig.wait(0)
            for lo, n in rest:
                self.p2p._reduce(lo, n, self.sumsq)
        else:
            self.sumsq.zero_()
            self.p2p.reduce_scatter_sumsq(self.lo, self.shard, self.sumsq)
        gshard = self.store.grad[self.lo:self.hi]
        for a, b in self._dup_ranges:
            a2, b2 = max(a, self.lo) - self.lo, min(b, self.hi) - self.lo
            if b2 > a2:
                self.sumsq -= gshard[a2:b2].float().pow(2).sum()
        if self.norm_group is not None and dist.get_world_size(self.norm_group) > 1:
            dist.all_reduce(self.sumsq, group=self.norm_group)
        norm = self.sumsq.sqrt()
        self.last_grad_norm = norm
        if c.clip_grad and c.clip_grad > 0:
            torch.clamp(c.clip_grad / (norm + 1e-6), max=1.0, out=self.gscale)
        else:
            self.gscale.fill_(1.0)
        self.p2p.adam_push(self.store.flat[self.lo:self.hi], self.lo16, gshard, self.m, self.v, self.lo, lr=c.lr,
                           beta1=c.beta1, beta2=c.beta2, eps=c.eps, weight_decay=c.weight_decay,
                           step=self.step_count, gscale=self.gscale)

    # -- 3 + 4 --
    def step(self) -> None:
        c = self.cfg
        self.step_count += 1
        if self.p2p is not None and self.dp > 1:
            self._step_peer()
            return
        reduced = self.reduce_gradients()
        gshard = reduced if reduced.numel() == self.shard else reduced[self.lo:self.hi]
        self._clip_factor(gshard)
        pshard = self.store.flat[self.lo:self.hi]
        if self.on_gpu:
            ew.adam_step_(pshard, self.lo16, gshard, self.m, self.v, lr=c.lr, beta1=c.beta1, beta2=c.beta2,
                          eps=c.eps, weight_decay=c.weight_decay, step=self.step_count, gscale=self.gscale)
        else:
            ew.adam_step_(self.master, None, gshard, self.m, self.v, lr=c.lr, beta1=c.beta1, beta2=c.beta2,
                          eps=c.eps, weight_decay=c.weight_decay, step=self.step_count, gscale=self.gscale)
            pshard.copy_(self.master.to(pshard.dtype))
        if self.dp > 1:
            dist.all_gather_into_tensor(self.store.flat, pshard.clone() if not self.on_gpu else pshard,
                                        group=self.dp_group)

    def resync_master(self) -> None:
        """Call after the parameters were overwritten from outside (weights loaded without optimizer
        state): the fp32 master copy is rebuilt from the parameters as they are now."""
        if self.on_gpu:
            self.lo16.zero_()
        else:
            self.master.copy_(self.store.flat[self.lo:self.hi].float())

    # -- checkpoint --
    def state_dict(self) -> dict:
        d = {"step": self.step_count, "m": self.m, "v": self.v, "shard_range": (self.lo, self.hi)}
        if self.on_gpu:
            d["lo16"] = self.lo16
        else:
            d["master"] = self.master
        return d

    def load_state_dict(self, d: dict) -> None:
        self.step_count = int(d["step"])
        self.m.copy_(d["m"]); self.v.copy_(d["v"])
        if self.on_gpu and "lo16" in d:
            self.lo16.copy_(d["lo16"])
        elif not self.on_gpu and "master" in d:
            self.master.copy_(d["master"])
