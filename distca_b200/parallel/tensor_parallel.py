"""Tensor parallelism with sequence parallelism (Megatron style): activations between the
linear blocks are sharded by token rows, the QKV / FC1 weights by output rows (heads, FFN
columns), the out-proj / FC2 weights by input columns, embedding and LM head by vocabulary.

    all_gather_rows      [T/tp, H] -> [T, H]      before QKV / FC1 (and their backward twins)
    reduce_scatter_rows  [T, H]    -> [T/tp, H]   after out-proj / FC2 (sum over ranks)

Two transports: NCCL collectives (works everywhere, gloo on CPU), or peer-memory kernels on a
:class:`~distca_b200.parallel.p2p.PeerArena` (pull-based all-gather / reduce-scatter over NVLink;
``use_p2p=True``). The reference gets both collectives from TransformerEngine linears with
``sequence_parallel = tp > 1`` (distca/utils/megatron_test_utils.py:334,
distca/runtime/megatron/model_patch.py:77-98).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class TensorParallel:
    def __init__(self, group, size: int, rank: int, device, use_p2p: bool = False, max_rows_local: int = 0,
                 max_cols: int = 0, tile_loads: bool = False):
        self.group, self.size, self.rank = group, size, rank
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        self.fused = None   # PeerCollectives: all-gather / reduce-scatter fused into the GEMMs
        self.nccl_row_collectives = 0   # all_gather_rows / reduce_scatter_rows calls that went to NCCL (diagnostic)
        self.use_p2p = use_p2p and self.on_gpu
        self._max_cols = max_cols
        self._tile_loads = tile_loads
        if self.use_p2p and max_rows_local > 0:
            self.ensure_fused(max_rows_local)

    def ensure_fused(self, rows_local: int) -> None:
        """Create (or grow) the peer arena of the fused collectives for ``rows_local`` tokens per rank.
        Collective over the group; every rank calls it with the same value (the trainers do, at the first
        step and whenever the micro-batch grows)."""
        if not self.use_p2p:
            return
        if self.fused is not None and self.fused.max_rows >= rows_local:
            return
        if self.fused is not None:
            self.fused.close()
        from .tp_p2p import PeerCollectives
        self.fused = PeerCollectives(self.group, self.size, self.rank, self.device, rows_local, self._max_cols,
                                     tile_loads=self._tile_loads)

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        self.nccl_row_collectives += 1
        out = torch.empty((x.shape[0] * self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        self.nccl_row_collectives += 1
        n = x.shape[0] // self.size
        if self.on_gpu:
            out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
            dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
            return out
        tmp = x.clone()
        dist.all_reduce(tmp, group=self.group)
        return tmp[self.rank * n:(self.rank + 1) * n].clone()

    def all_gather_stats(self, s: torch.Tensor) -> torch.Tensor:
        out = torch.empty((self.size * s.shape[0],) + tuple(s.shape[1:]), dtype=s.dtype, device=s.device)
        dist.all_gather_into_tensor(out, s.contiguous(), group=self.group)
        return out.view((self.size,) + tuple(s.shape))

    def all_reduce_(self, x: torch.Tensor) -> torch.Tensor:
        dist.all_reduce(x, group=self.group)
        return x

    def sync_replicated_grads(self, store) -> None:
        """Norm weights are replicated while their gradients come from this rank's token rows only:
        sum them over the group (Megatron's layer-norm gradient all-reduce under sequence parallel)."""
        names = [n for n, _ in store.shapes if n.endswith("norm_weight") or n.endswith("layernorm.weight")]
        if not names:
            return
        flat = torch.cat([store.g[n].reshape(-1).float() for n in names])
        dist.all_reduce(flat, group=self.group)
        off = 0
        for n in names:
            k = store.g[n].numel()
            store.g[n].copy_(flat[off:off + k].view_as(store.g[n]))
            off += k
