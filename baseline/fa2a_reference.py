"""Driver for the REFERENCE arm of the core-attention dispatch micro-benchmark.

Runs the reference's own stock path, unmodified, from the copy installed under ``baseline/_ref``:

    planner          distca/planner/planner.py  (``batch_to_items_general`` -> ``Planner.plan``)
    metadata         distca/runtime/compute_metadata.py::from_planner_output
    pack             distca/runtime/attn_kernels/dispatch.py::pre_a2a_qkv      (csrc/core/memcpy.cu)
    all-to-all       distca/runtime/attn_kernels/ops.py::fast_a2a             (csrc/core/fastalltoall.cu, NVSHMEM)
    unpack           distca/runtime/attn_kernels/dispatch.py::post_a2a_qkv

exactly as its multi-GPU test drives them (tests/test_dispatch_fast.py:32-165), with the two-buffer
acquire / release protocol of the training path (``instance_id`` alternating 0 / 1). The reference's native
library ``libas_comm.so`` is built from its ``csrc/`` for sm_100a against the installed NVSHMEM package and
placed next to ``ops.py`` (see ``baseline/README.md``). ``compute_metadata.py`` imports one dataclass from
Megatron-LM, which is absent offline: ``baseline/stubs`` provides that dataclass and nothing else.

None of this framework's kernels, planner or runtime is on this path; this file only feeds the documents in
and times the calls with CUDA events.
"""
from __future__ import annotations

import os
import sys
from types import SimpleNamespace

_HERE = os.path.dirname(os.path.abspath(__file__))


def available() -> str | None:
    """``None`` when the reference arm can run, else a one-line reason."""
    ref = os.path.join(_HERE, "_ref", "distca")
    if not os.path.isdir(ref):
        return "reference package not installed under baseline/_ref"
    if not os.path.exists(os.path.join(ref, "runtime", "attn_kernels", "libas_comm.so")):
        return "baseline/_ref/distca/runtime/attn_kernels/libas_comm.so not built (see baseline/README.md)"
    if not os.path.isdir(os.path.join(ref, "planner")):
        return "baseline/_ref/distca/planner missing (the reference's setup.py does not package it; see baseline/README.md)"
    return None


def _paths() -> None:
    for p in (os.path.join(_HERE, "_ref"), os.path.join(_HERE, "stubs")):
        if p not in sys.path:
            sys.path.insert(0, p)


def plan_metadata(docs_per_rank, world: int, tokens_per_rank: int, heads_q: int, heads_kv: int, head_dim: int,
                  tolerance: float):
    """(forward Q/K/V metadata, reverse metadata) from the reference planner, on the host."""
    _paths()
    import torch
    from distca.planner.planner import Planner, batch_to_items_general
    par = SimpleNamespace(pipeline_model_parallel_size=1, tensor_model_parallel_size=1)
    mc = SimpleNamespace(hidden_size=heads_q * head_dim, num_attention_heads=heads_q, num_key_value_heads=heads_kv)
    items = batch_to_items_general(docs_per_rank, tokens_per_rank, world, mc)
    planner = Planner(world, par, tolerance_factor=tolerance, model_config=mc, dtype=torch.bfloat16)
    fa2a, _attn, _mlp_len, _ranges = planner.plan(items, device="cpu")
    return fa2a[0], fa2a[1]


def required_buffer_bytes(md, world: int) -> int:
    """Largest send or receive footprint of any rank under ``md`` (bytes), rounded up to 1 MiB."""
    need = 0
    for r in range(world):
        s = md.get_slice(r)
        send_disp, send_sz, recv_disp, recv_sz = (t.to("cpu").long() for t in s.fa2a_metadata)
        need = max(need, int((send_disp + send_sz).max()), int(recv_sz.sum()), int(send_sz.sum()))
    return (need + (1 << 20)) // (1 << 20) * (1 << 20) + (1 << 20)


class ReferenceDispatcher:
    """NVSHMEM bootstrap + the reference's two ``DispatcherWrapper`` buffers, as
    ``MegatronBaseWorker.init_nvshmem`` sets them up (distca/utils/test_util.py:114-123)."""

    def __init__(self, rank: int, local_rank: int, world: int, buffer_bytes: int):
        _paths()
        os.environ.setdefault("NVSHMEM_DISABLE_NVLS", "1")          # plain peer stores only on shared machines
        os.environ.setdefault("NVSHMEM_SYMMETRIC_SIZE", str(4 * buffer_bytes + (256 << 20)))
        os.environ.setdefault("NVSHMEM_BOOTSTRAP_UID_SOCK_IFNAME", "lo")
        import torch
        import torch.distributed as dist
        from distca.runtime.attn_kernels import ops
        self.ops, self.torch = ops, torch
        uid = ops.nvshmem_get_unique_id() if rank == 0 else ops.nvshmem_alloc_empty_unique_id()
        dist.broadcast(uid, src=0)                                   # CPU tensor: goes over gloo
        ops.DispatcherWrapper.init(rank, local_rank, world, buffer_bytes, uid)
        ops.DispatcherWrapper.comm_stream = torch.cuda.Stream(priority=-1)

    def make_call(self, md_slice, q, k, v):
        """A closure that runs pack -> all-to-all -> unpack once for this rank's slice of the metadata."""
        torch = self.torch
        from distca.runtime.attn_kernels.dispatch import post_a2a_qkv, pre_a2a_qkv
        from distca.runtime.attn_kernels.ops import fast_a2a
        md = md_slice.normalize()
        dev, dt = q.device, q.dtype
        recv_q = torch.zeros(md.tensor_shape[0].recv_shape, dtype=dt, device=dev)
        recv_k = torch.zeros(md.tensor_shape[1].recv_shape, dtype=dt, device=dev)
        recv_v = torch.zeros_like(recv_k)
        state = {"i": 0}

        def call():
            iid = state["i"] & 1
            state["i"] += 1
            pre_a2a_qkv(q, k, v, md.kv_replica_mask, md.seq_lens[0].send_seqlens, md.seq_lens[1].send_seqlens,
                        *md.send_memcpy_metadata, is_fwd=True, instance_id=iid)
            fast_a2a(*md.fa2a_metadata, md.my_rank_send_offset, md.my_rank_recv_offset, md.my_rank_send_sz,
                     instance_id=iid)
            post_a2a_qkv(recv_q, recv_k, recv_v, md.kv_replica_mask, md.seq_lens[0].recv_seqlens,
                         md.seq_lens[1].recv_seqlens, *md.recv_memcpy_metadata, is_fwd=True, switch_buffer=False,
                         instance_id=iid)
            return recv_q, recv_k, recv_v
        return call

    def barrier(self) -> None:
        self.ops.nvshmem_barrier_all()
