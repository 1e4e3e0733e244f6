"""Core-attention dispatch micro-benchmark (the reference's "fast all-to-all" path: pack kernels
csrc/core/memcpy.cu:23-155 + NVSHMEM put/signal csrc/core/fastalltoall.cu:14-97), multi-GPU:

    torchrun --nproc-per-node 8 -m distca_b200.utils.fa2a_bench --tokens 2048 8192 32768 131072
    torchrun --nproc-per-node 8 -m distca_b200.utils.fa2a_bench --impl reference --tokens 2048 8192 32768 131072

For every payload size each rank owns ``tokens`` tokens of documents with log-uniform lengths in
[128, tokens]; a planner decides which server gets which Q rows and which K/V rows (with fan-out).
Timed, per rank, max over ranks, CUDA events on the launching stream:

* ``push``      – this repository's dispatch: the RoPE kernel rotates Q/K and stores Q, K, V rows
                  straight into the servers' arenas over NVLink, then signals; the timed region ends when
                  every peer's signal has arrived (``wait``), i.e. it includes the cross-rank skew. The
                  attention kernel reads the rows where they land: there is no unpack pass.
* ``nccl``      – NCCL twin: pack on the sender (row gather in destination order, K/V rows once per
                  destination), ``all_to_all_single`` with the same per-pair byte counts, unpack on the receiver.
* ``reference`` – (``--impl reference``) the reference's own planner, metadata, pack kernels, NVSHMEM
                  all-to-all and unpack kernels from ``baseline/_ref`` (driver: ``baseline/fa2a_reference.py``),
                  for the same documents. Its planner makes its own placement, so the bytes it moves are
                  reported beside the time.

Reported: GB/s per rank of REMOTE bytes (own-rank traffic excluded) against 900 GB/s per direction
(nominal) and 770 GB/s (measured peer copy).
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch
import torch.distributed as dist

from ..data.synthetic import pack_documents, sample_loguniform
from ..models.config import ParallelConfig, TrainConfig, get_model_config
from ..ops import elementwise as ew
from ..parallel.cad import SIG_QKV, CadRuntime
from ..parallel.groups import build_groups
from ..runtime.trainer import init_distributed


def _documents(rng, world: int, T: int) -> list[list[int]]:
    """One pack of ``T`` tokens per rank, document lengths log-uniform in [128, T]; batches whose causal work is
    already balanced (max / mean of the ranks' sum of L^2 below 1.3) are drawn again, so that every payload size
    of the sweep has something to dispatch. Both arms call this with the same generator state."""
    for _ in range(64):
        docs = []
        while len(docs) < world:
            lens = sample_loguniform(rng, 64, 128, T)
            docs += pack_documents(lens, T, max_packs=world - len(docs))
        work = [sum(float(L) * L for L in d) for d in docs]
        if max(work) >= 1.3 * (sum(work) / world):
            break
    return docs


def _time_max_over_ranks(fn, iters: int, warmup: int, dev) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def reference_main(a, rank: int, world: int, local: int, dev) -> None:
    """The reference's stock dispatch path on the same documents (see ``baseline/fa2a_reference.py``)."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "baseline", "fa2a_reference.py")
    spec = importlib.util.spec_from_file_location("fa2a_reference", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    why = ref.available()
    if why is not None:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        dist.destroy_process_group()
        return
    cfg = get_model_config(a.model)
    hq, hkv, D = cfg.heads_q, cfg.heads_kv, cfg.head_dim
    rng = np.random.default_rng(0)
    cases = []
    for T in a.tokens:
        docs = _documents(rng, world, T)          # same generator and seed as the other arm: same documents
        fwd, _rev = ref.plan_metadata(docs, world, T, hq, hkv, D, a.tolerance)
        cases.append((T, docs, fwd))
    buf = max(ref.required_buffer_bytes(fwd, world) for _, _, fwd in cases)
    disp = ref.ReferenceDispatcher(rank, local, world, buf)
    for T, docs, fwd in cases:
        s = fwd.get_slice(rank)
        send = s.fa2a_metadata[1].to("cpu").long()
        remote_bytes = int(send.sum() - send[rank])
        q = torch.randn(T, hq * D, device=dev).bfloat16()
        k = torch.randn(T, hkv * D, device=dev).bfloat16()
        v = torch.randn(T, hkv * D, device=dev).bfloat16()
        call = disp.make_call(s, q, k, v)
        ms = _time_max_over_ranks(call, a.iters, a.warmup, dev)
        rb = torch.tensor([float(remote_bytes)], device=dev)
        dist.all_reduce(rb, op=dist.ReduceOp.MAX)
        gbs = float(rb.item()) / (ms * 1e-3) / 1e9
        if rank == 0:
            print(json.dumps({"impl": "reference", "tokens_per_rank": T, "world": world,
                              "remote_mb_per_rank_max": float(rb.item()) / 1e6,
                              "reference": {"ms": ms, "remote_gb_per_s_per_rank": gbs, "frac_of_900": gbs / 900.0,
                                            "frac_of_measured_770": gbs / 770.0},
                              "note": "reference planner + pack + NVSHMEM all-to-all + unpack, unmodified, "
                                      "Megatron's PackedSeqParams dataclass stubbed"}), flush=True)
        disp.barrier()
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, nargs="+", default=[2048, 8192, 32768, 131072])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tolerance", type=float, default=0.02)
    a = ap.parse_args()
    rank, world, local = init_distributed()
    dev = torch.device("cuda", local)
    if a.impl == "reference":
        reference_main(a, rank, world, local, dev)
        return
    cfg = get_model_config(a.model)
    par = ParallelConfig(dp=world)
    groups = build_groups(par, rank)
    rng = np.random.default_rng(0)
    results = []
    for T in a.tokens:
        tc = TrainConfig(cad=True, comm_buffer_gb=max(2.0, T * 12288 * 6 / 2**30))
        rt = CadRuntime(cfg, par, tc, groups, dev, tolerance=a.tolerance)
        docs = _documents(rng, world, T)
        rt.plan_step(docs)
        rp = rt.last_plan.rank(rt.me)
        send = np.asarray(rp.send_bytes, dtype=np.int64)
        remote_bytes = int(send.sum() - send[rt.me])
        qkv = torch.randn(T, rt.qkvd, device=dev).bfloat16()
        pos = (torch.arange(T, device=dev) % 4096).int()
        table = ew.rope_table(4096, rt.D, 500000.0, dev)

        def push():
            rt.apply_rope(qkv, pos, table)     # rotate + remote stores + signal
            rt.sig.wait(SIG_QKV)               # all peers' rows have landed here

        # NCCL twin with the same per-pair byte counts: every row is packed into its destination's segment
        # ([Q rows | K rows | V rows] per destination, K/V rows once per destination), one all_to_all_single,
        # and one pass over the received bytes stands for the unpack
        qr = rp.q_dst_rank.astype(np.int64)
        C = max(1, int(rp.max_copies))
        kr = rp.kv_dst_rank.reshape(T, C).astype(np.int64)
        nq = np.bincount(qr, minlength=world)
        nk = np.bincount(kr[kr >= 0], minlength=world)
        send_n = nq * rt.q_bytes + 2 * nk * rt.kv_bytes       # bytes per destination, own rank included
        recv = np.zeros(world, dtype=np.int64)
        all_send = [None] * world
        dist.all_gather_object(all_send, send_n.tolist())
        for s in range(world):
            recv[s] = all_send[s][rt.me]
        sbuf = torch.empty(int(send_n.sum()), dtype=torch.uint8, device=dev)
        rbuf = torch.empty(int(recv.sum()), dtype=torch.uint8, device=dev)
        unpacked = torch.empty_like(rbuf)
        seg = np.concatenate([[0], np.cumsum(send_n)[:-1]]).astype(np.int64)
        base = sbuf.data_ptr()
        q_rank_in_dst = np.zeros(T, dtype=np.int64)
        for d in range(world):
            m = qr == d
            q_rank_in_dst[m] = np.arange(int(m.sum()))
        q_addr = torch.from_numpy(base + seg[qr] + q_rank_in_dst * rt.q_bytes).to(dev)
        k_addr = np.zeros((T, C), dtype=np.int64)
        fill = np.zeros(world, dtype=np.int64)
        for c in range(C):
            for d in range(world):
                m = kr[:, c] == d
                n = int(m.sum())
                k_addr[m, c] = base + seg[d] + nq[d] * rt.q_bytes + (fill[d] + np.arange(n)) * rt.kv_bytes
                fill[d] += n
        k_addr_dev = [torch.from_numpy(np.ascontiguousarray(k_addr[:, c])).to(dev) for c in range(C)]
        v_off = torch.from_numpy(nk[np.maximum(kr, 0)] * rt.kv_bytes).to(dev)       # V rows sit behind the destination's K rows
        v_addr_dev = [torch.where(k_addr_dev[c] != 0, k_addr_dev[c] + v_off[:, c], k_addr_dev[c]) for c in range(C)]
        from ..parallel.p2p import scatter_rows
        q_src, k_src, v_src = qkv[:, :rt.qd], qkv[:, rt.qd:rt.qd + rt.kd], qkv[:, rt.qd + rt.kd:]

        def nccl():
            scatter_rows(q_src, rt.q_bytes, q_addr)
            for c in range(C):
                scatter_rows(k_src, rt.kv_bytes, k_addr_dev[c])
                scatter_rows(v_src, rt.kv_bytes, v_addr_dev[c])
            dist.all_to_all_single(rbuf, sbuf, output_split_sizes=recv.tolist(), input_split_sizes=send_n.tolist())
            unpacked.copy_(rbuf)

        out = {"tokens_per_rank": T, "remote_mb_per_rank": remote_bytes / 1e6, "world": world}
        for name, fn in (("push", push), ("nccl", nccl)):
            ms = torch.tensor([_time_max_over_ranks(fn, a.iters, a.warmup, dev)])
            gbs = remote_bytes / (ms.item() * 1e-3) / 1e9 if remote_bytes else 0.0
            out[name] = {"ms": ms.item(), "remote_gb_per_s_per_rank": gbs, "frac_of_900": gbs / 900.0,
                         "frac_of_measured_770": gbs / 770.0}
        results.append(out)
        if rank == 0:
            print(json.dumps(out), flush=True)
        rt.close()
        torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
