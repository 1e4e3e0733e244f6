"""Collective micro-benchmark: time against payload for the collectives the step model needs, one JSON line each.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m distca_b200.utils.net_bench \\
        --sizes-mb 16 64 256 1024 --ops all_gather reduce_scatter all_reduce all_to_all push_all_gather > net.jsonl

``bytes_per_rank`` is what one rank contributes (its shard for all-gather / reduce-scatter / the push kernel, its
whole buffer for all-reduce and all-to-all); ``ms`` is device time (CUDA events on the launching stream, a buffer
larger than L2 written between iterations) and the maximum over ranks; ``bus_gbs`` is the usual bus bandwidth
(:func:`bus_bytes` over the time). ``push_all_gather`` is
this repository's peer-store all-gather (``PeerCollectives.all_gather_rows``: stores + signal round trip), the
others are NCCL. On CPU ranks (gloo) the NCCL-free operations run with wall-clock timing, for testing the tool.
The lines load into ``distca_b200.planner.NetworkModel.from_sweep``. The reference profiles the same collectives
with nccl-tests and torch (distca/profiling/modal-scripts/network-prof-pytorch.py, network-prof-nccl-test.py ->
distca/profiling/data/network-*.csv).
"""
from __future__ import annotations

import argparse
import json
import time

import torch
import torch.distributed as dist

from ..runtime.trainer import init_distributed

OPS = ("all_gather", "reduce_scatter", "all_reduce", "all_to_all", "push_all_gather")


def bus_bytes(op: str, world: int, bytes_per_rank: int) -> float:
    """Bytes that cross one rank's link in an ideal ring / switch schedule (the bus-bandwidth numerator of
    nccl-tests): (W-1) shards for all-gather, reduce-scatter and the push kernel, (W-1)/W of the buffer for
    all-to-all, 2 (W-1)/W of it for all-reduce."""
    if world <= 1:
        return 0.0
    if op in ("all_gather", "reduce_scatter", "push_all_gather"):
        return float(bytes_per_rank) * (world - 1)
    if op == "all_reduce":
        return 2.0 * bytes_per_rank * (world - 1) / world
    return float(bytes_per_rank) * (world - 1) / world


def _time(fn, iters: int, warmup: int, device: torch.device, flush) -> float:
    """Mean milliseconds per call on this rank."""
    for _ in range(warmup):
        fn()
    if device.type == "cuda":
        total = 0.0
        for _ in range(iters):
            if flush is not None:
                flush.zero_()
            torch.cuda.synchronize(device)
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize(device)
            total += a.elapsed_time(b)
        return total / iters
    total = 0.0
    for _ in range(iters):
        dist.barrier()
        t0 = time.perf_counter()
        fn()
        total += (time.perf_counter() - t0) * 1e3
    return total / iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-mb", type=float, nargs="+", default=[16, 64, 256, 1024])
    ap.add_argument("--ops", nargs="+", default=list(OPS), choices=OPS)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cols", type=int, default=4096, help="row width (bf16 elements) of the shards")
    a = ap.parse_args(argv)
    rank, world, local = init_distributed()
    on_gpu = torch.cuda.is_available()
    dev = torch.device("cuda", local) if on_gpu else torch.device("cpu")
    dtype = torch.bfloat16 if on_gpu else torch.float32
    esz = torch.empty((), dtype=dtype).element_size()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if on_gpu else None
    sizes = [int(mb * 1e6) // (a.cols * esz * world) * (a.cols * esz * world) for mb in a.sizes_mb]
    sizes = [s for s in sizes if s > 0]
    fused = None
    if "push_all_gather" in a.ops and on_gpu and world > 1:
        from ..parallel.tp_p2p import PeerCollectives
        fused = PeerCollectives(dist.group.WORLD, world, rank, dev, max(sizes) // (a.cols * esz), a.cols)
    for op in a.ops:
        for nbytes in sizes:
            rows = nbytes // (a.cols * esz)
            x = torch.randn(rows, a.cols, device=dev).to(dtype)
            if op == "all_gather":
                out = torch.empty(world * rows, a.cols, dtype=dtype, device=dev)
                fn = lambda: dist.all_gather_into_tensor(out.view(-1), x.view(-1))
            elif op == "reduce_scatter":
                big = torch.randn(world * rows, a.cols, device=dev).to(dtype)
                res = torch.empty(rows, a.cols, dtype=dtype, device=dev)
                if on_gpu:
                    fn = lambda: dist.reduce_scatter_tensor(res.view(-1), big.view(-1))
                else:       # gloo has no reduce-scatter: all-reduce of the whole buffer stands in
                    fn = lambda: dist.all_reduce(big)
            elif op == "all_reduce":
                fn = lambda: dist.all_reduce(x)
            elif op == "all_to_all":
                out = torch.empty_like(x)
                if on_gpu:
                    fn = lambda: dist.all_to_all_single(out.view(-1), x.view(-1))
                else:       # gloo: the same exchange as pairwise sends
                    def fn():
                        parts_in, parts_out = list(x.view(world, -1)), list(out.view(world, -1))
                        works = [dist.isend(parts_in[p].contiguous(), p) for p in range(world) if p != rank]
                        for p in range(world):
                            if p != rank:
                                dist.recv(parts_out[p], p)
                        for w in works:
                            w.wait()
            else:
                if fused is None:
                    continue
                def fn():
                    fused.all_gather_rows(x)
                    fused.release_gather()
            ms = _time(fn, a.iters, a.warmup, dev, flush)
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            if rank == 0:
                print(json.dumps({"kernel": "net_sweep", "op": op, "world": world, "bytes_per_rank": nbytes, "ms": ms,
                                  "bus_gbs": bus_bytes(op, world, nbytes) / ms / 1e6 if ms > 0 else None,
                                  "timing": "cuda events" if on_gpu else "wall clock"}), flush=True)
            del x
    if fused is not None:
        if on_gpu:
            from ..ops import _lib
            _lib.check_status(dev, "net_bench")
        fused.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
