"""Single-kernel micro-benchmarks (also the workloads of the committed ncu summaries); the counterpart of
the reference's profiling jobs (distca/profiling/modal-scripts/attn-prof.py:20-99, get_attn_data.py).

    python -m distca_b200.utils.kernel_bench --kernel gemm --m 8192 --n 6144 --k 4096
    python -m distca_b200.utils.kernel_bench --kernel attn_fwd --seqlen 16384
    python -m distca_b200.utils.kernel_bench --kernel attn_bwd --seqlen 16384

Each run warms up, times ``--iters`` launches with CUDA events on the launching stream (inputs
are larger than L2 or an L2-sized buffer is overwritten between launches) and prints one JSON line
with achieved TFLOP/s (or GB/s) and the fraction of the measured peak when the peaks file is present.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks(a):
    """Roofline denominators: ``--hbm-gbs`` / ``--bf16-tflops`` when given, else a peaks file (``--peaks-file``
    or ``MEASURED_PEAKS.json`` in the working directory), else an earlier measurement of the same GPU type."""
    if a.hbm_gbs and a.bf16_tflops:
        return {"hbm_gbs": a.hbm_gbs, "bf16_tflops": a.bf16_tflops}, "arguments"
    p = a.peaks_file or "MEASURED_PEAKS.json"
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": a.hbm_gbs or d["hbm_gbs"], "bf16_tflops": a.bf16_tflops or d["bf16_tflops"]}, "measured"
    return {"hbm_gbs": a.hbm_gbs or 6650.0, "bf16_tflops": a.bf16_tflops or 1590.0}, "fallback"


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


MEMORY_BOUND = ["rmsnorm", "rmsnorm_bwd", "swiglu_bwd", "add", "rope", "rope_bwd", "ce", "adam", "embedding",
                "embedding_bwd", "scatter_rows", "sum_slots", "attn_delta", "zero"]


def _memory_bound_case(name: str, a, dev):
    """(callable, algorithmic bytes per call, shape) of one memory-bound kernel at the shapes of a
    ``--tokens`` x ``--hidden`` training step (defaults: Llama-3-8B, 128K tokens)."""
    from ..ops import attention as A, elementwise as ew
    from ..parallel import p2p
    T, H, F, V = a.tokens, a.hidden, a.ffn, a.vocab
    Hq, Hkv, D = a.heads_q, a.heads_kv, 128
    bf = torch.bfloat16
    if name == "rmsnorm":
        x = torch.randn(T, H, device=dev).to(bf); g = torch.ones(H, device=dev, dtype=bf); y = torch.empty_like(x)
        return (lambda: ew.rmsnorm_fwd(x, g, 1e-5, out=y)), 2.0 * T * H * 2, [T, H]
    if name == "rmsnorm_bwd":
        x = torch.randn(T, H, device=dev).to(bf); g = torch.ones(H, device=dev, dtype=bf)
        dy = torch.randn(T, H, device=dev).to(bf); dres = torch.randn(T, H, device=dev).to(bf)
        _, rstd = ew.rmsnorm_fwd(x, g, 1e-5)
        dg = torch.zeros(H, device=dev, dtype=bf); dx = torch.empty_like(x)
        return (lambda: ew.rmsnorm_bwd(x, g, rstd, dy, dg, dres=dres, dx_out=dx)), 4.0 * T * H * 2, [T, H]
    if name == "swiglu_bwd":
        pre = torch.randn(T, 2 * F, device=dev).to(bf); dact = torch.randn(T, F, device=dev).to(bf)
        out = torch.empty_like(pre)
        def fn():
            rc = _swiglu_bwd_out(pre, dact, out)
        return fn, 5.0 * T * F * 2, [T, F]
    if name == "add":
        x = torch.randn(T, H, device=dev).to(bf); y = torch.randn(T, H, device=dev).to(bf)
        return (lambda: ew.add_(x, y)), 3.0 * T * H * 2, [T, H]
    if name in ("rope", "rope_bwd"):
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device=dev).to(bf)
        pos = (torch.arange(T, device=dev) % 65536).int()
        table = ew.rope_table(65536, D, 500000.0, dev)
        return (lambda: ew.rope_(qkv, pos, table, Hq, Hkv, D, backward=name == "rope_bwd")), \
            2.0 * T * (Hq + Hkv) * D * 2, [T, Hq, Hkv]
    if name == "ce":
        Tc = min(T, 8192)          # the LM head runs in token chunks of this size
        logits = torch.randn(Tc, V, device=dev); lab = torch.randint(0, V, (Tc,), device=dev)
        dl = torch.empty(Tc, V, device=dev, dtype=bf)
        def fn():
            st = ew.ce_stats(logits, lab)
            ew.ce_grad(logits, lab, st, 1.0, dlogits=dl)
        return fn, Tc * V * (4.0 + 4.0 + 2.0), [Tc, V]
    if name == "adam":
        n = a.flat_elems
        p = torch.randn(n, device=dev).to(bf); lo = torch.zeros(n, device=dev, dtype=torch.int16)
        g = torch.randn(n, device=dev).to(bf); m = torch.zeros(n, device=dev); v = torch.zeros(n, device=dev)
        return (lambda: ew.adam_step_(p, lo, g, m, v, lr=1e-5, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.01,
                                      step=1)), n * (2 + 2 + 2 + 8 + 2 + 2 + 8.0), [n]
    if name in ("embedding", "embedding_bwd"):
        ids = torch.randint(0, V, (T,), device=dev); tab = torch.randn(V, H, device=dev).to(bf)
        if name == "embedding":
            return (lambda: ew.embedding_fwd(ids, tab)), 2.0 * T * H * 2, [T, H]
        dout = torch.randn(T, H, device=dev).to(bf); dt = torch.zeros(V, H, device=dev, dtype=bf)
        return (lambda: ew.embedding_bwd(ids, dout, dt)), 3.0 * T * H * 2, [T, H]
    if name == "scatter_rows":
        src = torch.randn(T, H, device=dev).to(bf); dst = torch.empty_like(src)
        perm = torch.randperm(T, device=dev)
        addr = (dst.data_ptr() + perm * (H * 2)).to(torch.int64)
        return (lambda: p2p.scatter_rows(src, H * 2, addr)), 2.0 * T * H * 2, [T, H]
    if name == "sum_slots":
        C, kd2 = 2, 2 * Hkv * D
        slots = torch.randn(C, T, kd2, device=dev).to(bf); valid = torch.zeros(T, C, dtype=torch.int32, device=dev)
        out = torch.empty(T, (Hq + 2 * Hkv) * D, device=dev, dtype=bf)
        return (lambda: p2p.sum_slots(slots, valid, out[:, Hq * D:])), (C + 1.0) * T * kd2 * 2, [C, T, kd2]
    if name == "attn_delta":
        o = torch.randn(T, Hq, D, device=dev).to(bf); do = torch.randn(T, Hq, D, device=dev).to(bf)
        return (lambda: A.attn_delta_rows(o, do)), 2.0 * T * Hq * D * 2, [T, Hq, D]
    if name == "zero":
        z = torch.empty(a.flat_elems, device=dev, dtype=bf)
        return (lambda: z.zero_()), 2.0 * a.flat_elems, [a.flat_elems]
    raise ValueError(name)


def _swiglu_bwd_out(pre, dact, out):
    from ..ops import _lib
    T, F2 = pre.shape
    rc = _lib.lib().dca_swiglu_bwd(_lib.ptr(pre), _lib.ptr(dact), _lib.ptr(out), _lib.c_long(T), _lib.c_int(F2 // 2),
                                   _lib.stream_ptr())
    _lib.check_rc(rc, "swiglu_bwd")


def _attn_sweep(a, dev, flush, peaks, src) -> None:
    """Forward and backward time over (document length x documents) workloads, one JSON line each, then the
    least-squares fit ``ms = a * tile_pairs + b * query_tiles`` of forward + backward: the constants of the
    planner's cost model (``distca_b200.planner.default_cost_model``) and the attention table of its time
    model come from this table. The reference's counterpart is its FlashAttention latency profile
    (distca/profiling/modal-scripts/attn-prof.py:20-99 -> distca/profiling/data/compute-attn-H100.csv)."""
    import numpy as np
    from ..ops import _lib, attention as A
    Hq, Hkv, D = a.heads_q, a.heads_kv, 128
    cases = [(2048, 16), (4096, 8), (8192, 1), (8192, 4), (16384, 1), (32768, 1), (65536, 1), (131072, 1)]
    X, y = [], []
    for L, docs in cases:
        T = L * docs
        q = torch.randn(T, Hq, D, device=dev).bfloat16()
        k = torch.randn(T, Hkv, D, device=dev).bfloat16()
        v = torch.randn(T, Hkv, D, device=dev).bfloat16()
        tasks = A.AttnTasks.from_doc_lens([L] * docs)
        plan = A.AttnPlan(tasks, dev)
        o, lse = torch.empty_like(q), torch.empty(T, Hq, device=dev)
        do = torch.randn_like(q)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        iters = 1 if L >= 65536 else a.iters
        f = _time(lambda: A.flash_fwd(q, k, v, plan, out=o, lse=lse), iters, 1 if L >= 65536 else a.warmup, flush)
        b = _time(lambda: A.flash_bwd(q, k, v, o, lse, do, plan, dq=dq, dk=dk, dv=dv), iters, 1, flush)
        n = L // 128
        pairs, qtiles = docs * n * (n + 1) // 2, docs * n
        fl = tasks.flops_fwd(Hq, D)
        print(json.dumps({"kernel": "attn_sweep", "seqlen": L, "docs": docs, "fwd_ms": f, "bwd_ms": b,
                          "fwd_tflops": fl / f / 1e9, "bwd_tflops_2p5x": 2.5 * fl / b / 1e9,
                          "tile_pairs": pairs, "query_tiles": qtiles, "peak_source": src}))
        X.append([pairs, qtiles]); y.append(f + b)
        del q, k, v, o, do, dq, dk, dv
        torch.cuda.empty_cache()
    _lib.check_status()
    X, y = np.asarray(X, dtype=np.float64), np.asarray(y)
    w = 1.0 / y                                   # relative error: every workload counts alike
    coef, *_ = np.linalg.lstsq(X * w[:, None], y * w, rcond=None)
    pred = X @ coef
    print(json.dumps({"kernel": "attn_sweep_fit", "heads_q": Hq, "ms_per_tile_pair": float(coef[0]),
                      "ms_per_q_tile": float(coef[1]),
                      "max_rel_err": float(np.max(np.abs(pred - y) / y))}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True,
                    choices=["gemm", "gemm_dgrad", "gemm_wgrad", "gemm_swiglu", "attn_fwd", "attn_bwd", "attn_sweep",
                             *MEMORY_BOUND, "memory_bound"],
                    help="memory_bound: every kernel of the elementwise / loss / optimizer / row-copy family, one line each")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=6144)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--seqlen", type=int, default=16384)
    ap.add_argument("--docs", type=int, default=1)
    ap.add_argument("--heads-q", type=int, default=32)
    ap.add_argument("--heads-kv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=131072, help="rows of the memory-bound kernels")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=128256)
    ap.add_argument("--flat-elems", type=int, default=1 << 30, help="elements of the optimizer / memset cases")
    ap.add_argument("--hbm-gbs", type=float, default=0.0, help="copy bandwidth to report fractions against")
    ap.add_argument("--bf16-tflops", type=float, default=0.0, help="bf16 GEMM throughput to report fractions against")
    ap.add_argument("--peaks-file", default=None, help="JSON with hbm_gbs and bf16_tflops")
    a = ap.parse_args()
    from ..ops import _lib, attention as A, elementwise as ew, gemm
    dev = "cuda"
    torch.manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    peaks, src = _peaks(a)
    out = {"kernel": a.kernel}
    if a.kernel == "attn_sweep":
        _attn_sweep(a, dev, flush, peaks, src)
        return
    if a.kernel.startswith("gemm"):
        M, N, K = a.m, a.n, a.k
        x = torch.randn(M, K, device=dev).bfloat16()
        w = torch.randn(N, K, device=dev).bfloat16()
        dy = torch.randn(M, N, device=dev).bfloat16()
        if a.kernel == "gemm":
            y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            fn = lambda: gemm.linear_fwd(x, w, out=y)
        elif a.kernel == "gemm_dgrad":
            dx = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
            fn = lambda: gemm.linear_dgrad(dy, w, out=dx)
        elif a.kernel == "gemm_wgrad":
            dw = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
            fn = lambda: gemm.linear_wgrad(dy, x, out=dw)
        else:
            fn = lambda: gemm.linear_swiglu_fwd(x, w, keep_preact=False)
        ms = _time(fn, a.iters, a.warmup, flush)
        tf = 2.0 * M * N * K / ms / 1e9
        out.update(shape=[M, N, K], ms=ms, tflops=tf, frac_of_peak=tf / peaks["bf16_tflops"], peak_source=src)
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        L, Hq, Hkv, D = a.seqlen, a.heads_q, a.heads_kv, 128
        T = L * a.docs
        q = torch.randn(T, Hq, D, device=dev).bfloat16()
        k = torch.randn(T, Hkv, D, device=dev).bfloat16()
        v = torch.randn(T, Hkv, D, device=dev).bfloat16()
        tasks = A.AttnTasks.from_doc_lens([L] * a.docs)
        plan = A.AttnPlan(tasks, dev)
        o = torch.empty_like(q)
        lse = torch.empty(T, Hq, device=dev)
        fl = tasks.flops_fwd(Hq, D)
        if a.kernel == "attn_fwd":
            fn = lambda: A.flash_fwd(q, k, v, plan, out=o, lse=lse)
        else:
            A.flash_fwd(q, k, v, plan, out=o, lse=lse)
            do = torch.randn_like(q)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            fn = lambda: A.flash_bwd(q, k, v, o, lse, do, plan, dq=dq, dk=dk, dv=dv)
            fl *= 2.5
        ms = _time(fn, a.iters, a.warmup, flush)
        tf = fl / ms / 1e9
        out.update(seqlen=L, docs=a.docs, heads=[Hq, Hkv], ms=ms, tflops=tf,
                   frac_of_peak=tf / peaks["bf16_tflops"], peak_source=src)
    else:
        names = MEMORY_BOUND if a.kernel == "memory_bound" else [a.kernel]
        for name in names:
            fn, nbytes, shape = _memory_bound_case(name, a, dev)
            ms = _time(fn, a.iters, a.warmup, flush)
            gbs = nbytes / ms / 1e6
            rec = {"kernel": name, "shape": shape, "ms": ms, "algorithmic_gb": nbytes / 1e9, "gbs": gbs,
                   "frac_of_peak": gbs / peaks["hbm_gbs"], "peak_source": src}
            if name != names[-1]:
                print(json.dumps(rec))
            out = rec
            del fn
            torch.cuda.empty_cache()
    _lib.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
