"""CPU tests of the planner-side tools and the workload-balanced packing baseline."""
import numpy as np

from distca_b200.data.wlb import balance_documents, imbalance, workload
from distca_b200.planner.tools import compare_policies, recommend_buffer_gb

K = 1024


def test_wlb_packing_balances_workload_under_token_budget():
    rng = np.random.default_rng(0)
    docs = [int(x) for x in rng.integers(1 * K, 40 * K, size=40)] + [120 * K]
    ranks, l_max = 4, 2 * sum(docs) // 4
    bins = balance_documents(docs, ranks, l_max, breakpoint=64 * K)
    assert sorted(l for b in bins for l in b) == sorted(docs)          # nothing lost or duplicated
    assert all(sum(b) <= l_max for b in bins)
    stats = imbalance(bins, breakpoint=64 * K)
    naive = [docs[i::ranks] for i in range(ranks)]
    assert stats["workload_max_over_mean"] <= imbalance(naive, 64 * K)["workload_max_over_mean"] + 1e-9
    assert stats["workload_max_over_mean"] < 1.6      # one 120K document dominates; the rest fills around it
    assert workload([64 * K], 64 * K) == 2.0          # (l/B)^2 + l/B at the breakpoint


def test_buffer_recommendation_covers_every_sampled_plan():
    rec = recommend_buffer_gb("llama3-8b", world=4, tokens=32 * K, dist="mixture", iterations=5)
    assert rec["max_q_rows"] >= 32 * K * 0.5 and rec["max_kv_rows"] >= rec["max_q_rows"] * 0.5
    assert rec["recommended_comm_buffer_gb"] >= rec["receive_arena_gb"]


def test_policy_comparison_orders_the_baselines():
    res = compare_policies("llama3-8b", world=4, tokens=32 * K, dist="mixture", iterations=5)
    t = res["attention_ms_per_layer_forward_max_over_ranks"]
    assert t["cad"] <= t["local"] * 1.001          # balancing never makes the slowest server slower
    assert t["per_document_cp"] <= t["local"] * 1.05
    mb = res["remote_mb_per_rank_per_layer"]
    assert mb["cad"] < mb["per_document_cp"]       # CP ships every long document's context to every rank


def test_text_corpus_batches(tmp_path):
    """Local corpus -> byte tokens -> sequential packing with carry-over of a cut document."""
    from distca_b200.data.text import TextBatches
    p = tmp_path / "corpus.txt"
    p.write_text("\n\n".join(("doc %d " % i) * (20 + 7 * i) for i in range(12)), encoding="utf-8")
    tb = TextBatches(str(p), tokens_per_seq=512, num_seqs=3, vocab=32000, seed=0)
    packs = tb.next_doc_lens()
    assert len(packs) == 3 and all(sum(d) == 512 for d in packs) and all(L % 16 == 0 for d in packs for L in d)
    ids, labels, pos = tb.next_tokens(packs)
    assert ids.shape == (3, 512) and int(ids.max()) < 256
    off = 0
    for L in packs[0]:
        assert pos[0, off] == 0 and pos[0, off + L - 1] == L - 1 and labels[0, off + L - 1] == -100
        off += L
    first = bytes(ids[0, :6].tolist()).decode()
    assert first == "doc 0 "


def test_launcher_builds_one_torchrun_per_node():
    from distca_b200.launch import build_commands
    cmds = build_commands(["n0", "n1"], 8, ["pretrain_llama.py", "--output-dir", "runs/{hostname}"], port=1234, workdir="/w")
    assert [n for n, _ in cmds] == ["n0", "n1"]
    assert all("--nnodes=2" in c and "--nproc-per-node=8" in c and "--master-addr n0" in c for _, c in cmds)
    assert "--node-rank=1" in cmds[1][1] and "runs/n1" in cmds[1][1] and cmds[1][1].startswith("ssh ")
    local = build_commands(["localhost"], 2, ["bench.py"])
    assert "127.0.0.1" in local[0][1] and not local[0][1].startswith("ssh")


def test_training_guards_and_memory_estimate():
    import math
    import pytest
    from distca_b200.models.config import ParallelConfig, get_model_config
    from distca_b200.utils.guards import TrainingFault, TrainingGuards, estimate_memory_gb, quit_if_maybe_oom
    g = TrainingGuards(spiky_loss_factor=2.0, large_grad_factor=10.0, warmup_steps=2)
    for i, (l, n) in enumerate([(10.0, 1.0), (9.5, 1.2), (9.0, 0.9)]):
        g.check(i, l, n)
    with pytest.raises(TrainingFault, match="loss"):
        g.check(3, 25.0, 1.0)
    with pytest.raises(TrainingFault, match="gradient norm"):
        g.check(3, 9.0, 50.0)
    with pytest.raises(TrainingFault, match="nan"):
        g.check(4, math.nan, 1.0)
    cfg = get_model_config("llama3-8b")
    one = estimate_memory_gb(cfg, ParallelConfig(1, 1, 1), 131072, cad=False)
    assert 170 < one["total"] < 186 and abs(one["optimizer"] - 80.3) < 1.0      # measured peak: 177 GB
    eight = estimate_memory_gb(cfg, ParallelConfig(1, 1, 8), 131072, cad=True, comm_buffer_gb=6.0)
    assert eight["optimizer"] < 11 and eight["attention_arena"] > 5
    with pytest.raises(TrainingFault, match="exceeds"):
        quit_if_maybe_oom(estimate_memory_gb(cfg, ParallelConfig(1, 1, 1), 262144, cad=False), 180)
    quit_if_maybe_oom(eight, 180)


def test_split_nano_cuts_at_the_document_boundary_nearest_to_half():
    import torch
    from distca_b200.runtime.trainer import HostBatch, split_nano
    docs = [300, 200, 100, 400, 24]
    T = sum(docs)
    hb = HostBatch(torch.arange(T), torch.arange(T), torch.arange(T, dtype=torch.int32), docs, [docs, [T], [8] * 128],
                   num_valid_global=99)
    a, b = split_nano(hb)
    assert a.doc_lens == [300, 200] and b.doc_lens == [100, 400, 24]
    assert a.ids.numel() == 500 and b.ids[0] == 500 and a.num_valid_global == b.num_valid_global == 99
    # every rank's list is cut by the same rule; a single document cannot be cut: one side stays empty
    assert a.all_doc_lens[1] == [] and b.all_doc_lens[1] == [T] or a.all_doc_lens[1] == [T] and b.all_doc_lens[1] == []
    assert sum(a.all_doc_lens[2]) == sum(b.all_doc_lens[2]) == T // 2


def test_layer_store_device_placement_and_metrics_sink(tmp_path):
    import json
    import torch
    from distca_b200.utils.observability import MetricsSink
    from distca_b200.utils.offload import LayerStore, choose_placements
    assert choose_placements(5, 1 << 20, "cpu", 0) == ["device"] * 5
    st = LayerStore(["device", None, "device"], "cpu")
    st.never_asked = 1
    t = torch.arange(12.0).view(3, 4)
    st.save(0, t)
    u = t * 2
    st.save(2, u, clone=False)
    assert st.has(0) and not st.has(1) and st.placement == "device: 2"
    t.zero_()
    u.zero_()
    assert st.load(0).sum() == 66 and st.load(2).sum() == 0      # slot 0 was cloned, slot 2 aliases the caller's tensor
    sink = MetricsSink(True, 0, "p", None, {}, str(tmp_path))
    sink.log({"step": 3, "loss": 1.5, "note": "text is dropped"})
    sink.close()
    files = list(tmp_path.glob("metrics.offline.jsonl"))
    if files:      # no wandb in this environment: the offline file holds the record
        assert json.loads(files[0].read_text().strip()) == {"step": 3, "loss": 1.5}


def _backward_work_loops(tasks):
    """Straightforward restatement of the backward schedule: per context, per key tile, every query tile
    whose last row reaches the tile."""
    from distca_b200.ops.attention import TILE
    by_ctx = {}
    for i, ks in enumerate(tasks.k_start):
        by_ctx.setdefault(int(ks), []).append(i)
    kv_items, qt_items = [], []
    for ks, idxs in by_ctx.items():
        ctx_len = max(int(tasks.kv_len[i]) for i in idxs)
        for k0 in range(0, ctx_len, TILE):
            begin = len(qt_items)
            for i in idxs:
                ql, kl, qs = int(tasks.q_len[i]), int(tasks.kv_len[i]), int(tasks.q_start[i])
                off = kl - ql
                for r0 in range(0, ql, TILE):
                    valid = min(TILE, ql - r0)
                    if off + r0 + valid - 1 >= k0:
                        qt_items.append((qs + r0, valid, off + r0 - k0))
            if len(qt_items) > begin:
                kv_items.append((ks + k0, min(TILE, ctx_len - k0), begin, len(qt_items)))
    return kv_items, qt_items


def test_vectorised_backward_schedule_equals_the_loops():
    from distca_b200.ops.attention import AttnTasks, backward_work
    rng = np.random.default_rng(0)
    cases = [AttnTasks.from_doc_lens([777]), AttnTasks.from_doc_lens([128, 1, 129, 4096, 300]),
             AttnTasks.from_lists([(0, 1000, 0, 1000), (1000, 1000, 0, 3000), (2000, 700, 3000, 700)]),
             AttnTasks.from_lists([(0, 5, 0, 900), (5, 130, 0, 1030), (135, 64, 2000, 64)])]
    for _ in range(20):     # random shards of random documents, several shards sharing a context
        rows, q, k = [], 0, 0
        for _d in range(rng.integers(1, 5)):
            L = int(rng.integers(1, 3000))
            cuts = sorted(set(rng.integers(1, L + 1, size=rng.integers(1, 4)).tolist()) | {L})
            a = 0
            for b in cuts:
                if rng.random() < 0.7:
                    rows.append((q, b - a, k, b))
                    q += b - a
                a = b
            k += L
        if rows:
            cases.append(AttnTasks.from_lists(rows))
    for tasks in cases:
        kv, qt = backward_work(tasks)
        kv_ref, qt_ref = _backward_work_loops(tasks)
        assert len(qt) == len(qt_ref)
        assert [tuple(int(x) for x in (r["q_row0"], r["q_valid"], r["diag"])) for r in qt] == qt_ref
        got = sorted((int(r["k_row0"]), int(r["k_valid"]), int(r["qt_begin"]), int(r["qt_end"])) for r in kv)
        assert got == sorted(kv_ref)
        sizes = [int(r["qt_end"]) - int(r["qt_begin"]) for r in kv]
        assert sizes == sorted(sizes, reverse=True)          # heaviest key tiles first


def test_layout_search_enumerates_every_factorisation_and_prefers_disaggregation_for_skewed_batches():
    from distca_b200.planner.tools import search_layouts
    res = search_layouts("llama3-8b", 8, 32768, "mixture", iterations=2)
    got = {(r["tp"], r["pp"], r["dp"]) for r in res["layouts"]}
    assert {(1, 1, 8), (2, 2, 2), (8, 1, 1), (4, 2, 1)} <= got and all(t * p * d == 8 for t, p, d in got)
    for r in res["layouts"]:
        if r["dp"] * r["pp"] > 1:
            assert r["step_ms_cad"] <= r["step_ms_local_attention"] * 1.02
        else:
            assert r["step_ms_cad"] == r["step_ms_local_attention"]       # one server: nothing to disaggregate


def test_fused_path_rooflines_name_the_binding_resource_of_every_path():
    """The bench line's roofline block: per path the slower of FLOPs at the GEMM peak, bytes over NVLink and bytes
    through HBM, against the measured phase time; a path whose phase was not timed reports no fraction."""
    from distca_b200.utils.observability import fused_path_rooflines
    peaks = {"bf16_tflops": 1400.0, "hbm_gbs": 6455.0, "link_gbs": 770.0, "source": "test"}
    steps, layers, T, H, QKV = 2, 32, 131072, 4096, 6144
    phases = {"gemm_qkv": 2 * 400.0, "re_gemm_qkv": 2 * 400.0, "cad_attn_fwd": 2 * 3000.0, "cad_attn_bwd": 2 * 8000.0,
              "optimizer": 2 * 60.0}
    attn_fwd = 2.7e15
    r = fused_path_rooflines(phases, steps, tokens_per_rank=T, hidden=H, qkv_dim=QKV, layers=layers, passes_qkv=2,
                             attn_flops_fwd_per_rank=attn_fwd, remote_dispatch_bytes=1.0e9, remote_return_bytes=0.67e9,
                             grad_bytes_in=8e9 * 2 * 7 / 8, param_bytes_out=8e9 * 2 * 7 / 8,
                             optimizer_hbm_bytes=1e9 * (2 * 8 + 20 + 16), peaks=peaks)
    assert set(r) == {"qkv_gemm_rope_dispatch", "attention_forward_with_output_return",
                      "attention_backward_with_gradient_return", "gradient_reduce_scatter_adam_all_gather"}
    q = r["qkv_gemm_rope_dispatch"]
    flops_ms = 2.0 * T * H * QKV * layers * 2 / 1400e12 * 1e3
    link_ms = 1.0e9 * layers * 2 / 770e9 * 1e3
    assert q["ms"] == 800.0 and q["bound"] == ("tensor" if flops_ms > link_ms else "nvlink")
    assert abs(q["roofline_ms"] - max(flops_ms, link_ms)) < 0.01
    assert 0 < q["fraction_of_roofline"] <= 1.0
    assert r["attention_forward_with_output_return"]["bound"] == "tensor"
    assert r["gradient_reduce_scatter_adam_all_gather"]["bound"] == "nvlink"
    # nothing timed (timers off, one GPU): no division by zero, no fraction
    empty = fused_path_rooflines({}, 1, tokens_per_rank=T, hidden=H, qkv_dim=QKV, layers=layers, passes_qkv=2,
                                 attn_flops_fwd_per_rank=0.0, remote_dispatch_bytes=0.0, remote_return_bytes=0.0,
                                 grad_bytes_in=0.0, param_bytes_out=0.0, optimizer_hbm_bytes=0.0, peaks=peaks)
    assert all(v["fraction_of_roofline"] is None for v in empty.values())


def test_step_model_reproduces_the_measured_one_gpu_step_and_orders_the_tensor_parallel_transports():
    """``predict_step_ms`` is calibrated on one measured Llama-3-8B step (one B200, 131072 tokens, keep_attn:
    17.67 s with 5.9 s of linear layers). Its parts must add up to that for such a batch, the per-tile transport
    must cost more than gather-once (a remote tile is fetched once per N tile), and the per-document CP arm exists
    exactly for the layouts without pipeline stages."""
    from distca_b200.data.synthetic import SyntheticBatches
    from distca_b200.models.config import get_model_config
    from distca_b200.planner import default_time_model
    from distca_b200.planner.tools import predict_step_ms, search_layouts
    cfg, tm = get_model_config("llama3-8b"), default_time_model("b200")
    src = SyntheticBatches(131072, 1, "mixture", 0)
    steps = [predict_step_ms(cfg, tm, src.next_doc_lens(), 131072, 1, 1, 1, 1, "local") for _ in range(10)]
    lin = steps[0]["linear_ms"]
    assert abs(lin - 5889.0) / 5889.0 < 0.03                      # measured: 2853 + 2784 + norms, SwiGLU, RoPE backward
    mean = sum(s["step_ms"] for s in steps) / len(steps)
    assert 0.8 * 17669 < mean < 1.2 * 17669, mean                # the attention share moves with the documents drawn
    for s in steps:
        parts = s["linear_ms"] + s["lm_head_ms"] + s["tp_comm_ms"] + s["attention_ms"] + s["dispatch_ms"] + s["optimizer_ms"]
        assert abs(parts - s["step_ms"]) < 1e-6
    packs = SyntheticBatches(131072, 4, "mixture", 1).next_doc_lens()
    t = {tr: predict_step_ms(cfg, tm, packs, 131072, 2, 1, 4, 1, "cad", tp_transport=tr) for tr in ("gather", "nccl", "tile")}
    assert t["gather"]["tp_comm_ms"] < t["nccl"]["tp_comm_ms"] < t["tile"]["tp_comm_ms"]
    assert t["tile"]["tp_comm_ms"] > 10 * t["gather"]["tp_comm_ms"]
    full = predict_step_ms(cfg, tm, packs, 131072, 1, 1, 4, 1, "cad", recompute="full")
    keep = predict_step_ms(cfg, tm, packs, 131072, 1, 1, 4, 1, "cad", recompute="keep_attn")
    none = predict_step_ms(cfg, tm, packs, 131072, 1, 1, 4, 1, "cad", recompute="none")
    assert full["attention_ms"] > keep["attention_ms"] == none["attention_ms"] and keep["linear_ms"] > none["linear_ms"]
    res = search_layouts("llama3-8b", 8, 32768, "mixture", iterations=1)
    for r in res["layouts"]:
        assert ("step_ms_percp" in r) == (r["pp"] == 1 and r["dp"] > 1)


def test_cpu_affinity_slices_are_disjoint_and_the_environment_record_is_written(tmp_path):
    import os
    from distca_b200.utils import affinity
    cpus = list(range(4, 68))                                      # 64 allowed CPUs, not starting at 0
    slices = [affinity.plan_affinity(r, 8, cpus) for r in range(8)]
    assert all(len(s) == 8 for s in slices) and sorted(c for s in slices for c in s) == cpus
    assert slices[3] == list(range(28, 36)) and affinity.format_cpus(slices[3]) == "28-35"
    assert affinity.plan_affinity(1, 8, cpus, per_proc=4) == [12, 13, 14, 15]
    assert affinity.plan_affinity(5, 8, [0, 1, 2]) == [2]          # fewer CPUs than ranks: shared, not an error
    assert affinity.format_cpus([0, 1, 2, 3, 8, 9, 11]) == "0-3,8-9,11"
    before = affinity.allowed_cpus()
    try:
        mine = affinity.bind(0, 1)
        assert mine == before and affinity.allowed_cpus() == before
        if len(before) >= 2:
            half = affinity.bind(1, 2)
            assert affinity.allowed_cpus() == half and len(half) == len(before) // 2
    finally:
        if hasattr(os, "sched_setaffinity"):
            os.sched_setaffinity(0, before)
    path = affinity.dump_environment(str(tmp_path), rank=3, local_rank=1)
    text = open(path).read()
    assert path.endswith(".r3.lr1.env") and "PATH=" in text and "# cpus: " in text


def test_network_model_interpolates_and_feeds_the_step_model(tmp_path):
    """Collective time tables: latency floor below the smallest measured size, linear in between, bandwidth-
    proportional above; world sizes without a table use the nearest one; a `net_bench` file replaces the built-in
    estimate of the peer-store all-gather in the step model."""
    import json
    from distca_b200.models.config import get_model_config
    from distca_b200.planner import NetworkModel, default_network_model, default_time_model
    from distca_b200.planner.tools import predict_step_ms
    from distca_b200.utils.net_bench import bus_bytes
    n = NetworkModel({("all_gather", 8): [(1e6, 0.05), (1e8, 0.5), (1e9, 4.0)]})
    assert n.ms("all_gather", 8, 1e3) == 0.05 and n.ms("all_gather", 8, 1e8) == 0.5
    assert abs(n.ms("all_gather", 8, 5.5e8) - 2.25) < 1e-9 and abs(n.ms("all_gather", 8, 2e9) - 8.0) < 1e-9
    assert n.ms("all_gather", 4, 1e8) == 0.5 and n.ms("all_gather", 1, 1e8) == 0.0
    import pytest
    with pytest.raises(KeyError):
        n.ms("all_reduce", 8, 1e6)
    d = default_network_model()
    assert 500 < d.gbytes_per_s("push", 8, 1.0384e9) < 560 and d.ms("push", 8, 1e6) == 0.145
    assert bus_bytes("all_reduce", 8, 2**30) == 2 * 2**30 * 7 / 8 and bus_bytes("all_gather", 8, 100) == 700
    # a measured sweep: slow peer stores make the gather transport slower in the prediction
    p = tmp_path / "net.jsonl"
    rows = [{"kernel": "net_sweep", "op": "push_all_gather", "world": 2, "bytes_per_rank": b, "ms": b / 100e6}
            for b in (16e6, 256e6, 1024e6)]                       # 100 GB/s
    p.write_text("hello\n" + "\n".join(json.dumps(r) for r in rows) + "\n")
    slow = NetworkModel.from_sweep(str(p))
    cfg, tm = get_model_config("llama3-8b"), default_time_model("b200")
    packs = [[131072]] * 4
    a = predict_step_ms(cfg, tm, packs, 131072, 2, 1, 2, 1, "cad")
    b = predict_step_ms(cfg, tm, packs, 131072, 2, 1, 2, 1, "cad", network=slow)
    assert b["tp_comm_ms"] > 4 * a["tp_comm_ms"] and abs((b["step_ms"] - a["step_ms"]) - (b["tp_comm_ms"] - a["tp_comm_ms"])) < 1e-6


def test_rank_excepthook_prints_clickable_frames_and_the_rank():
    import io
    import sys
    from distca_b200.utils.profiler import install_rank_excepthook
    old = sys.excepthook
    buf = io.StringIO()
    try:
        install_rank_excepthook(5, out=buf)

        def boom():
            raise ValueError("plan does not fit")
        try:
            boom()
        except ValueError:
            sys.excepthook(*sys.exc_info())
    finally:
        sys.excepthook = old
    text = buf.getvalue()
    assert "[rank 5] ValueError: plan does not fit" in text and ": in boom" in text and __file__.split("/")[-1] in text
