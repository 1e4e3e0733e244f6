"""Host side of the GPU core-attention runtime without a GPU: ``CadRuntime.plan_step`` turns a plan
into address tables (peer base + region offset + row * pitch). Here every rank gets a fake arena in
its own address range and the tables are decoded back: each address must point at the region, rank
and row that holds (or must receive) the very token it is meant for."""
import numpy as np
import torch

from distca_b200.ops import attention as attn_ops
from distca_b200.parallel.cad import CadRuntime
from distca_b200.planner import Planner, PlannerConfig

K = 1024
SPACE = 1 << 40


class _FakeArena:
    def __init__(self, world):
        self.base = [(r + 1) * SPACE for r in range(world)]


def _runtime(me, world, T, hq=4, hkv=2, D=128):
    rt = object.__new__(CadRuntime)
    rt.me, rt.W, rt.device = me, world, torch.device("cpu")
    rt.hq, rt.hkv, rt.D = hq, hkv, D
    rt.qd, rt.kd = hq * D, hkv * D
    rt.qkvd = rt.qd + 2 * rt.kd
    rt.q_bytes, rt.kv_bytes = rt.qd * 2, rt.kd * 2
    rt.T, rt.arena = T, _FakeArena(world)
    rt.max_q, rt.max_kv = 2 * T, world * T
    sizes = {"Qr": rt.max_q * rt.q_bytes, "Kr": rt.max_kv * rt.kv_bytes, "Vr": rt.max_kv * rt.kv_bytes,
             "dOr": rt.max_q * rt.q_bytes, "DELTAr": rt.max_q * hq * 4, "LSE": rt.max_q * hq * 4,
             "AO": T * rt.q_bytes, "LSEo": T * hq * 4, "DQKV": T * rt.qkvd * 2, "SLOTS": world * T * 2 * rt.kv_bytes}
    rt.off, cur = {}, 4096
    for k, v in sizes.items():
        rt.off[k] = cur
        cur += v + 16 * 1024
    rt.sizes = sizes
    rt.plan_stats, rt.last_plan = {}, None
    import threading
    rt.use_cost_model, rt.speed_feedback, rt._plan_lock, rt._pending_speed = False, False, threading.Lock(), None
    return rt


def _decode(rt, addr):
    rank = int(addr) // SPACE - 1
    rel = int(addr) % SPACE
    for name, off in rt.off.items():
        if off <= rel < off + rt.sizes[name]:
            return rank, name, rel - off
    raise AssertionError(f"address {addr} outside every region")


import pytest


@pytest.mark.parametrize("layout", ["fixed", "span"])
def test_address_tables_point_at_the_right_rows(layout):
    world, T = 4, 8 * K
    p = Planner(PlannerConfig(world=world, tokens_per_rank=T, tolerance=0.05))
    if layout == "fixed":
        docs = [[8 * K], [4 * K, 4 * K], [2 * K] * 4, [1 * K] * 8]
        plan = p.plan_fixed(docs)
    else:   # one document of 20K tokens spans three ranks as head / tail pieces
        docs = None
        plan = p.plan([[20 * K, 4 * K], [2 * K] * 4])
    rts = []
    for r in range(world):
        rt = _runtime(r, world, T)
        rt.plan_step(docs, plan=plan)
        rts.append(rt)
    # identity of every token on its owner
    ident = []
    for r in range(world):
        tok = np.zeros((T, 2), dtype=np.int64)
        for doc, a, b, row0 in plan.rank(r).layout:
            tok[row0:row0 + (b - a)] = np.stack([np.full(b - a, doc), np.arange(a, b)], 1)
        ident.append(tok)
    # ---- owner side: Q, delta and statistics of token t go to the same row of the same server ----
    q_at = [dict() for _ in range(world)]      # server -> {q row: (doc, pos)}
    for r, rt in enumerate(rts):
        for t in range(0, T, 37):
            s, reg, byte = _decode(rt, rt.q_dst[t])
            assert reg == "Qr" and byte % rt.q_bytes == 0
            row = byte // rt.q_bytes
            assert _decode(rt, rt.delta_dst[t]) == (s, "DELTAr", row * rt.hq * 4)
            assert _decode(rt, rt.lse_dst[t]) == (s, "LSE", row * rt.hq * 4)
            q_at[s][row] = tuple(ident[r][t])
            for c in range(rt.copies):
                a = int(rt.kv_dst[t, c])
                if a:
                    ks, kreg, kbyte = _decode(rt, a)
                    assert kreg == "Kr" and kbyte % rt.kv_bytes == 0 and int(rt.kv_valid[t, c]) == ks
                else:
                    assert int(rt.kv_valid[t, c]) < 0
    # ---- server side: outputs, statistics and gradients go back to the row the query came from ----
    for s, rt in enumerate(rts):
        w = attn_ops.forward_work(rt.attn_plan.tasks)
        fw = np.frombuffer(rt.fwd_work.numpy().tobytes(), dtype=w.dtype)
        assert len(fw) == len(w)
        for tile in fw[::3]:
            owner, reg, byte = _decode(rt, tile["out_ptr"])
            assert reg == "AO" and byte % rt.q_bytes == 0
            orow = byte // rt.q_bytes
            assert _decode(rt, tile["lse_ptr"]) == (owner, "LSEo", orow * rt.hq * 4)
            qrow = int(tile["q_row0"])
            assert _decode(rt, rt.q_ret[qrow]) == (owner, "DQKV", orow * rt.qkvd * 2)
            if qrow in q_at[s]:
                assert q_at[s][qrow] == tuple(ident[owner][orow])       # the row really holds that token's query
        slot_bytes = T * 2 * rt.kv_bytes
        for krow in range(0, rt.kv_rows, 53):
            owner, reg, byte = _decode(rt, rt.kv_ret[krow])
            assert reg == "SLOTS"
            slot, rest = divmod(byte, slot_bytes)
            assert rest % (2 * rt.kv_bytes) == 0
            orow = rest // (2 * rt.kv_bytes)
            assert int(rts[owner].kv_valid[orow, slot]) == s            # the owner expects this server in that slot


def test_tables_built_on_a_worker_thread_equal_the_direct_ones():
    from concurrent.futures import ThreadPoolExecutor
    from distca_b200.models.config import TrainConfig
    world, T = 4, 8 * K
    docs = [[8 * K], [4 * K, 4 * K], [2 * K] * 4, [1 * K] * 8]
    direct, ahead = _runtime(1, world, T), _runtime(1, world, T)
    for rt in (direct, ahead):
        rt.planner = Planner(PlannerConfig(world=world, tokens_per_rank=T, tolerance=0.05))
        rt.tcfg, rt.capacity_hint = TrainConfig(), 0
    direct.plan_step(docs)
    with ThreadPoolExecutor(max_workers=1) as pool:
        def work():
            plan = ahead.make_plan(docs)
            return plan, ahead.make_tables(plan)
        plan, tables = pool.submit(work).result()
    ahead.plan_step(docs, plan=plan, tables=tables)
    for name in ("q_dst", "delta_dst", "lse_dst", "kv_dst", "kv_valid", "fwd_work", "q_ret", "kv_ret"):
        assert torch.equal(getattr(direct, name), getattr(ahead, name)), name
    assert direct.plan_stats == ahead.plan_stats and direct.Tcur == ahead.Tcur == T
    assert np.array_equal(direct.attn_plan.bwd_qt_host, ahead.attn_plan.bwd_qt_host)


def test_feedback_shares_move_work_towards_idle_servers():
    """One step's measurements -> next step's shares of the attention work: a server that idled less than the
    others (its other kernels ran slower) or that needed longer for the same predicted work gets a smaller share."""
    import numpy as np
    even = CadRuntime.feedback_shares([100] * 4, [100] * 4, [10] * 4)
    assert np.allclose(even, 1.0)
    slow_gemms = CadRuntime.feedback_shares([100] * 4, [100] * 4, [10, 10, 10, 0])
    assert slow_gemms[3] < 0.98 and np.all(slow_gemms[:3] > 1.0) and abs(slow_gemms.mean() - 1.0) < 1e-9
    slow_attention = CadRuntime.feedback_shares([100, 100, 100, 125], [100] * 4, [20, 20, 20, 0])
    assert slow_attention[3] < slow_gemms[3]
    assert np.all(CadRuntime.feedback_shares([1, 1, 1, 100], [1] * 4, [0] * 4) >= 0.75)      # bounded


def test_blocking_report_names_the_waits_that_kept_the_stream_idle():
    """The wait report (the reference's TickSync blocking detection): one record per signal wait above the
    threshold, with the wait's name and its index among the step's waits of that name (the layer)."""
    from distca_b200.parallel.cad import CadRuntime
    waits = [("qkv", 0.02), ("out", 0.4), ("qkv", 3.5), ("out", 0.1), ("dout", 1.2), ("dqkv", 0.0), ("dout", 0.9)]
    rep = CadRuntime.blocking_report(waits, threshold_ms=1.0, step=7)
    assert rep == [{"step": 7, "wait": "qkv", "index": 1, "ms": 3.5}, {"step": 7, "wait": "dout", "index": 0, "ms": 1.2}]
    assert CadRuntime.blocking_report(waits, threshold_ms=10.0) == []
    assert CadRuntime.blocking_report([], threshold_ms=0.0) == []


def test_end_of_step_feedback_with_stand_in_events(monkeypatch):
    """The bookkeeping of one step's attention / wait events (CUDA events on a GPU, stand-ins with a fake clock
    here): measured and idle time reach the planner's shares through the group collective, the wait report keeps
    the waits above its threshold, and the per-step lists are emptied."""
    import torch.distributed as dist

    class Ev:
        clock = [0.0]
        step = [1.0]

        def __init__(self, enable_timing=False):
            self.t = None

        def record(self, stream=None):
            Ev.clock[0] += Ev.step[0]
            self.t = Ev.clock[0]

        def elapsed_time(self, other):
            return other.t - self.t

    monkeypatch.setattr(torch.cuda, "Event", Ev)
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29733", rank=0, world_size=1)
    try:
        rt = _runtime(0, 1, 1024)
        rt.use_cost_model = rt.speed_feedback = True
        rt.group, rt.speed, rt.predicted_ms, rt._predicted_ms = dist.group.WORLD, None, 80.0, 0.0
        rt._attn_events, rt._wait_events, rt.blocking_events, rt._steps_seen = [], [], [], 0
        rt.wait_report_ms = 10.0
        for layer in range(3):
            Ev.step[0] = 0.5 if layer != 1 else 25.0            # the wait of layer 1 keeps the stream idle for 25 ms
            with rt._timed_wait("qkv"):
                pass
            Ev.step[0] = 30.0
            with rt._timed_attention(0.25):
                pass
        rt.end_of_step_feedback()
        assert rt.blocking_events == [{"step": 1, "wait": "qkv", "index": 1, "ms": 25.0}]
        assert rt._attn_events == [] and rt._wait_events == [] and rt._predicted_ms == 0.0
        assert rt.plan_stats["attention_ms_per_server"] == [90.0] and rt.plan_stats["idle_ms_per_server"] == [26.0]
        assert rt.plan_stats["speed"] == [1.0] and rt._pending_speed == [1.0]
        rt.wait_report_ms = None                                  # off: events are still consumed, nothing is recorded
        with rt._timed_wait("out"):
            pass
        with rt._timed_attention(1.0):
            pass
        rt.end_of_step_feedback()
        assert len(rt.blocking_events) == 1 and rt._steps_seen == 2
    finally:
        if created:
            dist.destroy_process_group()
