"""Failure detection without touching a GPU: a rank that never joins, a rank that dies between
steps, a step that hangs, a plan that cannot fit the communication arena."""
import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from distca_b200.planner import Planner, PlannerConfig
from distca_b200.utils.watchdog import Heartbeat, StepWatchdog


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_watchdog_fires_and_cancels():
    hit = []
    with StepWatchdog(0.2, on_timeout=lambda: hit.append(1)):
        time.sleep(0.5)
    assert hit == [1]
    hit.clear()
    with StepWatchdog(5.0, on_timeout=lambda: hit.append(1)):
        pass
    time.sleep(0.1)
    assert hit == []


def _hb_worker(rank, world, port, q):
    try:
        store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
        hb = Heartbeat(store, rank, world)
        if rank == 1:
            for _ in range(3):          # beats for a while, then stops (it "died" between steps)
                hb.beat()
                time.sleep(0.1)
            q.put((rank, "stopped"))
            time.sleep(3.0)
            return
        dead = []
        t0 = time.time()
        while time.time() - t0 < 5.0 and not dead:
            hb.beat()
            dead = hb.dead_ranks(stale_after_s=0.8)
            time.sleep(0.1)
        q.put((rank, dead))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))


def test_heartbeat_reports_lost_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_hb_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert res[1] == "stopped" and res[0] == [1]


def _timeout_worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        t = torch.ones(4)
        dist.all_reduce(t)               # both ranks: fine
        if rank == 1:
            q.put((rank, "left"))        # leaves between steps, never joins the next collective
            time.sleep(8)
            return
        t0 = time.time()
        try:
            dist.all_reduce(t)           # must end with an error, not hang
            q.put((rank, "no error"))
        except Exception as e:
            q.put((rank, ("error", time.time() - t0, type(e).__name__)))
    except Exception as e:  # pragma: no cover
        q.put((rank, repr(e)))


def test_collective_times_out_cleanly_when_a_rank_leaves():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_timeout_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert res[1] == "left"
    assert res[0][0] == "error" and res[0][1] < 20.0


def test_plan_that_cannot_fit_is_reported():
    p = Planner(PlannerConfig(world=2, tokens_per_rank=8192, max_q_rows=100, max_kv_rows=100))
    plan = p.plan_fixed([[8192], [4096, 4096]])
    assert not plan.fits


def _guard_worker(rank, world, port, q):
    """Two ranks train one step together; rank 1 then stops (its heartbeat thread ends, as when the process
    dies between steps). Rank 0's next ``train_step`` must raise on the host before launching anything."""
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank), DISTCA_HEARTBEAT_STALE_S="1.0")
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
        from distca_b200.models.config import PRESETS, ParallelConfig, TrainConfig
        from distca_b200.runtime.trainer import BatchSource, Trainer
        from distca_b200.utils.watchdog import RankLost
        cfg = PRESETS["tiny"]
        par = ParallelConfig(tp=1, pp=1, dp=2)
        tr = Trainer(cfg, par, TrainConfig(cad=True, recompute="full", lm_head_chunk=2048), device="cpu", seed=0)
        src = BatchSource(cfg, par, 1024, "loguniform64", seed=0, pinned=False)
        loss = tr.train_step(src.next(tr.dp_rank))
        assert loss == loss
        if rank == 1:
            tr.guard.close()             # "dies" between steps: no kernel or collective of its own in flight
            q.put((rank, "left"))
            time.sleep(6)
            return
        t0 = time.time()
        res = "no error"
        while time.time() - t0 < 10.0:
            try:
                tr.guard.check()
            except RankLost:
                break
            time.sleep(0.2)
        try:
            tr.train_step(src.next(tr.dp_rank))
        except RankLost as e:
            res = ("rank lost", time.time() - t0, str(e))
        q.put((rank, res))
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, repr(e) + traceback.format_exc()))


def test_trainer_refuses_next_step_when_a_peer_stopped():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_guard_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert res[1] == "left"
    assert res[0][0] == "rank lost" and "[1]" in res[0][2], res[0]


def test_step_guard_watchdog_fires_inside_trainer_step():
    """The watchdog that both trainers arm around a step: a step that overruns calls the timeout hook."""
    from distca_b200.utils.watchdog import StepGuard
    hit = []
    g = StepGuard(step_timeout_s=0.2, on_timeout=lambda: hit.append(1))
    with g.watch():
        time.sleep(0.5)
    assert hit == [1]
    g.check()          # single process: nothing to check, must not raise
    g.close()
