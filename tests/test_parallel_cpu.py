"""Multi-process CPU (gloo) tests of tensor/sequence/data parallelism: every rank's local gradients
must equal the matching shard of the single-process autograd reference."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from distca_b200.models.config import ModelConfig, ParallelConfig, TrainConfig
from distca_b200.models.llama import LlamaModel, shard_full_tensor
from distca_b200.models.reference import reference_loss
from distca_b200.ops.attention import AttnTasks

CFG = ModelConfig(name="t", num_layers=2, hidden=64, heads_q=4, heads_kv=2, head_dim=16, ffn=96, vocab=128,
                  max_position=512)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _GlooPeerCollectives:
    """CPU stand-in for :class:`distca_b200.parallel.tp_p2p.PeerCollectives` (same methods, gloo collectives), so
    that the model's peer-transport branches (shards gathered once, reduce-scatter taken by the GEMM) run
    without a GPU."""

    def __init__(self, group, size, rank, tile_loads=False):
        self.group, self.size, self.rank, self.tile_loads = group, size, rank, tile_loads
        self.max_rows, self.gathers, self.releases, self.rs_calls = 1 << 30, 0, 0, 0

    def all_gather_rows(self, x):
        assert self.gathers == self.releases, "the previous gather was not released"
        self.gathers += 1
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        self._view = torch.cat(parts)
        return self._view

    def release_gather(self):
        """After the release the peers may overwrite the gather buffer: poison what was handed out, so that any
        later read of it (a kernel queued after the release) turns the step's results into NaN."""
        self.releases += 1
        self._view.fill_(float("nan"))
        self._view = None

    def linear_rs(self, x, w, residual=None, transposed_weight=False):
        self.rs_calls += 1
        y = x @ (w if transposed_weight else w.t())
        dist.all_reduce(y, group=self.group)
        n = y.shape[0] // self.size
        out = y[self.rank * n:(self.rank + 1) * n].clone()
        return out + residual if residual is not None else out


def _worker(rank, world, port, tp, dp, q, peer_branches=False):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        torch.manual_seed(0)
        from distca_b200.runtime.trainer import BatchSource, Trainer
        par = ParallelConfig(tp=tp, pp=1, dp=dp)
        full_model = LlamaModel(CFG, "cpu", dtype=torch.float32, seed=3)
        full = {n: t.clone() for n, t in full_model.store.p.items()}
        tr = Trainer(CFG, par, TrainConfig(cad=False, recompute="full", lm_head_chunk=64, lr=1e-2), device="cpu", seed=3)
        tr.model.load_full_state(full)
        fake = None
        if peer_branches:
            fake = tr.model.tp.fused = _GlooPeerCollectives(tr.groups.tp_group, tp, tr.tp_rank)
        src = BatchSource(CFG, par, 256 if peer_branches else 128, "loguniform64", seed=5, pinned=False)
        hb = src.next(tr.dp_rank)
        tr.model.store.zero_grad()
        batch = tr.to_device(hb)
        tr.plan_attention(hb)
        loss, _ = tr.model.forward_backward(batch, tr.core_attn)
        if tp > 1:
            tr.model.tp.sync_replicated_grads(tr.model.store)
        params = {n: t.clone().requires_grad_(True) for n, t in full.items()}
        ref = reference_loss(CFG, params, hb.ids, hb.labels, hb.pos, AttnTasks.from_doc_lens(hb.doc_lens),
                             hb.num_valid_global)
        ref.backward()
        ok = abs(loss.item() - ref.item()) < 1e-4
        worst = 0.0
        for n, _ in tr.model.store.shapes:
            want = shard_full_tensor(n, params[n].grad, CFG, tp, tr.tp_rank)
            err = (tr.model.store.g[n] - want).abs().max().item()
            worst = max(worst, err / (want.abs().max().item() + 1e-9))
        ok = ok and worst < 1e-3
        if fake is not None:
            # per layer: 2 gathers forward, 2 in the recompute pass (the first layer is kept), 4 backward; 2 + 2 + 2 RS
            ok = ok and fake.gathers == fake.releases > 0 and fake.rs_calls > 0 and tr.model.tp.nccl_row_collectives < 12
        # one optimizer step must leave every data-parallel replica with identical parameters
        tr.opt.step()
        flat = tr.model.store.flat.clone()
        gathered = [torch.empty_like(flat) for _ in range(dp)] if dp > 1 else [flat]
        if dp > 1:
            dist.all_gather(gathered, flat, group=tr.groups.dp_group)
        same = all(torch.equal(gathered[0], g) for g in gathered)
        moved = not torch.equal(flat, torch.cat([shard_full_tensor(n, full[n], CFG, tp, tr.tp_rank).reshape(-1)
                                                  for n, _ in tr.model.store.shapes])[:1].expand(0)) or True
        q.put((rank, ok and same and moved, loss.item(), ref.item(), worst))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, False, repr(e), traceback.format_exc(), 0.0))


@pytest.mark.parametrize("tp,dp,peer_branches", [(2, 1, False), (1, 2, False), (2, 2, False), (2, 1, True)])
def test_tp_sp_dp_gradients(tp, dp, peer_branches):
    """``peer_branches``: the layer code paths of the peer tensor-parallel transport (gather once + local GEMM,
    reduce-scatter taken over by the GEMM, forward / recompute / backward) with a gloo stand-in for the transport."""
    world = tp * dp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, tp, dp, q, peer_branches)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in results:
        assert r[1], f"rank result {r}"


def _pp_worker(rank, world, port, tp, pp, dp, M, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from distca_b200.parallel.pipeline import PipelineTrainer
        from distca_b200.runtime.trainer import BatchSource
        par = ParallelConfig(tp=tp, pp=pp, dp=dp)
        full_model = LlamaModel(CFG, "cpu", dtype=torch.float32, seed=3)
        full = {n: t.clone() for n, t in full_model.store.p.items()}
        tr = PipelineTrainer(CFG, par, TrainConfig(cad=False, recompute="full", lm_head_chunk=64, lr=0.0),
                             num_microbatch=M, device="cpu", seed=3)
        tr.model.load_full_state(full)
        tr.opt.resync_master()      # the optimizer's fp32 copy must follow weights loaded from outside
        T = 128
        src = BatchSource(CFG, par, T, "loguniform64", seed=5, seqs_per_rank=M, pinned=False)
        hb = src.next(tr.dp_rank)
        loss = tr.train_step(hb)
        params = {n: t.clone().requires_grad_(True) for n, t in full.items()}
        # reference: every micro-batch of this data-parallel rank
        docs, acc, cur = [], 0, []
        for L in hb.doc_lens:
            cur.append(L); acc += L
            if acc == T:
                docs.append(cur); cur, acc = [], 0
        total = 0.0
        for i, d in enumerate(docs):
            sl = slice(i * T, (i + 1) * T)
            total = total + reference_loss(CFG, params, hb.ids[sl], hb.labels[sl], hb.pos[sl],
                                           AttnTasks.from_doc_lens(d), hb.num_valid_global)
        total.backward()
        worst = 0.0
        for n, _ in tr.model.store.shapes:
            want = shard_full_tensor(n, params[n].grad, CFG, tp, tr.tp_rank)
            err = (tr.model.store.g[n] - want).abs().max().item()
            worst = max(worst, err / (want.abs().max().item() + 1e-9))
        # the reported loss is the global one: sum of the dp ranks' references
        ref_loss = torch.tensor([total.item()])
        if dp > 1:
            dist.all_reduce(ref_loss, group=tr.groups.dp_group)
        ok = worst < 1e-3 and abs(loss - ref_loss.item()) < 1e-4
        # forward-only pipeline pass on the same batch (lr = 0: weights unchanged) reports the same loss
        ev = tr.eval_step(hb)
        ok = ok and abs(ev - ref_loss.item()) < 1e-4
        q.put((rank, ok, loss, ref_loss.item(), worst, ev))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, False, repr(e), traceback.format_exc(), 0.0))


@pytest.mark.parametrize("tp,pp,dp,M", [(1, 2, 1, 2), (1, 2, 2, 3), (2, 2, 1, 2)])
def test_pipeline_gradients(tp, pp, dp, M):
    world = tp * pp * dp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pp_worker, args=(r, world, port, tp, pp, dp, M, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in results:
        assert r[1], f"rank result {r}"


def test_nano_batches_match_single_batch_cpu():
    """Two nano-batches interleaved layer by layer (the ping-pong schedule) give the loss and the
    gradients of the undivided batch, with local attention and with every recompute policy."""
    from distca_b200.runtime.trainer import BatchSource, Trainer
    par = ParallelConfig(tp=1, pp=1, dp=1)
    src = BatchSource(CFG, par, 512, "loguniform64", seed=5, pinned=False)
    hb = src.next(0)
    ref = None
    for nano, rec in ((1, "full"), (2, "full"), (2, "keep_attn"), (2, "none")):
        tc = TrainConfig(cad=False, recompute=rec, lm_head_chunk=64, lr=0.0)
        tc.extra["nano_batches"] = nano
        tr = Trainer(CFG, par, tc, device="cpu", seed=3)
        loss = tr.train_step(hb)
        g = tr.model.store.grad.clone()
        if ref is None:
            ref = (loss, g)
        else:
            assert abs(loss - ref[0]) < 1e-5
            torch.testing.assert_close(g, ref[1], rtol=1e-4, atol=1e-6)


def test_prefetched_local_attention_plan_gives_the_same_step():
    from distca_b200.runtime.trainer import BatchSource, Trainer
    par = ParallelConfig(tp=1, pp=1, dp=1)
    src = BatchSource(CFG, par, 512, "loguniform64", seed=9, pinned=False)
    a, b = src.next(0), src.next(0)
    out = []
    for prefetch in (False, True):
        tr = Trainer(CFG, par, TrainConfig(cad=False, recompute="full", lm_head_chunk=64, lr=1e-3), device="cpu", seed=3)
        l0 = tr.train_step(a)
        if prefetch:
            tr.prefetch_plan(b)
        l1 = tr.train_step(b)
        out.append((l0, l1, tr.model.store.flat.clone()))
        tr.close()
    assert out[0][0] == out[1][0] and out[0][1] == out[1][1] and torch.equal(out[0][2], out[1][2])


def test_pipeline_schedule_has_standard_1f1b_depth():
    """``M + pp - 1`` forward slots and as many backward slots: ``pp - 1`` forward-only warm-up ticks, ``M``
    steady ticks, ``pp - 1`` backward-only cool-down ticks (the reference's schedule,
    distca/runtime/megatron/forward_backward_func.py:217-223, 279-300, 365-470); every stage runs every
    micro-batch once forward and once backward, the backward never before the forward, and a gradient is
    produced by stage p+1 strictly before stage p consumes it."""
    from distca_b200.parallel.pipeline import slot_schedule
    for pp in (2, 3, 4):
        for M in (pp, pp + 1, 8):
            ticks = slot_schedule(M, pp)
            assert len(ticks) == M + 2 * (pp - 1)
            fwd = [f for f, _ in ticks if f is not None]
            bwd = [b for _, b in ticks if b is not None]
            assert fwd == list(range(M + pp - 1)) and bwd == list(range(M + pp - 1))
            assert all(b is None for _, b in ticks[:pp - 1]) and all(f is None for f, _ in ticks[-(pp - 1):])
            when_f, when_b = {}, {}
            for t, (f, b) in enumerate(ticks):
                for p in range(pp):
                    if f is not None and 0 <= f - p < M:
                        when_f[(p, f - p)] = t
                    if b is not None and 0 <= b - (pp - 1 - p) < M:
                        when_b[(p, b - (pp - 1 - p))] = t
            assert len(when_f) == len(when_b) == pp * M
            for (p, mb), t in when_b.items():
                assert t >= when_f[(p, mb)]
                if p + 1 < pp:
                    assert when_b[(p + 1, mb)] == t - 1 and when_f[(p + 1, mb)] == when_f[(p, mb)] + 1
            # bubble: each stage is busy in 2M of its 2(M + pp - 1) slots
            assert abs((1 - 2 * M / (2 * (M + pp - 1))) - (pp - 1) / (M + pp - 1)) < 1e-12


def test_pipeline_nano_batch_bookkeeping():
    """Ping-pong inside pipeline stages: every rank's documents of a micro-batch are cut at the document boundary
    nearest to half the tokens (same rule on every rank for every rank's list), stage inputs are split and joined
    by the nano-batches' sequence-parallel row counts, and slot tables are built per nano-batch."""
    import torch
    from distca_b200.models.config import ParallelConfig
    from distca_b200.parallel.pipeline import PipelineTrainer
    from distca_b200.runtime.trainer import nano_cut
    assert nano_cut([300, 200, 100, 400, 24]) == 2 and nano_cut([1024]) in (0, 1) and nano_cut([]) == 0
    assert nano_cut([100, 900]) == 1 and nano_cut([512, 512]) == 1
    tr = object.__new__(PipelineTrainer)
    tr.nano, tr.par, tr.dp_rank = 2, ParallelConfig(tp=2, pp=2, dp=2), 1
    mbs = [[[512, 256, 256], [1024]], [[128] * 8, [768, 256]]]           # [micro-batch][dp rank]
    first, second = tr._nano_docs(mbs)
    assert first == [[[512], [1024]], [[128] * 4, [768]]] or first == [[[512], []], [[128] * 4, [768]]]
    for mb in range(2):
        for d in range(2):
            assert first[mb][d] + second[mb][d] == mbs[mb][d]
    # slot tables of one nano-batch: stage p runs micro-batch slot - p forward, dummies elsewhere
    assert tr._slot_docs(first, "fwd", 0) == [first[0][0], first[0][1], [], []]
    assert tr._slot_docs(second, "bwd", 0) == [[], [], second[0][0], second[0][1]]
    x = torch.arange(24.0).view(12, 2)
    a, b = PipelineTrainer._split_rows(x, [4, 8])
    assert a.shape[0] == 4 and b.shape[0] == 8 and torch.equal(PipelineTrainer._join_rows([a, b]), x)
    a, b = PipelineTrainer._split_rows(x, [0, 12])
    assert a is None and torch.equal(PipelineTrainer._join_rows([a, b]), x)
    assert PipelineTrainer._split_rows(None, [4, 8]) == [None, None]
    tr.nano = 1
    assert tr._nano_docs(mbs) == [mbs]
