"""The per-document context-parallel baseline (all-gather K/V, two query chunks per document and rank,
reduce-scatter of dK/dV; the reference's comparison point, baseline/wlbllm_original/wlbllm/per_doc_cp_attn.py:
117-304, 454-475): gloo ranks must reproduce the loss and the gradients of one process holding the whole batch."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from distca_b200.models.config import PRESETS, ParallelConfig, TrainConfig
from distca_b200.parallel.percp import percp_layout, perseq_layout, round_documents


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_layout_covers_every_token_once_and_balances_causal_work():
    docs, W = [96, 32, 160], 4
    seen = {}
    work = []
    for r in range(W):
        rows, pairs = 0, 0
        for d, a, b, row0 in percp_layout(docs, W, r):
            assert row0 == rows
            rows += b - a
            for t in range(a, b):
                assert (d, t) not in seen
                seen[(d, t)] = r
                pairs += t + 1
        assert rows == sum(docs) // W
        work.append(pairs)
    assert len(seen) == sum(docs)
    assert max(work) == min(work)            # head + tail chunks: identical causal work on every rank
    assert round_documents([100, 30, 158], 4) == [96, 32, 160]


def test_per_sequence_layout_balances_tokens_but_not_work():
    docs, W, S = [200, 56, 256, 128, 128], 2, 256              # three packed sequences of 256 tokens
    seen, work = {}, []
    for r in range(W):
        rows, pairs = 0, 0
        for d, a, b, row0 in perseq_layout(docs, W, r, S):
            assert row0 == rows and 0 <= a < b <= docs[d]
            rows += b - a
            for t in range(a, b):
                assert (d, t) not in seen
                seen[(d, t)] = r
                pairs += t + 1
        assert rows == sum(docs) // W
        work.append(pairs)
    assert len(seen) == sum(docs) and max(work) > min(work)      # document boundaries fall inside chunks
    # a sequence that is one document: the same chunks as per-document CP
    assert perseq_layout([256], 2, 1, 256) == percp_layout([256], 2, 1)


def _worker(rank, world, port, q, mode="percp"):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                          LOCAL_RANK=str(rank))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from distca_b200.models.llama import Batch, LlamaModel, LocalCoreAttention
        from distca_b200.ops.attention import AttnPlan, AttnTasks
        from distca_b200.runtime.trainer import SpanHostBatch, Trainer
        cfg = PRESETS["tiny"]
        docs = [1200, 400, 16, 432]                         # multiples of 2 x world; 2048 tokens, 1024 per rank
        toks = torch.from_numpy(np.random.default_rng(5).integers(0, cfg.vocab, size=sum(docs), dtype=np.int64))
        hb = SpanHostBatch(docs, toks)
        par = ParallelConfig(tp=1, pp=1, dp=world)
        out = {}
        for rc in ("full", "keep_attn"):
            tc = TrainConfig(cad=False, recompute=rc, lm_head_chunk=2048, lr=0.0)
            tc.extra["baseline_mode"] = mode
            tc.extra["cp_seq_len"] = sum(docs)            # per-sequence CP: the whole batch is one packed sequence
            tr = Trainer(cfg, par, tc, device="cpu", seed=0)
            loss = tr.train_step(hb)
            g = tr.model.store.grad.clone()
            dist.all_reduce(g)
            out[rc] = (loss, g)
        ref = LlamaModel(cfg, "cpu", recompute="full", lm_head_chunk=2048, seed=0, pad_params_to=world)
        labels = torch.roll(toks, -1)
        labels[np.cumsum(docs) - 1] = -100
        pos = torch.cat([torch.arange(L, dtype=torch.int32) for L in docs])
        ca = LocalCoreAttention(cfg)
        ca.set_batch(AttnPlan(AttnTasks.from_doc_lens(docs), "cpu", need_backward=False))
        ref.store.zero_grad()
        ref_loss, _ = ref.forward_backward(Batch(toks, labels, pos, hb.num_valid_global), ca)
        ok, worst = True, (0.0, 0.0)
        for rc, (loss, g) in out.items():
            dl = abs(loss - ref_loss.item())
            dg = (g - ref.store.grad).abs().max().item()
            ok = ok and dl < 1e-5 and dg < 1e-5 * max(1.0, ref.store.grad.abs().max().item())
            worst = (max(worst[0], dl), max(worst[1], dg))
        q.put((rank, ok, worst))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        import traceback
        q.put((rank, False, repr(e) + traceback.format_exc()))


@pytest.mark.parametrize("world,mode", [(2, "percp"), (4, "percp"), (2, "perseq")])
def test_per_document_cp_matches_single_process(world, mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=600) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for r in results:
        assert r[1], f"rank result {r}"
