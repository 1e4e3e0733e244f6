"""Differential tests of the C++ planner / metadata compiler against the reference's Python planner
(distca/planner/planner.py:58-328, 627-801) and metadata compiler (distca/runtime/compute_metadata.py:642-734),
on random batches, on the CPU. The reference modules are imported from an unmodified copy of the reference
(``baseline/_ref`` or ``$DISTCA_REFERENCE_ROOT``); Megatron's ``PackedSeqParams`` dataclass, the only thing they
need from Megatron-LM, comes from ``baseline/stubs``. Skipped when no copy of the reference is present.
"""
import os
import sys
import time
from types import SimpleNamespace

import numpy as np
import pytest

from distca_b200.planner import Planner, PlannerConfig, cp_list_to_mlp_list

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_REF = os.environ.get("DISTCA_REFERENCE_ROOT", os.path.join(_REPO, "baseline", "_ref"))


def _ref():
    if not os.path.isdir(os.path.join(_REF, "distca", "planner")):
        pytest.skip("no copy of the reference planner under baseline/_ref")
    for p in (_REF, os.path.join(_REPO, "baseline", "stubs")):
        if p not in sys.path:
            sys.path.insert(0, p)
    try:
        import distca.planner.planner as P
        import distca.runtime.compute_metadata as M
    except Exception as e:  # a dependency of the reference that is absent here
        pytest.skip(f"reference planner does not import: {e!r}")
    return P, M


MC = SimpleNamespace(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8)
PAR = SimpleNamespace(pipeline_model_parallel_size=1, tensor_model_parallel_size=1)


def _random_batches(rng, world, tokens_per_rank, max_doc):
    """Sequences of ``tokens_per_rank`` tokens each, documents even and multiples of 16 (the reference's FLOPs
    conservation only holds for even lengths, distca/planner/planner.py:446-473)."""
    out = []
    for _ in range(world):
        left, docs = tokens_per_rank, []
        while left > 0:
            L = int(np.exp(rng.uniform(np.log(64), np.log(max_doc)))) // 16 * 16
            L = max(16, min(L, left))
            docs.append(L)
            left -= L
        out.append(docs)
    return out


def _mine_as_ref_tuples(items):
    out = []
    for it in items:
        (ha, hb), (ta, tb) = it["head"], it["tail"]
        if tb == ta:      # a whole document
            out.append((it["doc"], it["src"], it["dst"], ("c", hb - ha, hb)))
        else:
            out.append((it["doc"], it["src"], it["dst"], ("h", hb - ha, hb), ("t", tb - ta, tb)))
    return out


def _ref_tuples(items):
    out = []
    for it in items:
        if it.complete:
            out.append((it.seqid, it.src_gpuid, it.gpuid, ("c", it.complete_item["q"], it.complete_item["kv"])))
        else:
            out.append((it.seqid, it.src_gpuid, it.gpuid, ("h", it.head["q"], it.head["kv"]),
                        ("t", it.tail["q"], it.tail["kv"])))
    return out


@pytest.mark.parametrize("world,tpr,max_doc", [(2, 1024, 4096), (4, 4096, 16384), (8, 8192, 8192), (3, 2048, 65536)])
def test_sequential_fill_layout_equals_reference(world, tpr, max_doc):
    P, _ = _ref()
    rng = np.random.default_rng(world * 1000 + tpr)
    for _ in range(10):
        # documents may be longer than one rank's share: they span ranks as head / tail pairs
        docs, left = [], world * tpr
        while left > 0:
            L = max(16, min(int(np.exp(rng.uniform(np.log(64), np.log(max_doc)))) // 16 * 16, left))
            docs.append(L)
            left -= L
        ref_items = P.batch_to_items_general([docs], tpr, world, MC)
        mine = Planner(PlannerConfig(world=world, tokens_per_rank=tpr)).items([docs])
        assert _mine_as_ref_tuples(mine) == _ref_tuples(ref_items)


def test_cp_list_to_mlp_list_equals_reference():
    P, _ = _ref()
    rng = np.random.default_rng(7)
    for _ in range(50):
        world = int(rng.integers(1, 6))
        tpr = int(rng.integers(2, 40)) * 16
        docs, left = [], world * tpr
        while left > 0:
            L = max(16, min(int(rng.integers(1, 3 * tpr // 16 + 2)) * 16, left))
            docs.append(L)
            left -= L
        ref = P.cp_list_to_mlp_list([docs], world, tpr)
        assert cp_list_to_mlp_list([docs], world, tpr) == [list(map(int, r)) for r in ref]


def _flops_per_rank_ref(items, world):
    f = [0.0] * world
    for it in items:
        f[it.gpuid] += it.total_flops
    return f


@pytest.mark.parametrize("world,tpr", [(4, 16384), (8, 32768), (8, 131072)])
def test_balancer_against_reference(world, tpr):
    """Same documents, same tolerance: both planners conserve every document's tokens and the total work; the
    C++ balancer ends at least as balanced as the reference's and is faster (the timed CPU baseline)."""
    P, _ = _ref()
    rng = np.random.default_rng(world + tpr)
    tol = 0.1
    t_ref = t_mine = 0.0
    for _ in range(5):
        batches = _random_batches(rng, world, tpr, max_doc=tpr)
        items = P.batch_to_items_general(batches, tpr, world, MC)
        pl = P.Planner(world, PAR, tolerance_factor=tol, model_config=MC)
        t0 = time.perf_counter()
        planned = pl.plan_items(items)
        t_ref += time.perf_counter() - t0
        f_ref = _flops_per_rank_ref(planned, world)
        mine = Planner(PlannerConfig(world=world, tokens_per_rank=tpr, tolerance=tol))
        t0 = time.perf_counter()
        bal = mine.balanced_items(batches)
        t_mine += time.perf_counter() - t0
        f_mine = [0.0] * world
        q_per_doc = {}
        for it in bal:
            f_mine[it["dst"]] += it["flops"]
            (ha, hb), (ta, tb) = it["head"], it["tail"]
            q_per_doc[it["doc"]] = q_per_doc.get(it["doc"], 0) + (hb - ha) + (tb - ta)
        docs_flat = [L for b in batches for L in b]
        assert [q_per_doc[d] for d in range(len(docs_flat))] == docs_flat          # every token placed exactly once
        # the reference counts q*kv - q(q-1)/2 pairs per chunk as well (distca/planner/planner.py:366-378)
        assert abs(sum(f_mine) - sum(f_ref)) <= 1e-6 * sum(f_ref)
        imb_ref = max(f_ref) / (sum(f_ref) / world)
        imb_mine = max(f_mine) / (sum(f_mine) / world)
        assert imb_mine <= max(imb_ref, 1.0 + tol) + 1e-9, (imb_mine, imb_ref)
    print(f"\nplanner time over 5 batches, world {world}, {tpr} tokens/rank: reference {t_ref * 1e3:.1f} ms, "
          f"C++ {t_mine * 1e3:.1f} ms ({t_ref / max(t_mine, 1e-9):.0f}x)")
    assert t_mine < t_ref


def _to_ref_shard_dicts(plan_items):
    out = []
    for it in plan_items:
        for a, b in (it["head"], it["tail"]):
            if b > a:
                out.append({"seqid": it["doc"], "src_gpuid": it["src"], "gpuid": it["dst"], "q": b - a, "kv": b})
    by_doc = {}
    for d in out:
        by_doc.setdefault(d["seqid"], []).append(d)
    for shards in by_doc.values():
        shards.sort(key=lambda x: x["kv"])
        for i, s in enumerate(shards):
            s["shard_id"] = i
    return out


@pytest.mark.parametrize("world,tpr", [(2, 2048), (4, 8192), (8, 16384)])
def test_fa2a_byte_matrices_equal_reference_metadata(world, tpr):
    """The C++ plan's shard placement is handed to the reference's ``from_planner_output``; its four [W, W]
    all-to-all matrices (send displacement, transfer size, receive displacement, receive size) must equal
    the ones the C++ metadata compiler derives for the same plan: same de-duplication of K/V shards per
    destination, same segment order, same offsets."""
    P, M = _ref()
    from distca.runtime.shard_info import items_into_shardinfos
    rng = np.random.default_rng(world * 31 + tpr)
    hq, hkv, D, elt = 32, 8, 128, 2
    for _ in range(5):
        batches = _random_batches(rng, world, tpr, max_doc=tpr)
        mine = Planner(PlannerConfig(world=world, tokens_per_rank=tpr, tolerance=0.05,
                                     q_row_bytes=hq * D * elt, kv_row_bytes=hkv * D * elt))
        plan = mine.plan(batches)
        assert any(it["src"] != it["dst"] for it in plan.items), "the batch should need re-balancing"
        shard_infos = items_into_shardinfos(_to_ref_shard_dicts(plan.items))
        fwd, _rev, _of, _or, _attn = M.from_planner_output(world, shard_infos, hq * D, hkv * D, 0, elt,
                                                           is_pipeline_tick=False)
        send_disp, transfer_sz, recv_disp, recv_sz = (np.asarray(t.cpu()).astype(np.int64) for t in fwd.fa2a_metadata)
        f = mine.fa2a_matrices(plan)
        np.testing.assert_array_equal(np.asarray(f.transfer_sz).reshape(world, world), transfer_sz)
        np.testing.assert_array_equal(np.asarray(f.recv_transfer_sz).reshape(world, world), recv_sz)
        np.testing.assert_array_equal(np.asarray(f.send_disp).reshape(world, world), send_disp)
        np.testing.assert_array_equal(np.asarray(f.recv_disp).reshape(world, world), recv_disp)
