"""CPU tests of the C++ CAD planner: layout, conservation laws, balance, dispatch tables.

The properties checked are the ones the reference asserts in tests/test_planner.py:20-180,
343-394 and 567-617 (query tokens per document conserved, contiguous head/tail structure, FLOPs
conserved, every server within tolerance of the mean)."""
import numpy as np
import pytest

from distca_b200.planner import Planner, PlannerConfig, chunk_flops, cp_list_to_mlp_list

K = 1024


def _planner(world, tpr, tol=0.1, **kw):
    return Planner(PlannerConfig(world=world, tokens_per_rank=tpr, tolerance=tol, **kw))


def _flops(item):
    f = 0
    for a, b in (item["head"], item["tail"]):
        if b > a:
            f += chunk_flops(b - a, b)
    return f


def test_layout_fits_and_zigzag():
    p = _planner(4, 16 * K)
    items = p.items([[32 * K], [8 * K, 8 * K], [4 * K] * 4])
    # the 32K document spans ranks 0 and 1 as head/tail pairs
    first, second = items[0], items[1]
    assert (first["src"], second["src"]) == (0, 1)
    assert first["head"] == (0, 8 * K) and first["tail"] == (24 * K, 32 * K)
    assert second["head"] == (8 * K, 16 * K) and second["tail"] == (16 * K, 24 * K)
    assert all(i["head"][0] == 0 and i["tail"][0] == i["tail"][1] for i in items[2:])
    assert [i["src"] for i in items[2:]] == [2, 2, 3, 3, 3, 3]


def test_layout_overflow_raises():
    p = _planner(2, 1024)
    with pytest.raises(RuntimeError):
        p.items([[4096]])


def test_cp_list_to_mlp_list_goldens():
    assert cp_list_to_mlp_list([[16 * K], [8 * K, 8 * K]], 2, 16 * K) == [[16 * K], [8 * K, 8 * K]]
    assert cp_list_to_mlp_list([[32 * K]], 2, 16 * K) == [[8 * K, 8 * K], [8 * K, 8 * K]]
    out = cp_list_to_mlp_list([[8 * K]], 4, 16 * K)
    assert out == [[8 * K], [], [], []]


@pytest.mark.parametrize("world,batch", [
    (4, [[16 * K], [8 * K, 8 * K], [4 * K] * 4, [2 * K] * 8]),
    (4, [[64 * K]]),
    (8, [[128 * K], [1 * K] * 128, [32 * K, 96 * K]] + [[16 * K] * 8] * 5),
])
@pytest.mark.parametrize("tol", [0.05, 0.1, 0.3])
def test_balance_conservation(world, batch, tol):
    total = sum(map(sum, batch))
    p = _planner(world, total // world, tol)
    before = p.items(batch)
    after = p.balanced_items(batch)
    # 1. query tokens per document conserved and disjoint
    for doc in {i["doc"] for i in before}:
        L = next(i["doc_len"] for i in before if i["doc"] == doc)
        cover = np.zeros(L, dtype=np.int32)
        for i in after:
            if i["doc"] == doc:
                for a, b in (i["head"], i["tail"]):
                    cover[a:b] += 1
        assert (cover == 1).all()
    # 2. FLOPs conserved
    assert sum(map(_flops, before)) == sum(map(_flops, after))
    # 3. every server within tolerance of the mean (documents have even lengths here)
    load = np.zeros(world)
    for i in after:
        load[i["dst"]] += _flops(i)
    avg = load.mean()
    assert load.min() >= avg * (1 - tol) - 1e-6 * avg - 2 * max(i["doc_len"] for i in after)
    assert load.max() <= avg * (1 + tol) + 2 * max(i["doc_len"] for i in after) + 1e-6 * avg or load.max() <= max(_flops(i) for i in before)


def test_plan_tables_are_consistent():
    world, tpr = 4, 16 * K
    batch = [[16 * K], [8 * K, 8 * K], [4 * K] * 4, [2 * K] * 8]
    p = _planner(world, tpr)
    plan = p.plan(batch)
    assert plan.fits and plan.imbalance_after <= 1.11
    assert plan.imbalance_before > 2.0
    seen_q = 0
    for r in range(world):
        rp = plan.rank(r)
        assert rp.num_tokens == tpr
        qr, qrow = rp.q_dst_rank, rp.q_dst_row
        assert (qr >= 0).all() and (qrow >= 0).all()
        seen_q += len(qr)
        # every local token's K/V goes at least to the server of its own query
        kr = rp.kv_dst_rank.reshape(tpr, rp.max_copies)
        assert ((kr == qr[:, None]).any(axis=1)).all()
    # server side: tasks tile the Q region without gaps, contexts cover what tasks need
    for s in range(world):
        rp = plan.rank(s)
        tasks = rp.tasks
        rows = 0
        for doc, qa, qb, qrow0, krow0, kvlen, owner, orow0 in tasks:
            assert qrow0 == rows and kvlen == qb
            rows += qb - qa
            # the owner's table points back at these rows
            own = plan.rank(int(owner))
            assert (own.q_dst_rank[orow0:orow0 + qb - qa] == s).all()
            assert (own.q_dst_row[orow0:orow0 + qb - qa] == np.arange(qrow0, qrow0 + qb - qa)).all()
        assert rows == rp.q_rows
        # context segments cover exactly the K/V rows in use
        cover = np.zeros(rp.kv_rows, dtype=np.int32)
        for k0, n, owner, orow0, slot in rp.ctx_segments:
            cover[k0:k0 + n] += 1
            own = plan.rank(int(owner))
            kr = own.kv_dst_rank.reshape(-1, own.max_copies)
            kw = own.kv_dst_row.reshape(-1, own.max_copies)
            assert (kr[orow0:orow0 + n, slot] == s).all()
            assert (kw[orow0:orow0 + n, slot] == np.arange(k0, k0 + n)).all()
        assert (cover == 1).all()
    assert seen_q == world * tpr


def test_capacity_backoff():
    world, tpr = 4, 16 * K
    batch = [[64 * K]]
    loose = _planner(world, tpr).plan(batch)
    assert loose.fits
    need = max(loose.rank(r).kv_rows for r in range(world))
    tight = _planner(world, tpr, max_q_rows=2 * tpr, max_kv_rows=need // 2).plan(batch)
    assert not tight.fits or max(tight.rank(r).kv_rows for r in range(world)) <= need // 2


def test_fa2a_matrices_and_simulator():
    from distca_b200.planner import default_time_model
    world, tpr = 4, 16 * K
    batch = [[48 * K], [4 * K] * 4]
    p = _planner(world, tpr)
    plan = p.plan(batch)
    m = p.fa2a_matrices(plan)
    sz = m.transfer_sz.reshape(world, world)
    sd = m.send_disp.reshape(world, world)
    rd = m.recv_disp.reshape(world, world)
    assert (sd[:, 1:] == np.cumsum(sz, axis=1)[:, :-1]).all() and (sd[:, 0] == 0).all()
    assert (rd[1:, :] == np.cumsum(sz, axis=0)[:-1, :]).all() and (rd[0, :] == 0).all()
    assert (m.recv_transfer_sz.reshape(world, world) == sz.T).all()
    sim = p.simulate(plan, default_time_model("b200"))
    assert sim.imbalance <= 1.2 and len(sim.attn_ms) == world


def test_per_document_cp_baseline_is_balanced_and_sends_more_context():
    """Baseline policy: every long document is cut into 2 x world head-tail chunks. It balances
    causal work like the CAD plan but ships each document's context to every server."""
    world, tpr = 4, 16 * K
    docs = [[16 * K], [8 * K, 8 * K], [4 * K] * 4, [2 * K] * 8]
    p = _planner(world, tpr)
    cad = p.plan_fixed(docs)
    cp = p.plan_fixed_cp(docs, min_len=1024)
    assert cp.fits and cp.imbalance_after <= 1.02
    assert abs(sum(cp.flops_after) - sum(cad.flops_after)) <= 1e-6 * sum(cad.flops_after)
    for r in range(world):
        rp = cp.rank(r)
        assert rp.num_tokens == tpr and (rp.q_dst_rank >= 0).all()
        assert rp.q_rows == tpr            # every server gets an equal share of every document
    sent = lambda plan: sum(int(np.asarray(plan.rank(r).send_bytes).sum() - plan.rank(r).send_bytes[r]) for r in range(world))
    assert sent(cp) > sent(cad)


def test_water_fill_policy_moves_only_the_longest_document():
    world, tpr = 4, 16 * K
    docs = [[16 * K], [4 * K] * 4, [2 * K] * 8, [1 * K] * 16]
    p = _planner(world, tpr)
    wf = p.plan_fixed_water_fill(docs)
    assert wf.fits and wf.imbalance_before > 2.0 and wf.imbalance_after < 1.05
    assert abs(sum(wf.flops_after) - sum(wf.flops_before)) <= 1e-6 * sum(wf.flops_before)
    # ranks 1..3 send nothing: only the long document of rank 0 is cut
    for r in range(1, world):
        sb = np.asarray(wf.rank(r).send_bytes)
        assert sb.sum() - sb[r] == 0
    # two long documents: water filling cannot fix the second one, the balancer can
    docs2 = [[16 * K], [12 * K, 4 * K], [2 * K] * 8, [1 * K] * 16]
    assert p.plan_fixed(docs2).imbalance_after <= p.plan_fixed_water_fill(docs2).imbalance_after + 1e-9


def test_cost_model_counts_the_tile_pairs_the_kernels_visit():
    """``CostModel.chunk_ms`` with unit tile-pair cost against a direct count over 128-row query tiles."""
    import numpy as np
    from distca_b200.planner import Planner, PlannerConfig
    cost = Planner(PlannerConfig(world=2, tokens_per_rank=1024, cost_model={"ms_per_tile_pair": 1.0})).options.cost
    rng = np.random.default_rng(0)
    for _ in range(500):
        kv = int(rng.integers(1, 6000))
        q = int(rng.integers(1, kv + 1))
        want = sum((kv - q + min((i + 1) * 128, q) + 127) // 128 for i in range((q + 127) // 128))
        assert cost.chunk_ms(q, kv) == want
    assert cost.chunk_ms(0, 100) == 0.0


def test_balancer_with_cost_model_and_server_speeds():
    """Balancing predicted milliseconds: every server ends within the tolerance of ITS share, and a server
    reported 10 % slower gets about 10 % less work."""
    import numpy as np
    from distca_b200.planner import Planner, PlannerConfig, default_cost_model
    from distca_b200.data.synthetic import SyntheticBatches
    cm = default_cost_model()
    docs = SyntheticBatches(65536, 8, "mixture", 5, 32000).next_doc_lens()
    even = Planner(PlannerConfig(world=8, tokens_per_rank=65536, tolerance=0.02, cost_model=cm)).plan_fixed(docs)
    c = np.asarray(even.cost_after)
    assert c.max() / c.mean() <= 1.03 and abs(even.cost_imbalance_after - c.max() / c.mean()) < 1e-9
    speed = [1.0] * 7 + [0.9]
    slow = Planner(PlannerConfig(world=8, tokens_per_rank=65536, tolerance=0.02, cost_model=cm, speed=speed)).plan_fixed(docs)
    c = np.asarray(slow.cost_after)
    share = c / c.sum()
    want = np.asarray(speed) / sum(speed)
    assert np.all(np.abs(share / want - 1.0) <= 0.035), share / want
    assert slow.cost_imbalance_after <= 1.035
    # every token is still placed exactly once
    q = {}
    for it in slow.items:
        (ha, hb), (ta, tb) = it["head"], it["tail"]
        q[it["doc"]] = q.get(it["doc"], 0) + hb - ha + tb - ta
    assert sorted(q.values()) == sorted(L for d in docs for L in d)


def test_cost_and_time_models_fitted_from_a_measured_sweep(tmp_path):
    """``kernel_bench --kernel attn_sweep`` output -> the balancer's cost model (relative least squares) and the
    simulator's attention table; other lines of the log are skipped."""
    import json
    from distca_b200.planner import cost_model_from_sweep, default_cost_model, time_model_from_sweep
    a, b = 1.0e-3, 2.0e-3
    rows = []
    for L, docs in [(2048, 16), (4096, 8), (8192, 1), (16384, 1), (32768, 1)]:
        n = L // 128
        pairs, qt = docs * n * (n + 1) // 2, docs * n
        total = a * pairs + b * qt
        rows.append({"kernel": "attn_sweep", "seqlen": L, "docs": docs, "heads": [32, 8], "fwd_ms": 0.25 * total,
                     "bwd_ms": 0.75 * total, "tile_pairs": pairs, "query_tiles": qt})
    p = tmp_path / "sweep.jsonl"
    p.write_text("warming up\n" + "\n".join(json.dumps(r) for r in rows)
                 + '\n{"kernel": "attn_sweep_fit", "ms_per_tile_pair": 1.0}\nnot json {\n')
    cm = cost_model_from_sweep(str(p))
    assert abs(cm["ms_per_tile_pair"] - a) < 1e-9 and abs(cm["ms_per_q_tile"] - b) < 1e-9 and cm["max_rel_err"] < 1e-9
    assert cm["workloads"] == 5 and cm["tile"] == 128
    half = cost_model_from_sweep(rows, heads_q=16)                   # a rank with half the query heads
    assert abs(half["ms_per_tile_pair"] - a / 2) < 1e-9
    # the three measured workloads of one B200: the fit stays within a few per cent of every one of them
    meas = [{"kernel": "attn_sweep", "seqlen": 8192, "docs": 1, "fwd_ms": 0.5347, "bwd_ms": 1.7322},
            {"kernel": "attn_sweep", "seqlen": 32768, "docs": 1, "fwd_ms": 7.2401, "bwd_ms": 25.5859},
            {"kernel": "attn_sweep", "seqlen": 2048, "docs": 16, "fwd_ms": 0.6636, "bwd_ms": 2.0348}]
    fit = cost_model_from_sweep(meas)
    assert fit["max_rel_err"] < 0.03 and 0.5 < fit["ms_per_tile_pair"] / default_cost_model(32)["ms_per_tile_pair"] < 1.5
    tm = time_model_from_sweep(rows)
    assert list(tm.attn_len) == [8192.0, 16384.0, 32768.0] and abs(tm.attn_ms_for(8192, 8192) - rows[2]["fwd_ms"]) < 1e-9
    import pytest
    with pytest.raises(ValueError):
        cost_model_from_sweep(rows[:1])
