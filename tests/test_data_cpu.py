"""Synthetic document-length distributions and packing."""
import json
import os

import numpy as np
import pytest

from distca_b200.data.synthetic import (SyntheticBatches, pack_documents, sample_doc_lens, sample_histogram,
                                        sample_mixture)

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DATA = os.path.join(os.environ.get("DISTCA_REFERENCE_ROOT", os.path.join(_REPO, "baseline", "_ref")),
                        "distca", "simulator", "data")


def test_data_set_distributions_have_the_reference_quantiles():
    """``wlbllm`` / ``prolong`` follow the published quantile tables: a few-thousand-token bulk and a thin tail."""
    rng = np.random.default_rng(0)
    w = sample_histogram(rng, 200000, "wlbllm", 10**7)
    p = sample_histogram(rng, 200000, "prolong", 10**7)
    for x, med, q90, q99 in ((w, 3227, 5784, 26058), (p, 1913, 6051, 16269)):
        assert abs(np.quantile(x, 0.5) - med) / med < 0.03
        assert abs(np.quantile(x, 0.9) - q90) / q90 < 0.03
        assert abs(np.quantile(x, 0.99) - q99) / q99 < 0.06
    assert 0.12 < w[w >= 32768].sum() / w.sum() < 0.22        # the rare long documents hold a sixth of the tokens
    assert w.min() >= 16 and sample_histogram(rng, 1000, "wlbllm", 4096).max() <= 4096
    with pytest.raises(ValueError):
        sample_histogram(rng, 10, "c5", 4096)


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_DATA, "dist_wlbllm.json")), reason="reference data not present")
@pytest.mark.parametrize("kind", ["wlbllm", "prolong"])
def test_data_set_distributions_against_the_reference_samples(kind):
    ref = np.asarray(json.load(open(os.path.join(REF_DATA, f"dist_{kind}.json"))), dtype=np.float64)
    x = sample_histogram(np.random.default_rng(1), 300000, kind, 10**7)
    for q in (0.05, 0.25, 0.5, 0.75, 0.95, 0.99):
        assert abs(np.quantile(x, q) - np.quantile(ref, q)) / np.quantile(ref, q) < 0.05, q
    assert abs(x.mean() - ref.mean()) / ref.mean() < 0.10


def test_shaping_options_move_mass_to_long_documents():
    """The reference's sampling options: short documents are thinned, long ones counted several times, lengths
    stretched; in ``prolong`` long documents can be replaced by full contexts."""
    rng = np.random.default_rng(2)
    base = sample_histogram(rng, 100000, "wlbllm", 10**7)
    shaped = sample_histogram(rng, 100000, "wlbllm", 10**7, up_sample_factor=4, filter_threshold=10000, filter_ratio=0.5)
    f0, f1 = (base >= 10000).mean(), (shaped >= 10000).mean()
    expect = 4 * f0 / (4 * f0 + 0.5 * (1 - f0))
    assert abs(f1 - expect) < 0.01 and f1 > 5 * f0
    twice = sample_histogram(np.random.default_rng(3), 50000, "wlbllm", 10**7, elongate_factor=2)
    once = sample_histogram(np.random.default_rng(3), 50000, "wlbllm", 10**7)
    assert np.all(np.abs(twice - 2 * once)[once > 16] <= 1)             # below 16 tokens the lower clip applies
    full = sample_histogram(rng, 100000, "prolong", 10**7, filter_threshold=10000, change_long_doc_ratio=0.5, elongate_factor=2)
    long_frac = (sample_histogram(rng, 100000, "prolong", 10**7) >= 10000).mean()
    assert abs((full == 131072).mean() - 0.5 * long_frac) < 0.005
    none = sample_histogram(rng, 1000, "wlbllm", 10**7, filter_threshold=0)      # no threshold: nothing is filtered
    assert none.size == 1000


def test_packing_fills_every_pack_and_carries_cut_documents_over():
    packs = pack_documents([5000, 100, 3000, 9000], 4096)
    assert all(sum(p) == 4096 for p in packs) and all(x % 16 == 0 for p in packs for x in p)
    assert packs[0] == [4096] and packs[1][0] == 5008 - 4096         # 5000 rounds up to 5008; its rest opens the next pack
    sb = SyntheticBatches(8192, 4, "wlbllm", seed=0, shape={"up_sample_factor": 4, "filter_threshold": 10000})
    docs = sb.next_doc_lens()
    assert len(docs) == 4 and all(sum(d) == 8192 for d in docs)
    ids, labels, pos = sb.next_tokens(docs)
    assert ids.shape == (4, 8192) and int((labels == -100).sum()) >= sum(len(d) for d in docs)
    m = sample_mixture(np.random.default_rng(0), 20000, 131072)
    assert 0.17 < (m >= 32768).mean() < 0.23
    assert sample_doc_lens(np.random.default_rng(0), 10, "full", 512).tolist() == [512] * 10


def test_debug_cases_open_the_stream_with_full_length_documents():
    sb = SyntheticBatches(4096, 2, "wlbllm", seed=0, debug_packs=3)
    assert sb.next_doc_lens() == [[4096], [4096]]
    second = sb.next_doc_lens()
    assert second[0] == [4096] and len(second[1]) >= 1 and sum(second[1]) == 4096
    assert sb.debug_packs == 0


def test_workload_balanced_packing_fills_equal_packs_and_evens_out_the_work():
    from distca_b200.data.wlb import pack_balanced, workload
    rng = np.random.default_rng(4)
    T, n = 32768, 8
    lens = []
    while sum(lens) < n * T:
        lens += [int(-(-x // 16) * 16) for x in sample_doc_lens(rng, 16, "loguniform", T // 2)]
    bal = pack_balanced(lens, n, T, breakpoint=T)
    seq = pack_documents(lens, T, max_packs=n)
    assert len(bal) == n and all(sum(p) == T for p in bal) and all(x % 16 == 0 for p in bal for x in p)
    spread = lambda packs: max(workload(p, T) for p in packs) / (sum(workload(p, T) for p in packs) / len(packs))
    assert spread(bal) < spread(seq) and spread(bal) < 1.25
    sb = SyntheticBatches(T, n, "mixture", seed=1, packing="wlb")
    docs = sb.next_doc_lens()
    assert len(docs) == n and all(sum(d) == T for d in docs)
    ids, labels, pos = sb.next_tokens(docs)
    assert ids.shape == (n, T) and int(pos.max()) < T
