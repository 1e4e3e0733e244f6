"""Synthetic packed-document batches.

Document-length samplers: log-uniform in a range, the long/short mixture used for 128K-256K
context runs (80 % log-uniform in [128, 8192], 20 % log-uniform in [32768, L_max]), and
the ``wlbllm`` / ``prolong`` length distributions of the reference's data sets, reproduced from their quantiles
and shaped by the same up-sample / filter / elongate options (distca/simulator/optimizers/samples.py:152-250). ``pack_documents`` fills fixed-size token
buffers, carrying the overflow of a document into the next pack and rounding lengths up to a
multiple of 16 (samples.py:253-305).

Token ids are uniform random; labels are next-token ids with -100 at the last token of every
document and pack (the reference's loss mask, pretrain_llama.py:102-141).
"""
from __future__ import annotations

import math

import numpy as np
import torch


def sample_loguniform(rng: np.random.Generator, n: int, lo: int, hi: int) -> np.ndarray:
    return np.exp(rng.uniform(math.log(lo), math.log(hi), size=n)).astype(np.int64)


def sample_mixture(rng: np.random.Generator, n: int, max_len: int, short=(128, 8192),
                   long_lo: int = 32768, long_frac: float = 0.2) -> np.ndarray:
    is_long = rng.random(n) < long_frac
    s = sample_loguniform(rng, n, *short)
    l = sample_loguniform(rng, n, min(long_lo, max_len), max_len)
    return np.where(is_long, l, s)


# Quantiles of the document-length samples the reference ships for its two data sets (summary statistics of
# distca/simulator/data/dist_wlbllm.json, 99 519 documents, mean 3 962 tokens, and dist_prolong.json, 77 932
# documents, mean 3 052; the samples themselves are the reference's data and are not redistributed). Both are
# dominated by documents of a few thousand tokens with a thin tail: 0.9 % (wlbllm) / 0.2 % (prolong) of the
# documents reach 32K tokens, and they hold 17 % / 5 % of all tokens.
_Q = (0.0, 0.01, 0.05, 0.10, 0.25, 0.50, 0.75, 0.90, 0.95, 0.99, 0.995, 0.999, 1.0)
_LENGTH_QUANTILES = {
    "wlbllm": (1, 63, 324, 646, 1606, 3227, 4832, 5784, 6110, 26058, 69097, 119793, 124913),
    "prolong": (575, 678, 801, 919, 1237, 1913, 3467, 6051, 8378, 16269, 21357, 47397, 340149),
}


def _cdf(kind: str, length: float) -> float:
    """Fraction of the ``kind`` documents shorter than ``length`` (log-linear between the quantile knots)."""
    q, v = np.asarray(_Q), np.log(np.asarray(_LENGTH_QUANTILES[kind], dtype=np.float64))
    return float(np.interp(math.log(max(length, 1.0)), v, q, left=0.0, right=1.0))


def sample_histogram(rng: np.random.Generator, n: int, kind: str, max_len: int, *, up_sample_factor: int = 1,
                     filter_threshold: int = 10000, filter_ratio: float = 1.0, elongate_factor: int = 1,
                     change_long_doc_ratio: float = 0.0) -> np.ndarray:
    """``n`` document lengths from the ``wlbllm`` / ``prolong`` length distributions (inverse-CDF sampling through
    the quantile table above), shaped the way the reference shapes its samples
    (distca/simulator/optimizers/samples.py:152-250): documents shorter than ``filter_threshold`` are kept with
    probability ``filter_ratio``, longer ones count ``up_sample_factor`` times; ``wlbllm`` lengths are multiplied by
    ``elongate_factor``; in ``prolong`` a long document becomes a full context of ``65536 * elongate_factor`` tokens
    with probability ``change_long_doc_ratio``. Lengths are clipped to ``[16, max_len]``."""
    if kind not in _LENGTH_QUANTILES:
        raise ValueError(kind)
    q, logv = np.asarray(_Q), np.log(np.asarray(_LENGTH_QUANTILES[kind], dtype=np.float64))
    f_thr = _cdf(kind, filter_threshold)                       # probability mass of the short documents
    w_short, w_long = f_thr * max(filter_ratio, 0.0), (1.0 - f_thr) * max(int(up_sample_factor), 1)
    p_long = w_long / (w_short + w_long) if (w_short + w_long) > 0 else 0.0
    is_long = rng.random(n) < p_long
    u = rng.random(n)
    u = np.where(is_long, f_thr + u * (1.0 - f_thr), u * f_thr)
    x = np.exp(np.interp(u, q, logv))
    if kind == "wlbllm":
        x = x * max(int(elongate_factor), 1)
    else:
        full = is_long & (rng.random(n) < change_long_doc_ratio)
        x = np.where(full, 65536.0 * max(int(elongate_factor), 1), x)
    return np.clip(x, 16, max_len).astype(np.int64)


def sample_doc_lens(rng: np.random.Generator, n: int, name: str, max_len: int, **shape) -> np.ndarray:
    """``shape``: the modifiers of :func:`sample_histogram` (only the data-set distributions have them)."""
    if name == "loguniform":
        return sample_loguniform(rng, n, 128, max_len)
    if name == "loguniform64":
        return sample_loguniform(rng, n, 64, min(4096, max_len))
    if name == "mixture":
        return sample_mixture(rng, n, max_len)
    if name in ("wlbllm", "prolong"):
        return sample_histogram(rng, n, name, max_len, **shape)
    if name == "full":
        return np.full(n, max_len, dtype=np.int64)
    raise ValueError(f"unknown document-length distribution {name!r}")


def pack_documents(doc_lens, tokens_per_pack: int, multiple_of: int = 16, max_packs: int | None = None
                   ) -> list[list[int]]:
    """Greedy sequential packing; a document that does not fit is cut and its rest opens the next pack."""
    packs: list[list[int]] = []
    cur: list[int] = []
    room = tokens_per_pack
    for L in doc_lens:
        L = int(math.ceil(int(L) / multiple_of) * multiple_of)
        while L > 0:
            take = min(L, room)
            cur.append(take)
            room -= take
            L -= take
            if room == 0:
                packs.append(cur)
                if max_packs is not None and len(packs) >= max_packs:
                    return packs
                cur, room = [], tokens_per_pack
    return packs


class SyntheticBatches:
    """Endless stream of global batches: ``num_seqs`` packs of ``tokens_per_seq`` tokens each."""

    def __init__(self, tokens_per_seq: int, num_seqs: int, dist: str = "mixture", seed: int = 0,
                 vocab: int = 32000, max_doc_len: int | None = None, shape: dict | None = None,
                 debug_packs: int = 0, packing: str = "sequential"):
        """``shape``: up_sample_factor / filter_threshold / filter_ratio / elongate_factor / change_long_doc_ratio
        for the ``wlbllm`` and ``prolong`` distributions (see :func:`sample_histogram`). ``debug_packs``: the first
        so many packs of the stream hold ONE document of the full length each (the reference's manual debug
        cases, distca/utils/global_batch_provider.py:132-152: the heaviest, perfectly balanced workload)."""
        self.tokens_per_seq, self.num_seqs, self.dist = tokens_per_seq, num_seqs, dist
        self.vocab = vocab
        self.max_doc_len = max_doc_len or tokens_per_seq
        self.shape = dict(shape or {})
        self.debug_packs = int(debug_packs)
        assert packing in ("sequential", "wlb")
        self.packing = packing          # wlb: workload-balanced packing of every global batch (data/wlb.py::pack_balanced)
        self.rng = np.random.default_rng(seed)

    def next_doc_lens(self) -> list[list[int]]:
        packs: list[list[int]] = []
        while self.debug_packs > 0 and len(packs) < self.num_seqs:
            packs.append([self.tokens_per_seq])
            self.debug_packs -= 1
        if self.packing == "wlb" and len(packs) < self.num_seqs:
            from .wlb import pack_balanced
            need, lens = self.num_seqs - len(packs), []
            while sum(lens) < need * self.tokens_per_seq:
                lens += [int(-(-x // 16) * 16) for x in
                         sample_doc_lens(self.rng, max(8, 4 * need), self.dist, self.max_doc_len, **self.shape)]
            return packs + pack_balanced(lens, need, self.tokens_per_seq)
        while len(packs) < self.num_seqs:
            need = self.num_seqs - len(packs)
            lens = sample_doc_lens(self.rng, max(8, 4 * need), self.dist, self.max_doc_len, **self.shape)
            packs += pack_documents(lens, self.tokens_per_seq, max_packs=need)
        return packs

    def next_tokens(self, packs: list[list[int]], pinned: bool = False):
        """ids / labels / positions for every pack, as CPU tensors (optionally pinned)."""
        n = self.tokens_per_seq
        ids = torch.from_numpy(self.rng.integers(0, self.vocab, size=(len(packs), n), dtype=np.int64))
        labels = torch.empty_like(ids)
        labels[:, :-1] = ids[:, 1:]
        labels[:, -1] = -100
        pos = torch.empty(len(packs), n, dtype=torch.int32)
        for i, docs in enumerate(packs):
            off = 0
            for L in docs:
                pos[i, off:off + L] = torch.arange(L, dtype=torch.int32)
                labels[i, off + L - 1] = -100
                off += L
        if pinned:
            ids, labels, pos = ids.pin_memory(), labels.pin_memory(), pos.pin_memory()
        return ids, labels, pos
