"""Workload-balanced packing of documents over data-parallel ranks (the WLB-LLM baseline).

Instead of moving core attention at run time, this baseline moves whole documents between ranks
before the step: documents are sorted by workload and placed greedily on the rank with the least
work whose token budget ``l_max`` still has room. The workload of a document of ``l`` tokens is
``(l / B)^2 + l / B`` with ``B`` the length at which attention and the linear layers cost the same
(``ATTN_LINEAR_BREAKPOINT`` in the reference, distca/planner/wlb_planner.py:13-25, greedy packing
under ``Lmax`` :36-126). Ranks end up with different token counts, which is exactly the cost this
baseline pays (linear layers and memory become unbalanced).
"""
from __future__ import annotations

import os


def breakpoint_tokens(default: int = 128 * 1024) -> int:
    try:
        return int(os.environ["ATTN_LINEAR_BREAKPOINT"])
    except (KeyError, ValueError):
        return default


def workload(doc_lens, breakpoint: int | None = None) -> float:
    b = float(breakpoint or breakpoint_tokens())
    return sum((l / b) ** 2 + l / b for l in doc_lens)


def balance_documents(doc_lens, ranks: int, l_max: int, breakpoint: int | None = None) -> list[list[int]]:
    """Greedy longest-processing-time packing: returns ``ranks`` lists of document lengths. A document
    that fits nowhere under ``l_max`` goes to the rank with the fewest tokens (and overflows it)."""
    b = breakpoint or breakpoint_tokens()
    bins: list[list[int]] = [[] for _ in range(ranks)]
    work = [0.0] * ranks
    tokens = [0] * ranks
    for l in sorted((int(x) for x in doc_lens), reverse=True):
        order = sorted(range(ranks), key=lambda r: (work[r], tokens[r]))
        dst = next((r for r in order if tokens[r] + l <= l_max), None)
        if dst is None:
            dst = min(range(ranks), key=lambda r: tokens[r])
        bins[dst].append(l)
        work[dst] += workload([l], b)
        tokens[dst] += l
    return bins


def imbalance(bins, breakpoint: int | None = None) -> dict:
    w = [workload(b, breakpoint) for b in bins]
    t = [sum(b) for b in bins]
    mean_w = sum(w) / max(1, len(w))
    mean_t = sum(t) / max(1, len(t))
    return {"workload_max_over_mean": max(w) / mean_w if mean_w else 1.0,
            "tokens_max_over_mean": max(t) / mean_t if mean_t else 1.0, "tokens": t}


def pack_balanced(doc_lens, packs: int, tokens_per_pack: int, breakpoint: int | None = None, multiple_of: int = 16
                  ) -> list[list[int]]:
    """Workload-balanced packing into ``packs`` packs of EXACTLY ``tokens_per_pack`` tokens (what a trainer whose
    ranks all hold the same number of tokens can use): documents longest first, each to the pack with the least
    work that still has room for all of it; a document that fits nowhere whole is cut and its pieces fill the
    packs with the most room. ``doc_lens`` must hold at least ``packs * tokens_per_pack`` tokens; documents are taken in the
    given order until that many tokens are reached (the last one is cut), the rest is not used. Lengths are rounded up to ``multiple_of`` first."""
    b = breakpoint or breakpoint_tokens()
    need = packs * tokens_per_pack
    docs = [-(-int(x) // multiple_of) * multiple_of for x in doc_lens]
    assert sum(docs) >= need and tokens_per_pack % multiple_of == 0, "not enough tokens to fill the packs"
    kept, total = [], 0
    for l in docs:                                     # in the given order (no preference for long documents)
        take = min(l, need - total)
        if take > 0:
            kept.append(take)
            total += take
    kept.sort(reverse=True)
    bins: list[list[int]] = [[] for _ in range(packs)]
    work, room = [0.0] * packs, [tokens_per_pack] * packs
    for l in kept:
        order = sorted(range(packs), key=lambda r: (work[r], -room[r]))
        dst = next((r for r in order if room[r] >= l), None)
        if dst is not None:
            bins[dst].append(l)
            work[dst] += workload([l], b)
            room[dst] -= l
            continue
        while l > 0:                                   # cut: fill the emptiest packs first
            dst = max(range(packs), key=lambda r: room[r])
            piece = min(l, room[dst])
            assert piece > 0
            bins[dst].append(piece)
            work[dst] += workload([piece], b)
            room[dst] -= piece
            l -= piece
    assert all(r == 0 for r in room)
    return bins
