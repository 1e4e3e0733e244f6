"""Per-document context parallelism WITHOUT core-attention disaggregation: the baseline the headline
comparison is defined against (``--baseline-mode percp``).

Every document of the global batch is cut into ``2 * W`` equal chunks; rank ``r`` of the ``W``-rank group owns
chunk ``r`` (head) and chunk ``2W - 1 - r`` (tail) of EVERY document, so tokens and causal work are balanced per
document by construction. Per layer:

    forward   all-gather K and V over the group (NCCL), bring them into per-document order, run this rank's
              two query chunks of every document against the document's prefix (bottom-right causal)
    backward  attention backward gives dK / dV for whole prefixes; they are brought back into rank order
              and reduce-scattered over the group (NCCL), each rank keeping the gradient of its own K / V rows

which is the WLB-LLM per-document CP attention the reference compares with
(baseline/wlbllm_original/wlbllm/per_doc_cp_attn.py:117-147 all-gather, :245-304 two attention calls per rank,
:472-475 reduce-scatter; the re-ordering is its shuffle kernel, baseline/wlbllm_original/csrc/memcpy.cu:21-79).
The attention kernels are this repository's; the collectives and the re-ordering are library calls (NCCL,
``index_select``) on purpose: this is the baseline, not the product. Traffic per layer and rank: every other
rank's K and V rows in, as many gradient rows out, independent of how long the documents are, against the
planner-chosen subset that disaggregation moves.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..models.llama import TwoPhaseCoreAttention
from ..ops import attention as attn_ops
from ..ops import elementwise as ew


def percp_layout(doc_lens: list[int], world: int, rank: int) -> list[tuple[int, int, int, int]]:
    """Segments ``(doc, a, b, row0)`` of rank ``rank``: head chunk then tail chunk of every document, in
    document order. Document lengths must be multiples of ``2 * world``."""
    out, row = [], 0
    for d, L in enumerate(doc_lens):
        assert L % (2 * world) == 0, f"document of {L} tokens is not a multiple of 2 x {world}"
        c = L // (2 * world)
        out.append((d, rank * c, (rank + 1) * c, row))
        out.append((d, (2 * world - 1 - rank) * c, (2 * world - rank) * c, row + c))
        row += 2 * c
    return out


def perseq_layout(doc_lens: list[int], world: int, rank: int, seq_len: int) -> list[tuple[int, int, int, int]]:
    """Per-SEQUENCE context parallelism: the documents are taken as packed sequences of ``seq_len`` tokens
    (consecutive documents that add up to ``seq_len``), every sequence is cut into ``2 * world`` equal chunks
    wherever the document boundaries are, and rank ``rank`` owns chunk ``rank`` and chunk ``2 * world - 1 - rank``
    of every sequence. Returns the segments ``(doc, a, b, row0)`` those chunks are made of. Tokens are balanced,
    causal work is not: a chunk that holds the end of a long document carries far more than one that holds short
    ones (the reference's second baseline, baseline/wlbllm_original/wlbllm/per_seq_cp_attn.py:26-57, 123-124)."""
    assert seq_len % (2 * world) == 0, f"sequence of {seq_len} tokens is not a multiple of 2 x {world}"
    c = seq_len // (2 * world)
    out, row = [], 0
    seq_docs, acc = [], 0          # (doc index, length) of the sequence being filled
    for d, L in enumerate(doc_lens):
        seq_docs.append((d, int(L)))
        acc += int(L)
        assert acc <= seq_len, "documents do not pack into sequences of seq_len tokens"
        if acc < seq_len:
            continue
        for lo in (rank * c, (2 * world - 1 - rank) * c):          # head chunk, tail chunk in sequence coordinates
            hi, start = lo + c, 0
            for dd, LL in seq_docs:
                a, b = max(lo, start) - start, min(hi, start + LL) - start
                if b > a:
                    out.append((dd, a, b, row))
                    row += b - a
                start += LL
        seq_docs, acc = [], 0
    assert not seq_docs, "the last sequence is incomplete"
    return out


def round_documents(doc_lens: list[int], world: int) -> list[int]:
    """Document lengths rounded so that each is a multiple of ``2 * world`` while the total is unchanged
    (tokens move between neighbouring documents); the total must itself be such a multiple."""
    unit = 2 * world
    total = sum(doc_lens)
    assert total % unit == 0
    out, carry = [], 0
    for L in doc_lens:
        L += carry
        r = L // unit * unit
        carry = L - r
        if r > 0:
            out.append(r)
    if carry:
        out[-1] += carry
    assert sum(out) == total and all(x % unit == 0 for x in out)
    return out


class PerDocCPAttention(TwoPhaseCoreAttention):
    """Core attention of one rank of a per-document context-parallel group (same interface as
    :class:`~distca_b200.models.llama.LocalCoreAttention`)."""

    def __init__(self, cfg: ModelConfig, group, world: int, rank: int, device, tp: int = 1, seq_len: int | None = None):
        """``seq_len``: cut packed sequences of that many tokens instead of documents (per-sequence CP,
        :func:`perseq_layout`)."""
        self.hq, self.hkv, self.D = cfg.heads_q // tp, cfg.heads_kv // tp, cfg.head_dim
        self.group, self.W, self.me = group, world, rank
        self.seq_len = seq_len
        self.device = torch.device(device)
        self.plan: attn_ops.AttnPlan | None = None
        self.scratch = attn_ops.BwdScratch()
        self.bytes_per_layer = 0       # K/V bytes this rank receives per layer forward (for reports)

    # ------------------------------------------------------------------------------------------
    def layout(self, doc_lens: list[int], rank: int | None = None):
        """Segments ``(doc, a, b, row0)`` of ``rank`` (default: this rank) for the global batch ``doc_lens``."""
        r = self.me if rank is None else rank
        if self.seq_len:
            return perseq_layout(doc_lens, self.W, r, self.seq_len)
        return percp_layout(doc_lens, self.W, r)

    def set_batch(self, doc_lens: list[int]) -> None:
        """``doc_lens``: every document of the GLOBAL batch, in order (all ranks pass the same list)."""
        W, me = self.W, self.me
        lens = np.asarray(doc_lens, dtype=np.int64)
        total = int(lens.sum())
        T_local = total // W
        doc_row0_global = np.concatenate([[0], np.cumsum(lens)[:-1]])       # first row in per-document order
        # gathered buffer row (rank-major: rank * T_local + local row) of every token in per-document order
        perm = np.empty(total, dtype=np.int64)
        mine = None
        for r in range(W):
            segs = self.layout(doc_lens, r)
            assert sum(b - a for _, a, b, _ in segs) == T_local, "ranks own unequal token counts"
            for d, a, b, row0 in segs:
                g0 = int(doc_row0_global[d])
                perm[g0 + a:g0 + b] = r * T_local + row0 + np.arange(b - a)
            if r == me:
                mine = segs
        inv = np.empty(total, dtype=np.int64)
        inv[perm] = np.arange(total)
        self.perm = torch.from_numpy(perm).to(self.device)
        self.inv = torch.from_numpy(inv).to(self.device)
        # this rank's tasks: the query rows of a segment see the keys of their document up to the segment's end
        tasks = [(row0, b - a, int(doc_row0_global[d]), b) for d, a, b, row0 in mine if b > a]
        self.plan = attn_ops.AttnPlan(attn_ops.AttnTasks.from_lists(tasks), self.device)
        self.T_local, self.total = T_local, total
        self.bytes_per_layer = (W - 1) * T_local * 2 * self.hkv * self.D * 2

    # ------------------------------------------------------------------------------------------
    def apply_rope(self, qkv, pos, table) -> None:
        ew.rope_(qkv, pos, table, self.hq, self.hkv, self.D)

    def qkv_epilogue(self):
        return {"write_local": True}

    def _split(self, qkv):
        qd, kd = self.hq * self.D, self.hkv * self.D
        return (qkv[:, :qd].unflatten(1, (self.hq, self.D)), qkv[:, qd:qd + kd].unflatten(1, (self.hkv, self.D)),
                qkv[:, qd + kd:].unflatten(1, (self.hkv, self.D)))

    def _gather_kv(self, qkv: torch.Tensor):
        """All-gather this layer's K and V rows and bring them into per-document order."""
        kd = self.hkv * self.D
        kv_local = qkv[:, self.hq * self.D:].contiguous()                    # [T_local, 2 * kd]
        gathered = torch.empty(self.W * self.T_local, 2 * kd, dtype=qkv.dtype, device=qkv.device)
        dist.all_gather_into_tensor(gathered, kv_local, group=self.group)
        ordered = gathered.index_select(0, self.perm)                        # the baseline's shuffle pass
        del gathered
        return (ordered[:, :kd].unflatten(1, (self.hkv, self.D)), ordered[:, kd:].unflatten(1, (self.hkv, self.D)))

    def forward(self, qkv: torch.Tensor, layer: int = 0):
        q, _, _ = self._split(qkv)
        k, v = self._gather_kv(qkv)
        o, lse = attn_ops.flash_fwd(q, k, v, self.plan)
        return o.flatten(1), (qkv, o, lse)        # K / V are gathered again in backward (nothing kept per layer)

    def pack_saved(self, attn_out: torch.Tensor, ctx) -> torch.Tensor:
        lse = ctx[2]
        if attn_out.dtype == torch.bfloat16:
            return torch.cat([attn_out, lse.contiguous().view(torch.bfloat16)], dim=1)
        return torch.cat([attn_out, lse.to(attn_out.dtype)], dim=1)

    def restore(self, qkv: torch.Tensor, saved: torch.Tensor, layer: int = 0):
        qd = self.hq * self.D
        o = saved[:, :qd]
        lse = saved[:, qd:].contiguous()
        lse = lse.view(torch.float32) if saved.dtype == torch.bfloat16 else lse.float()
        return o, (qkv, o.unflatten(1, (self.hq, self.D)), lse)

    def backward(self, ctx, dattn: torch.Tensor, layer: int = 0) -> torch.Tensor:
        qkv, o, lse = ctx
        q, _, _ = self._split(qkv)
        k, v = self._gather_kv(qkv)
        kd = self.hkv * self.D
        dqkv = torch.zeros_like(qkv) if not qkv.is_cuda else torch.empty_like(qkv)
        dq, _, _ = self._split(dqkv)
        do = dattn.unflatten(1, (self.hq, self.D))
        dkv = torch.zeros(self.total, 2 * kd, dtype=qkv.dtype, device=qkv.device)   # rows no task of mine sees stay zero
        dk = dkv[:, :kd].unflatten(1, (self.hkv, self.D))
        dv = dkv[:, kd:].unflatten(1, (self.hkv, self.D))
        if qkv.is_cuda:
            attn_ops.flash_bwd(q, k, v, o, lse, do, self.plan, dq=dq, dk=dk, dv=dv, scratch=self.scratch)
        else:
            gq, gk, gv = attn_ops.flash_bwd(q, k, v, o, lse, do, self.plan)
            dq.copy_(gq); dk.copy_(gk); dv.copy_(gv)
        del k, v
        rank_major = dkv.index_select(0, self.inv)          # back into (rank, local row) order
        del dkv
        mine = torch.empty(self.T_local, 2 * kd, dtype=qkv.dtype, device=qkv.device)
        if qkv.is_cuda:
            dist.reduce_scatter_tensor(mine, rank_major, group=self.group)
        else:
            dist.all_reduce(rank_major, group=self.group)
            mine.copy_(rank_major[self.me * self.T_local:(self.me + 1) * self.T_local])
        dqkv[:, self.hq * self.D:] = mine
        return dqkv
