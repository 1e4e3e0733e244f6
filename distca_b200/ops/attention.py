"""Core attention (CA) on task lists: the stateless ``softmax(QK^T)V`` that CAD moves around.

A *task* is ``(q_start, q_len, k_start, kv_len)``: ``q_len`` query rows starting at row
``q_start`` of the Q tensor attend, bottom-right causally, to the ``kv_len`` key rows starting at
row ``k_start`` of the K/V tensors (query ``i`` sees keys ``0 .. kv_len - q_len + i``).  A whole
document is the task ``(s, L, s, L)``; a Q shard that holds tokens ``[a, b)`` of a document is
``(q_pos, b - a, doc_k_start, b)``.  Several Q shards of one document share the same K/V rows.

GPU tensors run the tcgen05 kernels (``csrc/attn``); CPU tensors run an fp32/fp64-exact PyTorch
restatement that is also the oracle of the GPU tests.

Reference counterpart: ``FusedCommAttn`` / flash-attn varlen calls with per-shard materialised
K/V (distca/runtime/megatron/ops/fused_comm_attn.py:108-279).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib

TILE = 128

ATTN_WORK_DTYPE = np.dtype([("q_row0", "<i4"), ("q_valid", "<i4"), ("k_row0", "<i4"),
                            ("kv_limit_base", "<i4"), ("out_ptr", "<u8"), ("lse_ptr", "<u8"),
                            ("signal_ptr", "<u8"), ("reserved", "<u8")])
BWD_KV_DTYPE = np.dtype([("k_row0", "<i4"), ("k_valid", "<i4"), ("qt_begin", "<i4"), ("qt_end", "<i4")])
BWD_QT_DTYPE = np.dtype([("q_row0", "<i4"), ("q_valid", "<i4"), ("diag", "<i4"), ("reserved", "<i4")])
assert ATTN_WORK_DTYPE.itemsize == 48 and BWD_KV_DTYPE.itemsize == 16 and BWD_QT_DTYPE.itemsize == 16


@dataclass
class AttnTasks:
    """Host-side task table (int64 numpy arrays of equal length)."""
    q_start: np.ndarray
    q_len: np.ndarray
    k_start: np.ndarray
    kv_len: np.ndarray

    @staticmethod
    def from_lists(tasks) -> "AttnTasks":
        a = np.asarray(list(tasks), dtype=np.int64).reshape(-1, 4)
        return AttnTasks(a[:, 0].copy(), a[:, 1].copy(), a[:, 2].copy(), a[:, 3].copy())

    @staticmethod
    def from_doc_lens(doc_lens) -> "AttnTasks":
        """Plain packed batch: every document is one task over its own rows."""
        lens = np.asarray(list(doc_lens), dtype=np.int64)
        starts = np.concatenate([[0], np.cumsum(lens)[:-1]]) if len(lens) else lens
        return AttnTasks(starts.copy(), lens.copy(), starts.copy(), lens.copy())

    def __len__(self) -> int:
        return len(self.q_start)

    def flops_fwd(self, heads_q: int, head_dim: int) -> float:
        """Multiply-add FLOPs (x2) of QK^T and PV under the causal mask."""
        q, kv = self.q_len.astype(np.float64), self.kv_len.astype(np.float64)
        pairs = q * kv - q * (q - 1) / 2.0
        return float(4.0 * heads_q * head_dim * pairs.sum())


def forward_work(tasks: AttnTasks) -> np.ndarray:
    """Split tasks into 128-row query tiles, heaviest (most key tiles) first."""
    items = []
    for qs, ql, ks, kl in zip(tasks.q_start, tasks.q_len, tasks.k_start, tasks.kv_len):
        off = int(kl - ql)
        for r0 in range(0, int(ql), TILE):
            valid = min(TILE, int(ql) - r0)
            items.append((int(qs) + r0, valid, int(ks), off + r0))
    arr = np.zeros(len(items), dtype=ATTN_WORK_DTYPE)
    if items:
        a = np.asarray(items, dtype=np.int64)
        order = np.argsort(-(a[:, 3] + a[:, 1]), kind="stable")
        a = a[order]
        arr["q_row0"], arr["q_valid"], arr["k_row0"], arr["kv_limit_base"] = a[:, 0], a[:, 1], a[:, 2], a[:, 3]
    return arr


def backward_work(tasks: AttnTasks) -> tuple[np.ndarray, np.ndarray]:
    """Key-tile centred schedule of the backward pass.

    Tasks that share ``k_start`` are Q shards of one document context; each 128-key tile of the
    context lists every query tile (of any of those shards) that can see at least one of its keys.
    Returns ``(kv_work, q_tiles)`` with the heaviest key tiles first.
    """
    by_ctx: dict[int, list[int]] = {}
    for i, ks in enumerate(tasks.k_start):
        by_ctx.setdefault(int(ks), []).append(i)
    kv_parts, qt_parts, base = [], [], 0
    for ks, idxs in by_ctx.items():
        idx = np.asarray(idxs, dtype=np.int64)
        ql, kl, qs = (np.asarray(a, dtype=np.int64)[idx] for a in (tasks.q_len, tasks.kv_len, tasks.q_start))
        off = kl - ql
        ntile = (ql + TILE - 1) // TILE
        ctx_len = int(kl.max())
        k0 = np.arange(0, ctx_len, TILE, dtype=np.int64)                     # [K]
        # query tiles of a task that see key tile k0 form a suffix: the first is the smallest j whose last
        # row (off + j*T + valid - 1) reaches k0; none at all when the task's context ends before k0
        j0 = np.maximum(0, -((off[None, :] + TILE - 1 - k0[:, None]) // TILE))   # ceil((k0 - off - T + 1) / T), [K, n]
        cnt = np.where(kl[None, :] - 1 >= k0[:, None], np.maximum(ntile[None, :] - j0, 0), 0)
        # a short last tile may end before k0 although the full-tile formula admits it
        last_ok = off[None, :] + ql[None, :] - 1 >= k0[:, None]
        cnt = np.where(last_ok, cnt, 0)
        per_k = cnt.sum(axis=1)
        keep = per_k > 0
        total = int(per_k.sum())
        if total == 0:
            continue
        flat_cnt, flat_j0 = cnt.reshape(-1), j0.reshape(-1)
        seg_start = np.cumsum(flat_cnt) - flat_cnt
        seg = np.repeat(np.arange(flat_cnt.size), flat_cnt)                 # (k, task) pair of every entry
        j = np.arange(total) - seg_start[seg] + flat_j0[seg]
        ti, ki = seg % len(idx), seg // len(idx)
        q_row0 = qs[ti] + j * TILE
        q_valid = np.minimum(TILE, ql[ti] - j * TILE)
        diag = off[ti] + j * TILE - k0[ki]
        qt_parts.append(np.stack([q_row0, q_valid, diag], axis=1))
        ends = np.cumsum(per_k)
        begins = ends - per_k
        kv_parts.append(np.stack([ks + k0[keep], np.minimum(TILE, ctx_len - k0[keep]), base + begins[keep],
                                  base + ends[keep]], axis=1))
        base += total
    kv_items = np.concatenate(kv_parts) if kv_parts else np.zeros((0, 4), dtype=np.int64)
    qt_items = np.concatenate(qt_parts) if qt_parts else np.zeros((0, 3), dtype=np.int64)
    kv = np.zeros(len(kv_items), dtype=BWD_KV_DTYPE)
    qt = np.zeros(len(qt_items), dtype=BWD_QT_DTYPE)
    if len(kv_items):
        a = kv_items
        order = np.argsort(-(a[:, 3] - a[:, 2]), kind="stable")
        a = a[order]
        kv["k_row0"], kv["k_valid"], kv["qt_begin"], kv["qt_end"] = a[:, 0], a[:, 1], a[:, 2], a[:, 3]
        qt["q_row0"], qt["q_valid"], qt["diag"] = qt_items[:, 0], qt_items[:, 1], qt_items[:, 2]
    return kv, qt


def _to_device(arr: np.ndarray, device) -> torch.Tensor:
    t = torch.from_numpy(arr.view(np.uint8).reshape(-1).copy())
    return t.to(device, non_blocking=False)


class AttnPlan:
    """Device-resident work lists of one task table (forward tiles + backward schedule)."""

    def __init__(self, tasks: AttnTasks, device, *, out: torch.Tensor | None = None,
                 lse: torch.Tensor | None = None, need_backward: bool = True, upload: bool = True):
        """``upload=False`` builds the host arrays only (safe on a worker thread); :meth:`upload` then
        copies them to the device from the thread that owns the CUDA stream."""
        self.tasks = tasks
        self.device = torch.device(device)
        self.fwd_host = forward_work(tasks)
        self.num_fwd = len(self.fwd_host)
        self._fwd_dev = None
        self._fwd_key = None
        self.bwd_kv_dev = self.bwd_qt_dev = self.fwd_plain_dev = None
        if need_backward:
            kv, qt = backward_work(tasks)
            self.num_bwd = len(kv)
            self.bwd_kv_host, self.bwd_qt_host = kv, qt
            if upload:
                self.upload()
        else:
            self.num_bwd = 0

    def upload(self) -> None:
        if self.num_bwd is not None and hasattr(self, "bwd_kv_host") and self.device.type == "cuda" and self.bwd_kv_dev is None:
            self.bwd_kv_dev = _to_device(self.bwd_kv_host, self.device)
            self.bwd_qt_dev = _to_device(self.bwd_qt_host, self.device)
            # the query-centred dQ kernel walks the forward tile list (geometry fields only)
            self.fwd_plain_dev = _to_device(self.fwd_host, self.device)

    def fwd_device_work(self, out: torch.Tensor, lse: torch.Tensor | None) -> torch.Tensor:
        """Work list with output addresses resolved against local ``out``/``lse`` tensors."""
        key = (out.data_ptr(), out.stride(0), 0 if lse is None else lse.data_ptr())
        if self._fwd_key != key:
            w = self.fwd_host.copy()
            row_bytes = out.stride(0) * out.element_size()
            w["out_ptr"] = out.data_ptr() + w["q_row0"].astype(np.uint64) * np.uint64(row_bytes)
            if lse is not None:
                w["lse_ptr"] = lse.data_ptr() + w["q_row0"].astype(np.uint64) * np.uint64(lse.stride(0) * 4)
            self._fwd_dev = _to_device(w, self.device)
            self._fwd_key = key
        return self._fwd_dev


def attention_reference(q, k, v, tasks: AttnTasks, scale: float | None = None):
    """Plain PyTorch per-task causal attention. q: [Tq,Hq,D], k/v: [Tk,Hkv,D] -> (o, lse[Tq,Hq])."""
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    o = torch.zeros_like(q)
    lse = torch.zeros(Tq, Hq, dtype=torch.float32, device=q.device)
    for qs, ql, ks, kl in zip(tasks.q_start, tasks.q_len, tasks.k_start, tasks.kv_len):
        qs, ql, ks, kl = int(qs), int(ql), int(ks), int(kl)
        qq = q[qs:qs + ql].transpose(0, 1)                       # [Hq, ql, D]
        kk = k[ks:ks + kl].transpose(0, 1).repeat_interleave(g, dim=0)
        vv = v[ks:ks + kl].transpose(0, 1).repeat_interleave(g, dim=0)
        s = torch.matmul(qq, kk.transpose(1, 2)) * scale          # [Hq, ql, kl]
        i = torch.arange(ql, device=q.device)[:, None]
        j = torch.arange(kl, device=q.device)[None, :]
        s = s.masked_fill(j > i + (kl - ql), float("-inf"))
        lse_t = torch.logsumexp(s.float(), dim=-1)
        pr = torch.softmax(s.float(), dim=-1).to(q.dtype)
        o[qs:qs + ql] = torch.matmul(pr, vv).transpose(0, 1)
        lse[qs:qs + ql] = lse_t.transpose(0, 1)
    return o, lse


def flash_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, plan: AttnPlan,
              scale: float | None = None, out: torch.Tensor | None = None,
              lse: torch.Tensor | None = None, work_dev: torch.Tensor | None = None):
    """q: [Tq,Hq,D]; k, v: [Tk,Hkv,D] (row pitch free, inner dims contiguous). Returns (o, lse).

    ``work_dev`` overrides the plan's work list, e.g. with peer output addresses resolved by the
    CAD runtime; ``out``/``lse`` are then only used for their pitches.
    """
    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if not q.is_cuda:
        o, l = attention_reference(q, k, v, plan.tasks, scale)
        if out is not None:
            out.copy_(o); o = out
        if lse is not None:
            lse.copy_(l); l = lse
        return o, l
    assert q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == D
    assert k.stride(2) == 1 and k.stride(1) == D and v.stride(2) == 1 and v.stride(1) == D
    if out is None:
        out = torch.empty(Tq, Hq, D, dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty(Tq, Hq, dtype=torch.float32, device=q.device)
    if work_dev is None:
        work_dev = plan.fwd_device_work(out, lse)
    n = work_dev.numel() // ATTN_WORK_DTYPE.itemsize
    L = _lib.lib()
    rc = L.dca_flash_fwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.c_long(Tq), _lib.c_long(Tk),
        _lib.c_long(q.stride(0)), _lib.c_long(k.stride(0)), _lib.c_long(v.stride(0)),
        _lib.c_int(Hq), _lib.c_int(Hkv), _lib.c_int(D), _lib.ptr(work_dev), _lib.c_int(n),
        _lib.c_float(scale), _lib.c_long(out.stride(0) * 2), _lib.c_long(lse.stride(0) * 4),
        _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "flash_fwd")
    return out, lse


def attention_backward_reference(q, k, v, dout, tasks: AttnTasks, scale: float | None = None):
    """Autograd through :func:`attention_reference` (fp32 inputs recommended). Returns dq, dk, dv."""
    q = q.detach().clone().requires_grad_(True)
    k = k.detach().clone().requires_grad_(True)
    v = v.detach().clone().requires_grad_(True)
    if len(tasks) == 0:
        return torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    o, _ = attention_reference(q, k, v, tasks, scale)
    o.backward(dout)
    return q.grad, k.grad, v.grad


class BwdScratch:
    """Reusable scratch of the backward kernel (delta, lse2: fp32 [Hq, Tq])."""

    def __init__(self):
        self.delta = self.lse2 = None

    def get(self, Tq: int, Hq: int, D: int, device):
        if self.delta is None or self.delta.numel() < Hq * Tq or self.delta.device != device:
            self.delta = torch.empty(Hq * Tq, dtype=torch.float32, device=device)
            self.lse2 = torch.empty(Hq * Tq, dtype=torch.float32, device=device)
        return self.delta, self.lse2


_DEFAULT_SCRATCH = BwdScratch()


def flash_bwd(q, k, v, o, lse, dout, plan: AttnPlan, scale: float | None = None,
              dq=None, dk=None, dv=None, scratch: BwdScratch | None = None,
              delta_rows: torch.Tensor | None = None, dq_row_ptr: torch.Tensor | None = None,
              dkv_row_ptr: torch.Tensor | None = None, dv_off_bytes: int = 0):
    """Gradients of :func:`flash_fwd`. ``dk``/``dv`` rows not covered by any task are left as given
    (pass zero-filled tensors when such rows exist). With ``delta_rows`` (fp32 [Tq, Hq] =
    rowsum(dO o O), see :func:`attn_delta_rows`) ``o`` is not read and may be ``None``.
    With ``dq_row_ptr`` [Tq] / ``dkv_row_ptr`` [Tk] (device int64 addresses, 0 = skip the row) the kernels store
    every gradient row straight to that address (head 0 of the row; dV ``dv_off_bytes`` behind dK), e.g. into the
    token owners' arenas on other GPUs, and ``dq`` / ``dk`` / ``dv`` are not written.
    Returns ``(dq, dk, dv)``."""
    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if not q.is_cuda:
        gq, gk, gv = attention_backward_reference(q, k, v, dout, plan.tasks, scale)
        if dq is not None:
            dq.copy_(gq); gq = dq
        if dk is not None:
            dk.copy_(gk); gk = dk
        if dv is not None:
            dv.copy_(gv); gv = dv
        return gq, gk, gv
    dev = q.device
    if dq is None and dq_row_ptr is None:
        dq = torch.empty(Tq, Hq, D, dtype=torch.bfloat16, device=dev)
    if dk is None and dkv_row_ptr is None:
        dk = torch.zeros(Tk, Hkv, D, dtype=torch.bfloat16, device=dev)
    if dv is None and dkv_row_ptr is None:
        dv = torch.zeros(Tk, Hkv, D, dtype=torch.bfloat16, device=dev)
    for t in (q, k, v, dout, dq, dk, dv, o):
        assert t is None or (t.dtype == torch.bfloat16 and t.stride(2) == 1 and t.stride(1) == D)
    assert dq_row_ptr is None or (dq_row_ptr.dtype == torch.int64 and dq_row_ptr.numel() >= Tq)
    assert dkv_row_ptr is None or (dkv_row_ptr.dtype == torch.int64 and dkv_row_ptr.numel() >= Tk)
    delta, lse2 = (scratch or _DEFAULT_SCRATCH).get(Tq, Hq, D, dev)
    L = _lib.lib()
    rc = L.dca_flash_bwd(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(dout), _lib.ptr(lse),
        _lib.c_long(Tq), _lib.c_long(Tk), _lib.c_long(q.stride(0)), _lib.c_long(k.stride(0)),
        _lib.c_long(v.stride(0)), _lib.c_long(0 if o is None else o.stride(0)), _lib.c_long(dout.stride(0)),
        _lib.c_long(lse.stride(0)), _lib.c_int(Hq), _lib.c_int(Hkv), _lib.c_int(D),
        _lib.ptr(plan.bwd_kv_dev), _lib.c_int(plan.num_bwd), _lib.ptr(plan.bwd_qt_dev),
        _lib.ptr(plan.fwd_plain_dev), _lib.c_int(plan.num_fwd),
        _lib.c_float(scale), _lib.ptr(delta), _lib.ptr(lse2),
        _lib.ptr(dq), _lib.c_long(0 if dq is None else dq.stride(0)), _lib.ptr(dk),
        _lib.c_long(0 if dk is None else dk.stride(0)), _lib.ptr(dv), _lib.c_long(0 if dv is None else dv.stride(0)),
        _lib.ptr(delta_rows), _lib.c_long(0 if delta_rows is None else delta_rows.stride(0)),
        _lib.ptr(dq_row_ptr), _lib.ptr(dkv_row_ptr), _lib.c_long(dv_off_bytes),
        _lib.ptr(_lib.status_word(dev)), _lib.stream_ptr())
    _lib.check_rc(rc, "flash_bwd")
    return dq, dk, dv


def attn_delta_rows(o: torch.Tensor, dout: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``delta[t, h] = sum_d dO[t,h,d] * O[t,h,d]`` (fp32 [T, Hq]); ``o``/``dout``: [T, Hq, D]."""
    T, Hq, D = o.shape
    if not o.is_cuda:
        r = (o.float() * dout.float()).sum(-1)
        if out is not None:
            out.copy_(r); r = out
        return r
    if out is None:
        out = torch.empty(T, Hq, dtype=torch.float32, device=o.device)
    rc = _lib.lib().dca_attn_delta_rows(_lib.ptr(o), _lib.ptr(dout), _lib.ptr(out), _lib.c_long(T), _lib.c_int(Hq),
                                        _lib.c_int(D), _lib.c_long(o.stride(0)), _lib.c_long(dout.stride(0)),
                                        _lib.c_long(out.stride(0)), _lib.stream_ptr())
    _lib.check_rc(rc, "attn_delta_rows")
    return out


def dispatch_dout(o: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor, do_dst: torch.Tensor, do_off_bytes: int,
                  delta_dst: torch.Tensor, lse_dst: torch.Tensor) -> None:
    """Owner half of the backward dispatch as one kernel: ``delta = rowsum(dO o O)`` per head, then the dO row,
    the delta row and the log-sum-exp row of every token are stored at that token's destinations
    (``do_dst[t] + do_off_bytes``, ``delta_dst[t]``, ``lse_dst[t]``: device int64 addresses, possibly in other
    GPUs' arenas; 0 in ``do_dst`` skips the token). ``o`` / ``dout``: [T, Hq, 128] bf16; ``lse``: [T, Hq] fp32."""
    T, Hq, D = dout.shape
    rc = _lib.lib().dca_dispatch_dout(_lib.ptr(o), _lib.ptr(dout), _lib.ptr(lse), _lib.c_long(T), _lib.c_int(Hq),
                                      _lib.c_int(D), _lib.c_long(o.stride(0)), _lib.c_long(dout.stride(0)),
                                      _lib.c_long(lse.stride(0)), _lib.ptr(do_dst), _lib.c_long(do_off_bytes),
                                      _lib.ptr(delta_dst), _lib.ptr(lse_dst), _lib.stream_ptr())
    _lib.check_rc(rc, "dispatch_dout")
