"""Tensor-parallel collectives fused into the GEMMs, over peer memory (NVLink).

* ``ag_linear``  (all-gather -> GEMM): every rank leaves its [T/tp, K] activation shard in its arena;
  the GEMM's TMA producer loads each A tile straight from the arena of the rank that owns those
  rows, so the gathered [T, K] activation never exists in memory and the transfer overlaps the
  math tile by tile. TMA loads of peer memory are plain (non-multicast) loads.
* ``linear_rs``  (GEMM -> reduce-scatter): the GEMM epilogue stores each output row directly into the
  slot buffer of the rank that owns the row (``slots[src_rank]`` in that rank's arena); the owner
  then sums the tp slots (plus the residual) in one pass.

Synchronisation uses the arena's monotonic signals: "my shard / my partial rows are in place" and
"I have finished reading" per operation, so buffers are reused safely from call to call.

The reference gets both collectives from TransformerEngine + NCCL
(distca/runtime/megatron/model_patch.py:77-98, sequence_parallel = tp > 1).
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..ops import elementwise as ew
from .p2p import PeerArena, SignalBoard, sum_slots

SIG_STAGED, SIG_READ, SIG_PARTIAL, SIG_SUMMED, SIG_GIN, SIG_GDONE = 0, 1, 2, 3, 4, 5


class PeerCollectives:
    def __init__(self, group, size: int, rank: int, device, max_rows_local: int, max_cols: int,
                 tile_loads: bool = False):
        """``max_rows_local``: largest T/tp; ``max_cols``: largest K of ``ag_linear`` / N of ``linear_rs``.
        ``tile_loads``: the model's all-gather -> GEMM sites use :meth:`ag_linear` / :meth:`ag_linear_swiglu`
        (every CTA loads the remote tiles it needs: a remote tile crosses NVLink once per N tile that uses it)
        instead of :meth:`all_gather_rows` + a local GEMM (every shard crosses once)."""
        self.tile_loads = tile_loads
        self.size, self.rank = size, rank
        self.device = torch.device(device)
        self.max_rows, self.max_cols = max_rows_local, max_cols
        shard = max_rows_local * max_cols * 2
        self.arena = PeerArena(shard * (1 + 2 * size) + (1 << 20), group, device)
        self.sig = SignalBoard(self.arena, 6)
        self.off_x = self.arena.alloc(shard, align=4096)
        self.off_slots = self.arena.alloc(shard * size, align=4096)
        self.off_gather = self.arena.alloc(shard * size, align=4096)
        self.x_addrs = [self.arena.addr(p, self.off_x) for p in range(size)]
        self.gather_tbl = torch.tensor([self.arena.addr(p, self.off_gather) for p in range(size)],
                                       dtype=torch.int64, device=self.device)
        self._valid = None

    # ------------------------------------------------------------------------------------------
    def stage_buffer(self, rows: int, cols: int) -> torch.Tensor:
        """This rank's shard buffer in the arena ([rows, cols] bf16); write the activation shard here
        (e.g. as the output of RMSNorm) before calling :meth:`ag_linear`."""
        assert rows <= self.max_rows and cols <= self.max_cols
        self.sig.wait(SIG_READ)   # every peer has finished reading what was staged before
        return self.arena.view(self.off_x, (rows, cols), torch.bfloat16)

    def ag_linear(self, x_staged: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                  rope: dict | None = None, transposed_weight: bool = False) -> torch.Tensor:
        """``concat_over_ranks(x_staged) @ w.T`` with the all-gather fused into the GEMM's operand load.
        ``x_staged`` must be the tensor returned by :meth:`stage_buffer` (already filled).
        ``transposed_weight``: ``concat(...) @ w`` instead (``w`` [K, N]: the data-gradient twin of a
        row-parallel linear, e.g. ``dattn = all_gather(dh) @ W_o``)."""
        rows, K = x_staged.shape
        N = w.shape[1] if transposed_weight else w.shape[0]
        assert rope is None or not transposed_weight
        T = rows * self.size
        if out is None:
            out = torch.empty(T, N, dtype=torch.bfloat16, device=self.device)
        self.sig.signal(SIG_STAGED)
        self.sig.wait(SIG_STAGED)
        a_peers = (ctypes.c_void_p * self.size)(*self.x_addrs)
        if rope is not None:
            # QKV projection: RoPE (+ core-attention dispatch) in the epilogue of the same GEMM
            from ..ops import gemm
            out = gemm.linear_qkv_rope(None, w, a_peers=a_peers, a_rows_per_peer=rows, **rope)
            self.sig.signal(SIG_READ)
            return out
        rc = _lib.lib().dca_gemm_bf16_tp(
            None, _lib.ptr(w), _lib.ptr(out), _lib.c_int(T), _lib.c_int(N), _lib.c_int(K), _lib.c_long(K),
            _lib.c_long(w.stride(0)), _lib.c_long(out.stride(0)), _lib.c_int(1 if transposed_weight else 0), a_peers,
            _lib.c_int(self.size), _lib.c_long(rows), None, _lib.c_int(0), _lib.c_long(0),
            _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "gemm_ag")
        self.sig.signal(SIG_READ)
        return out

    def ag_linear_swiglu(self, x_staged: torch.Tensor, w_gate_up: torch.Tensor, keep_preact: bool = False):
        """FC1: ``silu(gate) * up`` of ``concat_over_ranks(x_staged) @ w_gate_up.T`` with the all-gather fused
        into the GEMM's operand load and SwiGLU in its epilogue. Returns ``(act, pre or None)``."""
        rows, K = x_staged.shape
        F2 = w_gate_up.shape[0]
        T = rows * self.size
        act = torch.empty(T, F2 // 2, dtype=torch.bfloat16, device=self.device)
        pre = torch.empty(T, F2, dtype=torch.bfloat16, device=self.device) if keep_preact else None
        self.sig.signal(SIG_STAGED)
        self.sig.wait(SIG_STAGED)
        a_peers = (ctypes.c_void_p * self.size)(*self.x_addrs)
        rc = _lib.lib().dca_gemm_swiglu_tp(
            _lib.ptr(w_gate_up), _lib.ptr(act), _lib.c_int(T), _lib.c_int(F2), _lib.c_int(K), _lib.c_long(K),
            _lib.c_long(w_gate_up.stride(0)), _lib.c_long(F2 // 2), _lib.ptr(pre), _lib.c_long(F2), a_peers,
            _lib.c_int(self.size), _lib.c_long(rows), _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "gemm_ag_swiglu")
        self.sig.signal(SIG_READ)
        return act, pre

    def linear_rs(self, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None,
                  transposed_weight: bool = False) -> torch.Tensor:
        """``reduce_scatter_rows(x @ w.T) (+ residual)`` with the scatter fused into the GEMM epilogue.
        ``transposed_weight``: ``x @ w`` instead (``w`` [K, N]: the data-gradient twin of a column-parallel
        linear, e.g. ``dn = reduce_scatter(dqkv @ W_qkv)``)."""
        T, K = x.shape
        N = w.shape[1] if transposed_weight else w.shape[0]
        rows = T // self.size
        assert rows <= self.max_rows and N <= self.max_cols
        self.sig.wait(SIG_SUMMED)  # every owner has consumed the previous partial rows
        slot_bytes = self.max_rows * self.max_cols * 2
        c_peers = (ctypes.c_void_p * self.size)(*[self.arena.addr(p, self.off_slots + self.rank * slot_bytes)
                                                 for p in range(self.size)])
        rc = _lib.lib().dca_gemm_bf16_tp(
            _lib.ptr(x), _lib.ptr(w), None, _lib.c_int(T), _lib.c_int(N), _lib.c_int(K), _lib.c_long(x.stride(0)),
            _lib.c_long(w.stride(0)), _lib.c_long(N), _lib.c_int(1 if transposed_weight else 0), None, _lib.c_int(0),
            _lib.c_long(0), c_peers, _lib.c_int(self.size), _lib.c_long(rows), _lib.ptr(_lib.status_word(self.device)),
            _lib.stream_ptr())
        _lib.check_rc(rc, "gemm_rs")
        self.sig.signal(SIG_PARTIAL)
        self.sig.wait(SIG_PARTIAL)
        slots = self.arena.local[self.off_slots:self.off_slots + self.size * slot_bytes].view(torch.bfloat16)
        slots = slots.view(self.size, self.max_rows * self.max_cols)[:, :rows * N].unflatten(1, (rows, N))
        if self._valid is None or self._valid.shape[0] < rows:
            self._valid = torch.zeros(self.max_rows, self.size, dtype=torch.int32, device=self.device)
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=self.device)
        sum_slots(slots, self._valid[:rows], out)
        if residual is not None:
            ew.add_(out, residual)
        self.sig.signal(SIG_SUMMED)
        return out

    # ------------------------------------------------------------------------------------------
    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        """All-gather of row shards by peer stores (this repository's push kernel over NVLink, no NCCL): every
        rank stores its [rows, cols] shard into every peer's gather buffer. Returns the gathered
        [size * rows, cols] view of THIS rank's gather buffer; call :meth:`release_gather` once the kernels that
        read it are queued (the next gather waits until every peer has released)."""
        rows, cols = x.shape
        assert rows <= self.max_rows and cols <= self.max_cols and x.dtype == torch.bfloat16
        x = x.contiguous()
        nbytes = rows * cols * 2
        self.sig.wait(SIG_GDONE)          # every peer has finished reading the previous gather
        mine = self.arena.view(self.off_gather + self.rank * nbytes, (rows, cols), torch.bfloat16)
        mine.copy_(x)
        rc = _lib.lib().dca_push_shard(_lib.ptr(x), _lib.ptr(self.gather_tbl), _lib.c_int(self.size), _lib.c_int(self.rank),
                                       _lib.c_long(self.rank * nbytes), _lib.c_long(nbytes), _lib.stream_ptr())
        _lib.check_rc(rc, "push_shard")
        self.sig.signal(SIG_GIN)
        self.sig.wait(SIG_GIN)
        return self.arena.view(self.off_gather, (self.size * rows, cols), torch.bfloat16)

    def release_gather(self) -> None:
        self.sig.signal(SIG_GDONE)

    def close(self) -> None:
        self.arena.close()
