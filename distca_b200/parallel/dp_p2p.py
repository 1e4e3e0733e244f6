"""Data-parallel gradient reduction and parameter all-gather over peer memory, fused with the
work that follows / precedes them (``csrc/comm/p2p.cu``, ``csrc/elementwise/loss_optim.cu``):

* ``reduce_scatter_sumsq``: every rank pulls its parameter-shard slice of all peers' bf16 gradient
  buffers over NVLink, sums in fp32, writes the result in place and accumulates the squared norm
  of the reduced shard in the same pass (what the global-norm clip needs).
* ``adam_push``: the AdamW update of the shard stores the new bf16 parameters directly into every
  peer's flat parameter buffer, so the update IS the all-gather.

Parameter and gradient buffers therefore live in a :class:`PeerArena` of the data-parallel group.
The reference leaves both collectives to Megatron's DistributedOptimizer over NCCL
(distca/utils/megatron_test_utils.py:235-258).
"""
from __future__ import annotations

import torch

from ..ops import _lib
from .p2p import PeerArena, SignalBoard


class PeerDataParallel:
    def __init__(self, group, device, numel: int, grad_dtype=torch.bfloat16):
        """``grad_dtype``: bf16 (one micro-batch per step: the weight-gradient GEMMs round once) or fp32
        (several micro-batches accumulate; the reference's ``grad_reduce_in_fp32``)."""
        self.device = torch.device(device)
        nbytes = numel * 2
        gbytes = numel * (4 if grad_dtype == torch.float32 else 2)
        self.grad_dtype = grad_dtype
        self.arena = PeerArena(nbytes + gbytes + (1 << 20), group, device)
        self.size, self.rank = self.arena.size, self.arena.rank
        self.sig = SignalBoard(self.arena, 3)      # 0: backward complete, 1: parameters pushed, 2: bucket complete
        self.side = torch.cuda.Stream(self.device)  # bucket reductions run here, beside the rest of backward
        self.off_param = self.arena.alloc(nbytes, align=4096)
        self.off_grad = self.arena.alloc(gbytes, align=4096)
        self.flat = self.arena.view(self.off_param, (numel,), torch.bfloat16)
        self.grad = self.arena.view(self.off_grad, (numel,), grad_dtype)
        self.param_tbl = torch.tensor([self.arena.addr(p, self.off_param) for p in range(self.size)],
                                      dtype=torch.int64, device=device)
        self.grad_tbl = torch.tensor([self.arena.addr(p, self.off_grad) for p in range(self.size)],
                                     dtype=torch.int64, device=device)

    def reduce_scatter_sumsq(self, lo: int, n: int, sumsq: torch.Tensor) -> None:
        """own_grad[lo:lo+n] = sum over ranks; ``sumsq[0] += ||that||^2``. Collective over the group."""
        self.sig.signal(0)      # my backward is complete (stream order) ...
        self.sig.wait(0)        # ... and so is everybody else's
        fn = (_lib.lib().dca_reduce_scatter_sumsq_f32 if self.grad_dtype == torch.float32
              else _lib.lib().dca_reduce_scatter_sumsq_bf16)
        rc = fn(_lib.ptr(self.grad_tbl), _lib.c_int(self.size), _lib.c_int(self.rank),
                _lib.c_long(lo), _lib.c_long(n), _lib.ptr(sumsq), _lib.stream_ptr())
        _lib.check_rc(rc, "reduce_scatter_sumsq")

    def _reduce(self, lo: int, n: int, sumsq: torch.Tensor) -> None:
        fn = (_lib.lib().dca_reduce_scatter_sumsq_f32 if self.grad_dtype == torch.float32
              else _lib.lib().dca_reduce_scatter_sumsq_bf16)
        rc = fn(_lib.ptr(self.grad_tbl), _lib.c_int(self.size), _lib.c_int(self.rank),
                _lib.c_long(lo), _lib.c_long(n), _lib.ptr(sumsq), _lib.stream_ptr())
        _lib.check_rc(rc, "reduce_scatter_sumsq")

    def bucket_ready(self, ranges: list[tuple[int, int]], sumsq: torch.Tensor) -> None:
        """The gradients of one bucket (a layer) are final on this rank: on the side stream, tell the peers,
        wait until theirs are final too, and reduce the parts ``ranges`` = [(lo, n), ...] of the bucket that
        belong to this rank's shard (possibly none), while the main stream goes on with the next layer's
        backward. Every rank calls this for every bucket, in the same order."""
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            self.sig.signal(2)
            self.sig.wait(2)
            for lo, n in ranges:
                self._reduce(lo, n, sumsq)

    def join_buckets(self) -> None:
        """Make the current stream wait for the bucket reductions queued so far."""
        torch.cuda.current_stream(self.device).wait_stream(self.side)

    def adam_push(self, pshard, lo16, gshard, m, v, lo: int, *, lr, beta1, beta2, eps, weight_decay, step, gscale) -> None:
        rc = _lib.lib().dca_adam_push(_lib.ptr(pshard), _lib.ptr(lo16), _lib.ptr(gshard),
                                      _lib.c_int(1 if gshard.dtype == torch.float32 else 0), _lib.ptr(m), _lib.ptr(v),
                                      _lib.c_long(pshard.numel()), _lib.c_float(lr), _lib.c_float(beta1),
                                      _lib.c_float(beta2), _lib.c_float(eps), _lib.c_float(weight_decay), _lib.c_int(step),
                                      _lib.ptr(gscale), _lib.ptr(self.param_tbl), _lib.c_int(self.size), _lib.c_long(lo),
                                      _lib.ptr(_lib.status_word(pshard.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "adam_push")
        self.sig.signal(1)      # my shard has been stored everywhere, and I no longer read peers' gradients
        self.sig.wait(1)        # everybody's shard has arrived here; peers are done with my gradient buffer

    def close(self) -> None:
        self.flat = self.grad = None
        self.arena.close()
