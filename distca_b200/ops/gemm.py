"""bf16 GEMMs of the linear layers on the tcgen05 kernel (``csrc/gemm/gemm_tcgen05.cu``).

The three products of a linear layer ``y = x W^T`` map onto one kernel with different operand
majors (no transposes are ever materialised):

========  =======================  ====================================
product   math                     operands as the kernel sees them
========  =======================  ====================================
forward   ``y  = x @ W.T``          A = x  (K-major),  B = W (K-major)
dgrad     ``dx = dy @ W``           A = dy (K-major),  B = W (MN-major)
wgrad     ``dW = dy.T @ x``         A = dy (MN-major), B = x (MN-major)
========  =======================  ====================================

On CPU tensors (used by the tests of the engine logic and the gloo configuration) the same
functions evaluate with plain torch in the tensor's own dtype.
The reference gets these from TransformerEngine (distca/runtime/megatron/model_patch.py:89-112).
"""
from __future__ import annotations

import torch

from . import _lib

EPI_STORE = 0
EPI_SWIGLU = 1


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with unit inner stride, got {tuple(t.shape)} / {t.stride()}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bf16")


def gemm_raw(a, b, c, M, N, K, a_mn, b_mn, *, accumulate=False, epi=EPI_STORE, preact=None, residual=None):
    """Direct launcher. ``a``/``b`` are the stored 2-D tensors; pitches come from stride(0)."""
    L = _lib.lib()
    out_fp32 = 1 if c.dtype == torch.float32 else 0
    rc = L.dca_gemm_bf16(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(c), _lib.c_int(M), _lib.c_int(N), _lib.c_int(K),
        _lib.c_long(a.stride(0)), _lib.c_long(b.stride(0)), _lib.c_long(c.stride(0)),
        _lib.c_int(a_mn), _lib.c_int(b_mn), _lib.c_int(out_fp32), _lib.c_int(1 if accumulate else 0),
        _lib.c_int(epi), _lib.ptr(preact), _lib.c_long(0 if preact is None else preact.stride(0)),
        _lib.ptr(residual), _lib.c_long(0 if residual is None else residual.stride(0)),
        _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_bf16")
    return c


def linear_fwd(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
               residual: torch.Tensor | None = None) -> torch.Tensor:
    """``x[T,K] @ w[N,K].T (+ residual[T,N]) -> [T,N]``; ``out`` may alias ``residual``."""
    if not x.is_cuda:
        y = x @ w.t()
        if residual is not None:
            y = y + residual
        if out is not None:
            out.copy_(y)
            return out
        return y
    _check2d(x, "x"); _check2d(w, "w")
    T, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    return gemm_raw(x, w, out, T, N, K, 0, 0, residual=residual)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """``dy[T,N] @ w[N,K] -> [T,K]``."""
    if not dy.is_cuda:
        r = dy @ w
        if out is not None:
            if accumulate:
                out.add_(r)
            else:
                out.copy_(r)
            return out
        return r
    _check2d(dy, "dy"); _check2d(w, "w")
    T, N = dy.shape
    K = w.shape[1]
    if out is None:
        out = torch.empty(T, K, dtype=torch.bfloat16, device=dy.device)
        accumulate = False
    return gemm_raw(dy, w, out, T, K, N, 0, 1, accumulate=accumulate)


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """``dy[T,N].T @ x[T,K] -> [N,K]`` (``out`` may be bf16 or fp32; ``accumulate`` adds)."""
    if not dy.is_cuda:
        r = dy.t() @ x
        if out is not None:
            if accumulate:
                out.add_(r.to(out.dtype))
            else:
                out.copy_(r)
            return out
        return r
    _check2d(dy, "dy"); _check2d(x, "x")
    T, N = dy.shape
    K = x.shape[1]
    if out is None:
        out = torch.empty(N, K, dtype=torch.bfloat16, device=dy.device)
        accumulate = False
    return gemm_raw(dy, x, out, N, K, T, 1, 1, accumulate=accumulate)


def linear_swiglu_fwd(x: torch.Tensor, w_gate_up: torch.Tensor, *, keep_preact: bool = False):
    """FC1 with SwiGLU in the epilogue: ``silu(x Wg^T) * (x Wu^T)`` for ``w = [Wg; Wu]`` ([2F,K]).

    Returns ``(act[T,F], preact[T,2F] or None)``; ``preact`` holds the bf16 (gate | up) pair that
    the backward pass needs and is only written when ``keep_preact`` is set.
    """
    F2, K = w_gate_up.shape
    F = F2 // 2
    if not x.is_cuda:
        h = x @ w_gate_up.t()
        g, u = h[:, :F], h[:, F:]
        act = torch.nn.functional.silu(g) * u
        return act, (h if keep_preact else None)
    _check2d(x, "x"); _check2d(w_gate_up, "w")
    T = x.shape[0]
    act = torch.empty(T, F, dtype=torch.bfloat16, device=x.device)
    pre = torch.empty(T, F2, dtype=torch.bfloat16, device=x.device) if keep_preact else None
    gemm_raw(x, w_gate_up, act, T, F2, K, 0, 0, epi=EPI_SWIGLU, preact=pre)
    return act, pre


def linear_qkv_rope(x: torch.Tensor, w: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, heads_q: int,
                    heads_kv: int, *, write_local: bool = True, q_dst: torch.Tensor | None = None,
                    kv_dst: torch.Tensor | None = None, max_copies: int = 0, v_off_bytes: int = 0,
                    a_peers=None, a_rows_per_peer: int = 0) -> torch.Tensor | None:
    """QKV projection whose epilogue applies RoPE (head_dim 128, position ``pos[t]`` of each token
    inside its document) and stores the rows where core attention reads them: the returned local
    ``[T, (heads_q + 2 heads_kv) * 128]`` tensor (``write_local``) and / or the per-token destinations
    ``q_dst`` [T] / ``kv_dst`` [T, max_copies] (uint64 addresses, possibly in peer GPUs' arenas; the V
    row of a destination sits ``v_off_bytes`` behind its K row). With ``a_peers`` (ctypes array of
    ``len`` device addresses) the activation is read shard by shard from the peers' buffers."""
    import ctypes
    _check2d(w, "w")
    N, K = w.shape
    assert N == (heads_q + 2 * heads_kv) * 128 and table.shape[1] == 128 and table.dtype == torch.float32
    assert pos.dtype == torch.int32 and (write_local or q_dst is not None)
    if a_peers is None:
        _check2d(x, "x")
        T = x.shape[0]
        a_ptr, lda, n_peers = _lib.ptr(x), x.stride(0), 0
    else:
        T = a_rows_per_peer * len(a_peers)
        a_ptr, lda, n_peers = None, K, len(a_peers)
    out = torch.empty(T, N, dtype=torch.bfloat16, device=w.device) if write_local else None
    rc = _lib.lib().dca_gemm_qkv_rope(
        a_ptr, _lib.ptr(w), _lib.ptr(out), _lib.c_int(T), _lib.c_int(N), _lib.c_int(K), _lib.c_long(lda),
        _lib.c_long(w.stride(0)), _lib.c_long(N), _lib.ptr(pos), _lib.ptr(table), _lib.c_int(table.shape[0]),
        _lib.c_int(heads_q), _lib.c_int(heads_kv), _lib.ptr(q_dst), _lib.ptr(kv_dst), _lib.c_int(max_copies), _lib.c_long(v_off_bytes),
        a_peers, _lib.c_int(n_peers), _lib.c_long(a_rows_per_peer), _lib.ptr(_lib.status_word(w.device)),
        _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_qkv_rope")
    return out
