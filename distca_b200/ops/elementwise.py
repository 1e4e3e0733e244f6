"""Memory-bound ops: RMSNorm, SwiGLU, residual add, RoPE, cross-entropy, embedding, Adam.

Every function takes CUDA bf16 tensors to the sm_100a kernels in ``csrc/elementwise`` and CPU
tensors (any float dtype) to an equivalent PyTorch expression, which doubles as the oracle in the
GPU tests and runs the fp32 gloo configuration.

The reference takes these from TransformerEngine / Megatron / Apex (fused RMSNorm + linear and SwiGLU in
distca/runtime/megatron/model_patch.py:89-112, ``vocab_parallel_cross_entropy`` in pretrain_llama.py:228,
Megatron's distributed Adam in distca/utils/megatron_test_utils.py:102-113) and rotates in plain torch
(distca/runtime/megatron/distca_rope.py:24-68).
"""
from __future__ import annotations

import math

import torch

from . import _lib


# --------------------------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------------------------
def rmsnorm_fwd(x: torch.Tensor, g: torch.Tensor, eps: float, out: torch.Tensor | None = None):
    """Returns ``(y, rstd)`` with ``y = x * rsqrt(mean(x^2) + eps) * g``; ``rstd`` is fp32 [T]."""
    T, H = x.shape
    if not x.is_cuda:
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        y = (xf * rstd[:, None] * g.float()).to(x.dtype)
        if out is not None:
            out.copy_(y); y = out
        return y, rstd
    if out is None:
        out = torch.empty_like(x)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    rc = _lib.lib().dca_rmsnorm_fwd(_lib.ptr(x), _lib.ptr(g), _lib.ptr(out), _lib.ptr(rstd),
                                    _lib.c_int(T), _lib.c_int(H), _lib.c_float(eps), _lib.stream_ptr())
    _lib.check_rc(rc, "rmsnorm_fwd")
    return out, rstd


def rmsnorm_bwd(x, g, rstd, dy, dg_out: torch.Tensor, *, dres: torch.Tensor | None = None,
                dx_out: torch.Tensor | None = None, accumulate_dg: bool = True):
    """``dx = d(rmsnorm)/dx (+ dres)``; ``dg_out (+)= d/dg``. Returns dx."""
    T, H = x.shape
    if not x.is_cuda:
        xf, dyf, gf = x.float(), dy.float(), g.float()
        xh = xf * rstd[:, None]
        dyg = dyf * gf
        dx = rstd[:, None] * (dyg - xh * (dyg * xh).mean(-1, keepdim=True))
        if dres is not None:
            dx = dx + dres.float()
        dg = (dyf * xh).sum(0)
        if accumulate_dg:
            dg_out.add_(dg.to(dg_out.dtype))
        else:
            dg_out.copy_(dg)
        dx = dx.to(x.dtype)
        if dx_out is not None:
            dx_out.copy_(dx); dx = dx_out
        return dx
    L = _lib.lib()
    if dx_out is None:
        dx_out = torch.empty_like(x)
    P = L.dca_rmsnorm_bwd_partials(_lib.c_int(T))
    partial = torch.empty(P, H, dtype=torch.float32, device=x.device)
    rc = L.dca_rmsnorm_bwd(_lib.ptr(x), _lib.ptr(g), _lib.ptr(rstd), _lib.ptr(dy), _lib.ptr(dres),
                           _lib.ptr(dx_out), _lib.ptr(partial), _lib.ptr(dg_out),
                           _lib.c_int(1 if dg_out.dtype == torch.float32 else 0),
                           _lib.c_int(1 if accumulate_dg else 0), _lib.c_int(T), _lib.c_int(H),
                           _lib.stream_ptr())
    _lib.check_rc(rc, "rmsnorm_bwd")
    return dx_out


# --------------------------------------------------------------------------------------------
# SwiGLU / add
# --------------------------------------------------------------------------------------------
def swiglu_fwd(pre: torch.Tensor) -> torch.Tensor:
    """``pre`` [T, 2F] = (gate | up) -> silu(gate) * up."""
    T, F2 = pre.shape
    F = F2 // 2
    if not pre.is_cuda:
        return torch.nn.functional.silu(pre[:, :F]) * pre[:, F:]
    act = torch.empty(T, F, dtype=pre.dtype, device=pre.device)
    rc = _lib.lib().dca_swiglu_fwd(_lib.ptr(pre), _lib.ptr(act), _lib.c_long(T), _lib.c_int(F), _lib.stream_ptr())
    _lib.check_rc(rc, "swiglu_fwd")
    return act


def swiglu_bwd(pre: torch.Tensor, dact: torch.Tensor, inplace: bool = True) -> torch.Tensor:
    """Gradient w.r.t. (gate | up); overwrites ``pre`` when ``inplace``."""
    T, F2 = pre.shape
    F = F2 // 2
    if not pre.is_cuda:
        g, u = pre[:, :F].float(), pre[:, F:].float()
        s = torch.sigmoid(g)
        d = dact.float()
        out = torch.cat([d * u * s * (1 + g * (1 - s)), d * g * s], dim=1).to(pre.dtype)
        if inplace:
            pre.copy_(out)
            return pre
        return out
    out = pre if inplace else torch.empty_like(pre)
    rc = _lib.lib().dca_swiglu_bwd(_lib.ptr(pre), _lib.ptr(dact), _lib.ptr(out), _lib.c_long(T), _lib.c_int(F),
                                   _lib.stream_ptr())
    _lib.check_rc(rc, "swiglu_bwd")
    return out


def add_(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """In-place ``a += b`` (bf16 on GPU through the vectorised kernel)."""
    if not a.is_cuda or a.dtype != torch.bfloat16 or a.numel() % 8 or not a.is_contiguous() or not b.is_contiguous():
        return a.add_(b)
    rc = _lib.lib().dca_add_bf16(_lib.ptr(a), _lib.ptr(b), _lib.ptr(a), _lib.c_long(a.numel()), _lib.stream_ptr())
    _lib.check_rc(rc, "add")
    return a


# --------------------------------------------------------------------------------------------
# RoPE
# --------------------------------------------------------------------------------------------
def rope_table(max_pos: int, dim: int, theta: float, device) -> torch.Tensor:
    """fp32 [max_pos, dim] = (cos | sin) of pos * theta^(-2i/dim), i < dim/2."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=1).float().to(device)


def rope_(qkv: torch.Tensor, pos: torch.Tensor, table: torch.Tensor, heads_q: int, heads_kv: int,
          head_dim: int, backward: bool = False, *, q_dst=None, kv_dst=None, max_copies: int = 0,
          v_off_bytes: int = 0, write_inplace: bool = True) -> torch.Tensor:
    """Rotate the Q and K heads of ``qkv`` [T, (Hq+2Hkv)*D] in place (V untouched).

    With ``q_dst``/``kv_dst`` (device uint64 address tables) the rotated Q and K rows and the V rows
    are additionally scattered to those addresses (see ``csrc/elementwise/rope.cu``).
    """
    T = qkv.shape[0]
    D = head_dim
    if not qkv.is_cuda:
        assert q_dst is None
        half = D // 2
        n_rot = heads_q + heads_kv
        x = qkv[:, :n_rot * D].reshape(T, n_rot, D).float()
        cs = table[pos.long()].to(torch.float32)
        cos, sin = cs[:, None, :half], cs[:, None, half:]
        if backward:
            sin = -sin
        x1, x2 = x[..., :half], x[..., half:]
        out = torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
        qkv[:, :n_rot * D] = out.reshape(T, n_rot * D).to(qkv.dtype)
        return qkv
    assert pos.dtype == torch.int32 and table.dtype == torch.float32 and table.shape[1] == D
    rc = _lib.lib().dca_rope(_lib.ptr(qkv), _lib.ptr(pos), _lib.ptr(table), _lib.c_int(table.shape[0]), _lib.c_long(T),
                             _lib.c_int(heads_q), _lib.c_int(heads_kv), _lib.c_int(D), _lib.c_long(qkv.stride(0)),
                             _lib.c_int(1 if backward else 0), _lib.ptr(q_dst), _lib.ptr(kv_dst),
                             _lib.c_int(max_copies), _lib.c_long(v_off_bytes),
                             _lib.c_int(1 if write_inplace else 0), _lib.ptr(_lib.status_word(qkv.device)),
                             _lib.stream_ptr())
    _lib.check_rc(rc, "rope")
    return qkv


# --------------------------------------------------------------------------------------------
# cross entropy (vocabulary-parallel aware)
# --------------------------------------------------------------------------------------------
def ce_stats(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """Per-token (max, sum exp(x-max), target logit or 0) over this vocabulary slice: fp32 [T, 3]."""
    T, V = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        m = lf.max(-1).values
        s = (lf - m[:, None]).exp().sum(-1)
        local = labels - vocab_start
        ok = (local >= 0) & (local < V)
        tgt = torch.where(ok, lf.gather(1, local.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(m))
        return torch.stack([m, s, tgt], dim=1)
    assert logits.dtype == torch.float32 and labels.dtype == torch.int64
    stats = torch.empty(T, 3, dtype=torch.float32, device=logits.device)
    rc = _lib.lib().dca_ce_stats(_lib.ptr(logits), _lib.c_long(logits.stride(0)), _lib.ptr(labels),
                                 _lib.c_int(vocab_start), _lib.c_int(V), _lib.ptr(stats), _lib.c_long(T),
                                 _lib.stream_ptr())
    _lib.check_rc(rc, "ce_stats")
    return stats


def ce_grad(logits: torch.Tensor, labels: torch.Tensor, stats_all: torch.Tensor, grad_scale: float,
            vocab_start: int = 0, dlogits: torch.Tensor | None = None):
    """Returns ``(loss[T] fp32, dlogits)`` from the statistics of all slices ``stats_all`` [R,T,3].

    Tokens with a negative label contribute neither loss nor gradient.
    """
    T, V = logits.shape
    if stats_all.dim() == 2:
        stats_all = stats_all[None]
    R = stats_all.shape[0]
    if not logits.is_cuda:
        gm = stats_all[..., 0].max(0).values
        gs = (stats_all[..., 1] * (stats_all[..., 0] - gm).exp()).sum(0)
        tgt = stats_all[..., 2].sum(0)
        lse = gm + gs.log()
        valid = labels >= 0
        loss = torch.where(valid, lse - tgt, torch.zeros_like(lse))
        g = (logits.float() - lse[:, None]).exp()
        local = labels - vocab_start
        ok = valid & (local >= 0) & (local < V)
        rows = torch.nonzero(ok)[:, 0]
        g[rows, local[rows]] -= 1.0
        g = g * (valid[:, None].float() * grad_scale)
        g = g.to(logits.dtype if dlogits is None else dlogits.dtype)
        if dlogits is not None:
            dlogits.copy_(g); g = dlogits
        return loss, g
    if dlogits is None:
        dlogits = torch.empty(T, V, dtype=torch.bfloat16, device=logits.device)
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    stats_all = stats_all.contiguous()
    rc = _lib.lib().dca_ce_grad(_lib.ptr(logits), _lib.c_long(logits.stride(0)), _lib.ptr(labels),
                                _lib.c_int(vocab_start), _lib.c_int(V), _lib.ptr(stats_all), _lib.c_int(R),
                                _lib.c_long(T), _lib.c_float(grad_scale), _lib.ptr(dlogits),
                                _lib.c_long(dlogits.stride(0)), _lib.ptr(loss), _lib.stream_ptr())
    _lib.check_rc(rc, "ce_grad")
    return loss, dlogits


# --------------------------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------------------------
def embedding_fwd(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    T = ids.shape[0]
    V, H = table.shape
    if not table.is_cuda:
        local = ids - vocab_start
        ok = (local >= 0) & (local < V)
        out = table[local.clamp(0, V - 1)]
        return out * ok[:, None].to(out.dtype)
    out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    rc = _lib.lib().dca_embedding_fwd(_lib.ptr(ids), _lib.ptr(table), _lib.ptr(out), _lib.c_long(T), _lib.c_int(H),
                                      _lib.c_int(vocab_start), _lib.c_int(V), _lib.stream_ptr())
    _lib.check_rc(rc, "embedding_fwd")
    return out


def embedding_bwd(ids: torch.Tensor, dout: torch.Tensor, dtable: torch.Tensor, vocab_start: int = 0,
                  accumulate: bool = True) -> torch.Tensor:
    """``dtable[id] (+)= sum of dout rows with that id`` (deterministic)."""
    T = ids.shape[0]
    V, H = dtable.shape
    if not dtable.is_cuda:
        local = ids - vocab_start
        ok = (local >= 0) & (local < V)
        if not accumulate:
            dtable.zero_()
        dtable.index_add_(0, local[ok], dout[ok].to(dtable.dtype))
        return dtable
    if not accumulate:
        dtable.zero_()
    sorted_ids, order = torch.sort(ids)
    rc = _lib.lib().dca_embedding_bwd(_lib.ptr(sorted_ids), _lib.ptr(order), _lib.ptr(dout), _lib.ptr(dtable),
                                      _lib.c_int(1 if dtable.dtype == torch.float32 else 0), _lib.c_int(1),
                                      _lib.c_long(T), _lib.c_int(H), _lib.c_int(vocab_start), _lib.c_int(V),
                                      _lib.stream_ptr())
    _lib.check_rc(rc, "embedding_bwd")
    return dtable


# --------------------------------------------------------------------------------------------
# optimizer pieces
# --------------------------------------------------------------------------------------------
def sumsq_(g: torch.Tensor, acc: torch.Tensor) -> torch.Tensor:
    """``acc[0] += sum(g^2)`` without leaving the device (``acc`` fp32 [>=1])."""
    if not g.is_cuda:
        acc[0] += g.float().pow(2).sum()
        return acc
    g = g.reshape(-1)
    rc = _lib.lib().dca_sumsq(_lib.ptr(g), _lib.c_int(1 if g.dtype == torch.float32 else 0), _lib.c_long(g.numel()),
                              _lib.ptr(acc), _lib.stream_ptr())
    _lib.check_rc(rc, "sumsq")
    return acc


def adam_step_(param: torch.Tensor, lo16: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
               *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float, step: int,
               gscale: torch.Tensor | None = None) -> None:
    """AdamW on flat tensors. GPU: ``param`` bf16 + ``lo16`` int16 form the exact fp32 master.
    CPU: ``param`` is the fp32 master itself and ``lo16`` is ignored."""
    n = param.numel()
    if not param.is_cuda:
        g = grad.float() * (1.0 if gscale is None else float(gscale[0]))
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        w = param.float()
        upd = (m / bc1) / ((v / bc2).sqrt() + eps) + weight_decay * w
        param.copy_((w - lr * upd).to(param.dtype))
        return
    assert param.dtype == torch.bfloat16 and lo16.dtype == torch.int16
    rc = _lib.lib().dca_adam(_lib.ptr(param), _lib.ptr(lo16), _lib.ptr(grad),
                             _lib.c_int(1 if grad.dtype == torch.float32 else 0), _lib.ptr(m), _lib.ptr(v),
                             _lib.c_long(n), _lib.c_float(lr), _lib.c_float(beta1), _lib.c_float(beta2),
                             _lib.c_float(eps), _lib.c_float(weight_decay), _lib.c_int(step), _lib.ptr(gscale),
                             _lib.ptr(_lib.status_word(param.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "adam")


def master_from_split(param_bf16: torch.Tensor, lo16: torch.Tensor) -> torch.Tensor:
    """Reassemble the fp32 master weights kept as (bf16 | int16 remainder)."""
    hi = param_bf16.view(torch.int16).to(torch.int32) << 16
    return (hi + lo16.to(torch.int32)).view(torch.float32)
