"""Llama-family decoder with hand-written forward AND backward (no autograd on the hot path).

The layer is cut exactly where core-attention disaggregation cuts it:

    pre-CA   : RMSNorm -> QKV GEMM -> RoPE               (stays with the tokens)
    CA       : softmax(QK^T)V per document                (stateless; any attention server)
    post-CA  : out-proj GEMM + residual -> RMSNorm -> FC1 GEMM with SwiGLU epilogue -> FC2 GEMM + residual

``core_attn`` is a pluggable object (local attention, or the CAD runtime that ships Q/K/V to
attention servers and receives O back), mirroring the reference's split of
``TransformerLayer`` into ``_forward_pre_core_attn / _forward_core_attn / _forward_post_core_attn``
(distca/runtime/megatron/base_transformer_layer.py:320-660).

Parameters live in one flat buffer per rank (bf16 on GPU) with a same-shaped flat gradient
buffer, so the data-parallel reduce-scatter, the sharded Adam update and the parameter
all-gather each run over contiguous ranges. Names follow Megatron ``GPTModel`` so checkpoints
can be written in that layout.

Activation policy ``recompute="full"`` keeps only each layer's input and re-runs the layer's
forward inside the backward pass (the reference's full-recompute configuration); ``"none"``
keeps everything; ``"keep_attn"`` is full recompute except core attention: each layer's attention
output (and the softmax statistics) is stored in HBM or pinned host memory, so the quadratic part
of the layer runs once forward and once backward (pipeline stages keep the outputs of every
micro-batch in flight in HBM).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import gemm
from ..utils import timers
from .config import ModelConfig


# ---------------------------------------------------------------------------------------------
# parameters
# ---------------------------------------------------------------------------------------------
def param_shapes(cfg: ModelConfig, tp: int = 1, layer_range: tuple[int, int] | None = None,
                 first_stage: bool = True, last_stage: bool = True) -> list[tuple[str, tuple[int, ...]]]:
    """Ordered (Megatron name, local shape) list for one pipeline stage / tensor-parallel rank."""
    H = cfg.hidden
    lo, hi = layer_range if layer_range is not None else (0, cfg.num_layers)
    out: list[tuple[str, tuple[int, ...]]] = []
    if first_stage:
        out.append(("embedding.word_embeddings.weight", (cfg.vocab // tp, H)))
    for l in range(lo, hi):
        p = f"decoder.layers.{l}."
        out += [
            (p + "self_attention.linear_qkv.layer_norm_weight", (H,)),
            (p + "self_attention.linear_qkv.weight", (cfg.qkv_dim // tp, H)),
            *([(p + "self_attention.linear_qkv.bias", (cfg.qkv_dim // tp,))] if cfg.qkv_bias else []),
            (p + "self_attention.linear_proj.weight", (H, cfg.q_dim // tp)),
            (p + "mlp.linear_fc1.layer_norm_weight", (H,)),
            (p + "mlp.linear_fc1.weight", (2 * cfg.ffn // tp, H)),
            (p + "mlp.linear_fc2.weight", (H, cfg.ffn // tp)),
        ]
    if last_stage:
        out.append(("decoder.final_layernorm.weight", (H,)))
        if not cfg.tie_embeddings or not first_stage:
            out.append(("output_layer.weight", (cfg.vocab // tp, H)))
    return out


class ParamStore:
    """Flat parameter + gradient buffers with named views."""

    ALIGN = 128  # elements; keeps every view 256-byte aligned for TMA

    def __init__(self, shapes, device, dtype=torch.bfloat16, grad_dtype=torch.bfloat16, pad_to: int = 1,
                 buffers=None):
        """``buffers``: optional callable ``numel -> (flat, grad)`` that provides the two flat buffers
        (e.g. views of a peer-mapped arena) instead of ordinary allocations."""
        self.shapes = list(shapes)
        self.offsets: dict[str, tuple[int, int]] = {}
        off = 0
        for name, shp in self.shapes:
            n = math.prod(shp)
            self.offsets[name] = (off, n)
            off += (n + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        unit = self.ALIGN * pad_to
        self.numel = (off + unit - 1) // unit * unit
        if buffers is not None:
            self.flat, self.grad = buffers(self.numel)
            assert self.flat.dtype == dtype and self.flat.numel() == self.numel and self.grad.numel() == self.numel
            self.flat.zero_(); self.grad.zero_()
        else:
            self.flat = torch.zeros(self.numel, dtype=dtype, device=device)
            self.grad = torch.zeros(self.numel, dtype=grad_dtype, device=device)
        self.p: dict[str, torch.Tensor] = {}
        self.g: dict[str, torch.Tensor] = {}
        for name, shp in self.shapes:
            o, n = self.offsets[name]
            self.p[name] = self.flat[o:o + n].view(*shp)
            self.g[name] = self.grad[o:o + n].view(*shp)

    def init_weights(self, std: float, seed: int) -> None:
        gen = torch.Generator(device=self.flat.device)
        for i, (name, shp) in enumerate(self.shapes):
            if name.endswith("layer_norm_weight") or name.endswith("layernorm.weight"):
                self.p[name].fill_(1.0)
            elif name.endswith(".bias"):
                gen.manual_seed(seed * 1000003 + i)   # small random bias so that tests exercise it
                self.p[name].copy_(torch.randn(shp, generator=gen, device=self.flat.device, dtype=torch.float32) * std)
            else:
                gen.manual_seed(seed * 1000003 + i)
                self.p[name].copy_(torch.randn(shp, generator=gen, device=self.flat.device,
                                               dtype=torch.float32) * std)

    def zero_grad(self) -> None:
        self.grad.zero_()


def shard_full_tensor(name: str, full: torch.Tensor, cfg: ModelConfig, tp: int, tp_rank: int) -> torch.Tensor:
    """Slice a full (unsharded, this repository's row order) tensor for one tensor-parallel rank."""
    if tp == 1 or (full.dim() == 1 and not name.endswith("linear_qkv.bias")):
        return full
    if name.endswith("linear_qkv.weight") or name.endswith("linear_qkv.bias"):
        q, k, v = full.split([cfg.q_dim, cfg.kv_dim, cfg.kv_dim], dim=0)
        return torch.cat([t.chunk(tp, 0)[tp_rank] for t in (q, k, v)], dim=0)
    if name.endswith("linear_fc1.weight"):
        g, u = full.chunk(2, 0)
        return torch.cat([g.chunk(tp, 0)[tp_rank], u.chunk(tp, 0)[tp_rank]], dim=0)
    if name.endswith("linear_proj.weight") or name.endswith("linear_fc2.weight"):
        return full.chunk(tp, 1)[tp_rank]
    return full.chunk(tp, 0)[tp_rank]  # embedding / output layer: vocabulary-parallel


# ---------------------------------------------------------------------------------------------
# tensor-parallel hooks (identity when tp == 1)
# ---------------------------------------------------------------------------------------------
class NoTP:
    """Sequence-parallel collectives of a tensor-parallel group of size 1."""
    size = 1
    rank = 0

    def all_gather_rows(self, x):
        return x

    def reduce_scatter_rows(self, x):
        return x

    def all_gather_stats(self, s):
        return s[None]

    def all_reduce_(self, x):
        return x


# ---------------------------------------------------------------------------------------------
# core attention, local flavour
# ---------------------------------------------------------------------------------------------
class TwoPhaseCoreAttention:
    """Default split of a core-attention module's calls into the halves a ping-pong schedule
    interleaves (dispatch / serve / collect). Modules without communication run everything in the
    first half; :class:`~distca_b200.parallel.cad.CadRuntime` overrides these with real halves."""

    def no_tokens_dispatch(self) -> None:
        pass

    def qkv_epilogue(self):
        """Arguments for the QKV GEMM's RoPE / dispatch epilogue, or ``None`` when this module wants
        the plain projection followed by :meth:`apply_rope`."""
        return None

    def qkv_dispatched(self) -> None:
        """Called after a QKV GEMM that used :meth:`qkv_epilogue` (stand-in for ``apply_rope``'s signal)."""

    def forward_begin(self, qkv, layer: int = 0) -> None:
        self._fwd_result = self.forward(qkv, layer) if qkv is not None else self.forward_no_tokens(layer)

    def forward_end(self):
        r, self._fwd_result = self._fwd_result, None
        return r

    def forward_no_tokens(self, layer: int = 0):
        return None, None

    def restore_no_tokens(self, layer: int = 0) -> None:
        pass

    def backward_dispatch(self, ctx, dattn, layer: int = 0) -> None:
        self._bwd_args = (ctx, dattn, layer)

    def backward_serve(self, layer: int = 0) -> None:
        ctx, dattn, layer = self._bwd_args
        self._bwd_result = self.backward(ctx, dattn, layer) if dattn is not None else self.backward_no_tokens(layer)

    def backward_end(self):
        r, self._bwd_result = self._bwd_result, None
        return r

    def backward_no_tokens(self, layer: int = 0):
        return None


class LocalCoreAttention(TwoPhaseCoreAttention):
    """Core attention on the rank that owns the tokens (no disaggregation)."""

    def __init__(self, cfg: ModelConfig, tp: int = 1):
        self.hq = cfg.heads_q // tp
        self.hkv = cfg.heads_kv // tp
        self.D = cfg.head_dim
        self.plan: attn_ops.AttnPlan | None = None
        self.scratch = attn_ops.BwdScratch()

    def set_batch(self, plan: attn_ops.AttnPlan) -> None:
        self.plan = plan

    def apply_rope(self, qkv, pos, table) -> None:
        ew.rope_(qkv, pos, table, self.hq, self.hkv, self.D)

    def qkv_epilogue(self):
        return {"write_local": True}

    def _split(self, qkv):
        T = qkv.shape[0]
        qd, kd = self.hq * self.D, self.hkv * self.D
        q = qkv[:, :qd].unflatten(1, (self.hq, self.D))
        k = qkv[:, qd:qd + kd].unflatten(1, (self.hkv, self.D))
        v = qkv[:, qd + kd:].unflatten(1, (self.hkv, self.D))
        return q, k, v

    def forward(self, qkv: torch.Tensor, layer: int = 0):
        q, k, v = self._split(qkv)
        o, lse = attn_ops.flash_fwd(q, k, v, self.plan)
        return o.flatten(1), (qkv, o, lse)

    def pack_saved(self, attn_out: torch.Tensor, ctx) -> torch.Tensor:
        """What ``keep_attn`` stores per layer: O and the softmax statistics side by side,
        [T, hq * D + 2 * hq] in the activation dtype (the fp32 statistics are stored as raw bits)."""
        lse = ctx[2]
        if attn_out.dtype == torch.bfloat16:
            return torch.cat([attn_out, lse.contiguous().view(torch.bfloat16)], dim=1)
        return torch.cat([attn_out, lse.to(attn_out.dtype)], dim=1)      # CPU fp32 / fp64 configurations

    def restore(self, qkv: torch.Tensor, saved: torch.Tensor, layer: int = 0):
        """Context for :meth:`backward` from what :meth:`pack_saved` stored: core attention is not recomputed."""
        qd = self.hq * self.D
        o = saved[:, :qd]
        lse = saved[:, qd:].contiguous()
        lse = lse.view(torch.float32) if saved.dtype == torch.bfloat16 else lse.float()
        return o, (qkv, o.unflatten(1, (self.hq, self.D)), lse)

    def backward(self, ctx, dattn: torch.Tensor, layer: int = 0) -> torch.Tensor:
        qkv, o, lse = ctx
        q, k, v = self._split(qkv)
        dqkv = torch.zeros_like(qkv) if not qkv.is_cuda else torch.empty_like(qkv)
        dq, dk, dv = self._split(dqkv)
        do = dattn.unflatten(1, (self.hq, self.D))
        if qkv.is_cuda:
            attn_ops.flash_bwd(q, k, v, o, lse, do, self.plan, dq=dq, dk=dk, dv=dv, scratch=self.scratch)
        else:
            gq, gk, gv = attn_ops.flash_bwd(q, k, v, o, lse, do, self.plan)
            dq.copy_(gq); dk.copy_(gk); dv.copy_(gv)
        return dqkv


# ---------------------------------------------------------------------------------------------
# one transformer layer, forward and backward by hand
# ---------------------------------------------------------------------------------------------
@dataclass
class LayerCtx:
    x: torch.Tensor
    rstd1: torch.Tensor
    n1: torch.Tensor
    ca_ctx: object
    attn_out: torch.Tensor
    h: torch.Tensor
    rstd2: torch.Tensor
    n2: torch.Tensor
    pre: torch.Tensor
    act: torch.Tensor


def _on(streams, k: int):
    """Context that queues what follows on ``streams[k]`` (no-op without streams)."""
    import contextlib
    return torch.cuda.stream(streams[k]) if streams is not None else contextlib.nullcontext()


class LlamaLayer:
    def __init__(self, cfg: ModelConfig, store: ParamStore, index: int, tp=None):
        self.cfg, self.index = cfg, index
        self.tp = tp or NoTP()
        p = f"decoder.layers.{index}."
        self.names = {
            "ln1": p + "self_attention.linear_qkv.layer_norm_weight",
            "wqkv": p + "self_attention.linear_qkv.weight",
            **({"bqkv": p + "self_attention.linear_qkv.bias"} if cfg.qkv_bias else {}),
            "wo": p + "self_attention.linear_proj.weight",
            "ln2": p + "mlp.linear_fc1.layer_norm_weight",
            "w13": p + "mlp.linear_fc1.weight",
            "w2": p + "mlp.linear_fc2.weight",
        }
        self.w = {k: store.p[n] for k, n in self.names.items()}
        self.g = {k: store.g[n] for k, n in self.names.items()}
        self.hq = cfg.heads_q // self.tp.size
        self.hkv = cfg.heads_kv // self.tp.size
        self.fuse_rope = True   # QKV GEMM epilogue does RoPE (+ dispatch); False: separate RoPE kernel

    # ---- pieces, in the order the ping-pong scheduler interleaves them ----
    def pre_ca(self, x, pos, rope_table, core_attn):
        fused = getattr(self.tp, "fused", None)
        # RoPE and the core-attention dispatch run in the QKV GEMM's epilogue when the attention module
        # supports it (GPU, head_dim 128): the projection is never stored un-rotated
        rope = None
        if x.is_cuda and self.fuse_rope and self.cfg.head_dim == 128 and not self.cfg.qkv_bias:
            ep = core_attn.qkv_epilogue()
            if ep is not None:
                rope = dict(ep, pos=pos, table=rope_table, heads_q=self.hq, heads_kv=self.hkv)
        if fused is not None and x.shape[0] % 128 == 0 and fused.tile_loads:
            # all-gather fused into the QKV GEMM's operand load: the normalised shard is written into the peer
            # arena and every CTA reads the tile it needs from its owner over NVLink (each remote tile crosses
            # the link once per N tile that uses it: only worth it for narrow outputs)
            with timers.phase("norm"):
                buf = fused.stage_buffer(x.shape[0], x.shape[1])
                _, rstd1 = ew.rmsnorm_fwd(x, self.w["ln1"], self.cfg.norm_eps, out=buf)
            with timers.phase("gemm_qkv"):
                qkv = fused.ag_linear(buf, self.w["wqkv"], rope=rope)
            n1f = buf.clone()   # local shard only; gathered again for the weight gradient
        elif fused is not None and x.shape[0] % 128 == 0:
            # every rank stores its normalised shard into every peer's gather buffer (each shard crosses NVLink
            # once), then the GEMM (with RoPE + dispatch in its epilogue) reads the gathered rows locally
            with timers.phase("norm"):
                n1f, rstd1 = ew.rmsnorm_fwd(x, self.w["ln1"], self.cfg.norm_eps)
            with timers.phase("gemm_qkv"):
                g = fused.all_gather_rows(n1f)
                if rope is not None:
                    qkv = gemm.linear_qkv_rope(g, self.w["wqkv"], **rope)
                else:
                    qkv = gemm.linear_fwd(g, self.w["wqkv"])
                fused.release_gather()
                del g
        else:
            with timers.phase("norm"):
                n1, rstd1 = ew.rmsnorm_fwd(x, self.w["ln1"], self.cfg.norm_eps)
            n1f = self.tp.all_gather_rows(n1)
            with timers.phase("gemm_qkv"):
                if rope is not None:
                    qkv = gemm.linear_qkv_rope(n1f, self.w["wqkv"], **rope)
                else:
                    qkv = gemm.linear_fwd(n1f, self.w["wqkv"])
        if rope is not None:
            core_attn.qkv_dispatched()
        else:
            if self.cfg.qkv_bias:
                qkv += self.w["bqkv"]      # Qwen2: the bias is added before the rotation
            with timers.phase("rope"):
                core_attn.apply_rope(qkv, pos, rope_table)
        return qkv, n1f, rstd1

    def post_ca(self, x, attn_out, keep: bool, need_output: bool = True):
        """``need_output=False`` (the recompute pass of backward): the layer's output is not needed again (it is
        the next layer's saved input), so the FC2 GEMM is skipped."""
        fused = getattr(self.tp, "fused", None)
        if fused is not None and x.shape[0] % 128 != 0:
            fused = None
        with timers.phase("gemm_fwd"):
            if self.tp.size == 1:
                h = gemm.linear_fwd(attn_out, self.w["wo"], residual=x)
            elif fused is not None:
                h = fused.linear_rs(attn_out, self.w["wo"], residual=x)   # reduce-scatter fused into the GEMM
            else:
                h = self.tp.reduce_scatter_rows(gemm.linear_fwd(attn_out, self.w["wo"]))
                ew.add_(h, x)
        if fused is not None and fused.tile_loads:
            # FC1: the normalised shard goes into the peer arena, the GEMM reads every rank's shard tile by tile
            # (all-gather fused into the operand load) and applies SwiGLU in its epilogue
            with timers.phase("norm"):
                buf = fused.stage_buffer(h.shape[0], h.shape[1])
                _, rstd2 = ew.rmsnorm_fwd(h, self.w["ln2"], self.cfg.norm_eps, out=buf)
            with timers.phase("gemm_fwd"):
                act, pre = fused.ag_linear_swiglu(buf, self.w["w13"], keep_preact=keep)
            n2f = buf.clone() if keep else None    # local shard only; gathered again for the weight gradient
        elif fused is not None:
            # FC1: shards gathered once by peer stores, SwiGLU in the epilogue of the local GEMM
            with timers.phase("norm"):
                n2f, rstd2 = ew.rmsnorm_fwd(h, self.w["ln2"], self.cfg.norm_eps)
            with timers.phase("gemm_fwd"):
                g = fused.all_gather_rows(n2f)
                act, pre = gemm.linear_swiglu_fwd(g, self.w["w13"], keep_preact=keep)
                fused.release_gather()
                del g
        else:
            with timers.phase("norm"):
                n2, rstd2 = ew.rmsnorm_fwd(h, self.w["ln2"], self.cfg.norm_eps)
            n2f = self.tp.all_gather_rows(n2)
            with timers.phase("gemm_fwd"):
                act, pre = gemm.linear_swiglu_fwd(n2f, self.w["w13"], keep_preact=keep)
        with timers.phase("gemm_fwd"):
            if not need_output:
                y = None
            elif self.tp.size == 1:
                y = gemm.linear_fwd(act, self.w["w2"], residual=h)
            elif fused is not None:
                y = fused.linear_rs(act, self.w["w2"], residual=h)
            else:
                y = self.tp.reduce_scatter_rows(gemm.linear_fwd(act, self.w["w2"]))
                ew.add_(y, h)
        return y, h, rstd2, n2f, pre, act

    def forward(self, x, pos, rope_table, core_attn, keep: bool, attn_store=None, saved_attn=None,
                need_output: bool = True):
        """``attn_store`` (first forward under ``keep_attn``): the core-attention output is saved there and
        the attention module keeps the softmax statistics. ``saved_attn`` (recompute under ``keep_attn``):
        that saved output; core attention is not run again. ``need_output=False``: recompute pass, only the
        context for backward is wanted."""
        qkv, n1f, rstd1 = self.pre_ca(x, pos, rope_table, core_attn)
        with timers.phase("attn_fwd"):
            if saved_attn is not None:
                attn_out, ca_ctx = core_attn.restore(qkv, saved_attn, self.index)
            else:
                attn_out, ca_ctx = core_attn.forward(qkv, self.index)
                if attn_store is not None and not keep:
                    attn_store.save(self.index, core_attn.pack_saved(attn_out, ca_ctx), clone=False)
        y, h, rstd2, n2f, pre, act = self.post_ca(x, attn_out, keep, need_output)
        if not keep:
            return y, None
        return y, LayerCtx(x, rstd1, n1f, ca_ctx, attn_out, h, rstd2, n2f, pre, act)

    def forward_nano(self, xs, poss, rope_table, cas, keep: bool, stores=None, saved=None, need_output: bool = True,
                     streams=None, pre=None, next_layer=None):
        """Forward of this layer for several nano-batches, ping-pong order: every nano-batch runs
        pre-CA (which dispatches its Q/K/V), then every attention server call is issued, and only then
        does each nano-batch collect its attention output and run post-CA, so one nano-batch's
        communication and attention overlap the other's linear layers. ``xs[k]`` is ``None`` when this
        rank owns no tokens of nano-batch ``k`` (it still serves attention for it).
        ``streams``: one CUDA stream per nano-batch; every kernel of nano-batch ``k`` (its signal waits
        included) is queued on ``streams[k]``, so while one nano-batch waits for its servers the GPU runs the
        other's kernels (the reference's compute / communication stream pair with ``TickSync``,
        distca/runtime/megatron/ping_pong/transformer_block.py:122-129, 234-344, ops/stream_sync_fn.py:80-136).
        ``next_layer`` (tick fusion): as soon as nano-batch ``k`` has its output, the NEXT layer's pre-CA runs for
        it (its Q/K/V leave for the servers before the other nano-batch's post-CA of this layer starts), and the
        results come back as a second return value to be passed to that layer as ``pre``; the reference fuses
        post-CA of layer l-1 with pre-CA of layer l into one tick the same way
        (distca/runtime/megatron/ping_pong/tick_ops.py:338-354).
        Reference: distca/runtime/megatron/ping_pong/transformer_layer.py:260-417."""
        n = len(xs)
        if pre is None:
            pre = [None] * n
            for k in range(n):
                with _on(streams, k):
                    if xs[k] is None:
                        cas[k].no_tokens_dispatch()
                    else:
                        pre[k] = self.pre_ca(xs[k], poss[k], rope_table, cas[k])
        pre_next = [None] * n if next_layer is not None else None
        saving = stores is not None and not keep     # keep_attn: O and its statistics are stored per layer
        if saved is None:
            for k in range(n):
                with _on(streams, k), timers.phase("attn_fwd"):
                    cas[k].forward_begin(pre[k][0] if pre[k] is not None else None, self.index)
        outs = []
        for k in range(n):
            with _on(streams, k):
                if saved is None:
                    with timers.phase("attn_fwd"):
                        attn_out, ca_ctx = cas[k].forward_end()
                if xs[k] is None:
                    if saved is not None:
                        cas[k].restore_no_tokens(self.index)
                    if next_layer is not None:
                        cas[k].no_tokens_dispatch()          # the next layer's (empty) dispatch of this nano-batch
                    outs.append((None, None))
                    continue
                qkv, n1f, rstd1 = pre[k]
                if saved is not None:
                    attn_out, ca_ctx = cas[k].restore(qkv, saved[k], self.index)
                elif saving:
                    stores[k].save(self.index, cas[k].pack_saved(attn_out, ca_ctx), clone=False)
                y, h, rstd2, n2f, prea, act = self.post_ca(xs[k], attn_out, keep, need_output)
                outs.append((y, LayerCtx(xs[k], rstd1, n1f, ca_ctx, attn_out, h, rstd2, n2f, prea, act) if keep else None))
                if next_layer is not None:
                    pre_next[k] = next_layer.pre_ca(y, poss[k], rope_table, cas[k])
        if next_layer is not None:
            return outs, pre_next
        return outs

    def backward_nano(self, cs, dys, poss, rope_table, cas, streams=None):
        """Backward twin of :meth:`forward_nano`: post-CA backward + dO dispatch for every nano-batch,
        then the attention-server backward calls, then collect and pre-CA backward. With ``streams`` the
        nano-batches run on their own streams; both accumulate into the same weight-gradient buffers, so the
        second nano-batch's half of a layer starts after the first one's half has finished (an event), which is
        the order the kernels would take on one stream anyway."""
        n = len(cs)
        dhs = [None] * n
        done = None
        for k in range(n):
            with _on(streams, k):
                if cs[k] is None:
                    cas[k].backward_dispatch(None, None, self.index)
                    continue
                if streams is not None and done is not None:
                    streams[k].wait_event(done)
                dattn, dhs[k] = self.bwd_post_ca(cs[k], dys[k])
                if streams is not None:
                    done = torch.cuda.Event()
                    done.record(streams[k])
                cas[k].backward_dispatch(cs[k].ca_ctx, dattn, self.index)
                del dattn
        for k in range(n):
            with _on(streams, k), timers.phase("attn_bwd"):
                cas[k].backward_serve(self.index)
        dxs = []
        done = None
        for k in range(n):
            with _on(streams, k):
                with timers.phase("attn_bwd"):
                    dqkv = cas[k].backward_end()
                if cs[k] is None:
                    dxs.append(None)
                    continue
                cs[k].ca_ctx = None
                if streams is not None and done is not None:
                    streams[k].wait_event(done)
                dxs.append(self.bwd_pre_ca(cs[k], dqkv, dhs[k], poss[k], rope_table))
                if streams is not None:
                    done = torch.cuda.Event()
                    done.record(streams[k])
        return dxs

    # ---- backward pieces ----
    def bwd_post_ca(self, c: LayerCtx, dy):
        """dy -> (dattn, dh). Accumulates dW2, dW13, dln2, dWo."""
        fused = getattr(self.tp, "fused", None)
        if fused is not None and dy.shape[0] % 128 == 0:
            return self._bwd_post_ca_fused(c, dy, fused)
        dyf = self.tp.all_gather_rows(dy)
        with timers.phase("gemm_bwd"):
            dact = gemm.linear_dgrad(dyf, self.w["w2"])
            gemm.linear_wgrad(dyf, c.act, out=self.g["w2"], accumulate=True)
        c.act = None
        with timers.phase("swiglu_bwd"):
            dpre = ew.swiglu_bwd(c.pre, dact, inplace=True)
        del dact
        n2f = c.n2 if c.n2.shape[0] == dpre.shape[0] else self.tp.all_gather_rows(c.n2)
        with timers.phase("gemm_bwd"):
            dn2 = self.tp.reduce_scatter_rows(gemm.linear_dgrad(dpre, self.w["w13"]))
            gemm.linear_wgrad(dpre, n2f, out=self.g["w13"], accumulate=True)
        del n2f
        c.pre = c.n2 = None
        del dpre
        with timers.phase("norm_bwd"):
            dh = ew.rmsnorm_bwd(c.h, self.w["ln2"], c.rstd2, dn2, self.g["ln2"], dres=dy)
        del dn2
        dhf = self.tp.all_gather_rows(dh)
        with timers.phase("gemm_bwd"):
            dattn = gemm.linear_dgrad(dhf, self.w["wo"])
            gemm.linear_wgrad(dhf, c.attn_out, out=self.g["wo"], accumulate=True)
        c.attn_out = c.h = None
        return dattn, dh

    def _bwd_post_ca_fused(self, c: LayerCtx, dy, fused):
        """Tensor + sequence parallel backward of the post-attention half without NCCL: sharded operands are
        gathered by peer stores (``all_gather_rows``: every shard crosses NVLink once and serves both the
        data-gradient and the weight-gradient GEMM), and the GEMMs whose output is reduce-scattered store their
        rows to the owners from their epilogues (GEMM -> reduce-scatter)."""
        rows, H = dy.shape
        with timers.phase("gemm_bwd"):
            # one gather of dy (peer stores) serves the data-gradient and the weight-gradient GEMM
            dyf = fused.all_gather_rows(dy)
            dact = gemm.linear_dgrad(dyf, self.w["w2"])                                  # all_gather(dy) @ W2
            gemm.linear_wgrad(dyf, c.act, out=self.g["w2"], accumulate=True)
            fused.release_gather()
            del dyf
        c.act = None
        with timers.phase("swiglu_bwd"):
            dpre = ew.swiglu_bwd(c.pre, dact, inplace=True)
        del dact
        with timers.phase("gemm_bwd"):
            dn2 = fused.linear_rs(dpre, self.w["w13"], transposed_weight=True)          # reduce_scatter(dpre @ W13)
            n2f = c.n2 if c.n2.shape[0] == dpre.shape[0] else fused.all_gather_rows(c.n2)
            gemm.linear_wgrad(dpre, n2f, out=self.g["w13"], accumulate=True)
            if c.n2.shape[0] != dpre.shape[0]:
                fused.release_gather()
        del n2f
        c.pre = c.n2 = None
        del dpre
        with timers.phase("norm_bwd"):
            dh = ew.rmsnorm_bwd(c.h, self.w["ln2"], c.rstd2, dn2, self.g["ln2"], dres=dy)
        del dn2
        with timers.phase("gemm_bwd"):
            dhf = fused.all_gather_rows(dh)
            dattn = gemm.linear_dgrad(dhf, self.w["wo"])                                 # all_gather(dh) @ Wo
            gemm.linear_wgrad(dhf, c.attn_out, out=self.g["wo"], accumulate=True)
            fused.release_gather()
            del dhf
        c.attn_out = c.h = None
        return dattn, dh

    def bwd_pre_ca(self, c: LayerCtx, dqkv, dh, pos, rope_table):
        """(dqkv, dh) -> dx. Accumulates dWqkv, dln1."""
        with timers.phase("rope"):
            ew.rope_(dqkv, pos, rope_table, self.hq, self.hkv, self.cfg.head_dim, backward=True)
        if self.cfg.qkv_bias:
            self.g["bqkv"] += dqkv.float().sum(0).to(self.g["bqkv"].dtype)
        fused = getattr(self.tp, "fused", None)
        if fused is not None and dqkv.is_contiguous() and dh.shape[0] % 128 == 0:
            with timers.phase("gemm_bwd"):
                dn1 = fused.linear_rs(dqkv, self.w["wqkv"], transposed_weight=True)     # reduce_scatter(dqkv @ Wqkv)
                gathered = c.n1.shape[0] != dqkv.shape[0]
                n1f = fused.all_gather_rows(c.n1) if gathered else c.n1
                gemm.linear_wgrad(dqkv, n1f, out=self.g["wqkv"], accumulate=True)
                if gathered:
                    fused.release_gather()
        else:
            n1f = c.n1 if c.n1.shape[0] == dqkv.shape[0] else self.tp.all_gather_rows(c.n1)
            with timers.phase("gemm_bwd"):
                dn1 = self.tp.reduce_scatter_rows(gemm.linear_dgrad(dqkv, self.w["wqkv"]))
                gemm.linear_wgrad(dqkv, n1f, out=self.g["wqkv"], accumulate=True)
        del n1f
        c.n1 = None
        with timers.phase("norm_bwd"):
            dx = ew.rmsnorm_bwd(c.x, self.w["ln1"], c.rstd1, dn1, self.g["ln1"], dres=dh)
        return dx

    def backward(self, c: LayerCtx, dy, pos, rope_table, core_attn):
        dattn, dh = self.bwd_post_ca(c, dy)
        with timers.phase("attn_bwd"):
            dqkv = core_attn.backward(c.ca_ctx, dattn, self.index)
        c.ca_ctx = None
        del dattn
        return self.bwd_pre_ca(c, dqkv, dh, pos, rope_table)


class _ListStore:
    """Per-micro-batch stand-in for :class:`~distca_b200.utils.offload.LayerStore` in pipeline stages:
    everything stays in HBM, one entry per layer, dropped when read."""

    def __init__(self):
        self.d: dict = {}

    def has(self, i: int) -> bool:
        return True

    def save(self, i: int, t, clone: bool = True) -> None:
        self.d[i] = t.clone() if clone else t

    def load(self, i: int):
        return self.d.pop(i)

    def prefetch(self, i: int) -> None:
        pass


# ---------------------------------------------------------------------------------------------
# full model (one pipeline stage)
# ---------------------------------------------------------------------------------------------
@dataclass
class Batch:
    """One micro-batch as the model sees it (all on the model's device).

    ids/labels: int64 [T]; labels < 0 are ignored. pos: int32 [T] position inside the document.
    """
    ids: torch.Tensor
    labels: torch.Tensor
    pos: torch.Tensor
    num_valid_global: int  # denominator of the mean loss over the whole global batch


class LlamaModel:
    def __init__(self, cfg: ModelConfig, device, *, tp=None, layer_range=None, first_stage=True,
                 last_stage=True, dtype=None, grad_dtype=None, seed: int = 0, recompute: str = "full",
                 lm_head_chunk: int = 8192, pad_params_to: int = 1, param_buffers=None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.tp = tp or NoTP()
        self.first_stage, self.last_stage = first_stage, last_stage
        self.layer_range = layer_range or (0, cfg.num_layers)
        on_gpu = self.device.type == "cuda"
        self.dtype = dtype or (torch.bfloat16 if on_gpu else torch.float32)
        self.grad_dtype = grad_dtype or self.dtype
        self.recompute = recompute
        self.lm_head_chunk = lm_head_chunk
        shapes = param_shapes(cfg, self.tp.size, self.layer_range, first_stage, last_stage)
        self.store = ParamStore(shapes, self.device, self.dtype, self.grad_dtype, pad_to=pad_params_to,
                                buffers=param_buffers)
        self.store.init_weights(cfg.init_std, seed * 97 + self.tp.rank)
        self.layers = [LlamaLayer(cfg, self.store, l, self.tp) for l in range(*self.layer_range)]
        self.rope_table = ew.rope_table(cfg.max_position, cfg.head_dim, cfg.rope_theta, self.device)
        self.vocab_local = cfg.vocab // self.tp.size
        self.vocab_start = self.tp.rank * self.vocab_local
        self._lm_acc = None
        self._store = None
        self._stores = None
        self._pinned = []
        self.grad_ready_hook = None        # called with a layer's parameter names once its gradients are final
        self.nano_streams = True           # ping-pong: every nano-batch on its own CUDA stream
        self._nano_stream_objs = None
        self.store_sync_group = None       # gloo-capable group over which the keep_attn placement is agreed
        self.attn_store_placement = None   # "device" | "host" to override the automatic choice
        self.check_finite = False          # debug: test every layer's output / input gradient (one sync per layer pass)
        self.fuse_ticks = False            # ping-pong: pre-CA of layer l+1 right after post-CA of layer l per nano-batch

    def _attn_store(self, tokens: int, host_copies: int = 1):
        """Store of the per-layer core-attention outputs for ``recompute="keep_attn"`` (created at the
        first step): HBM first, then pinned host memory; layers that fit in neither are fully recomputed."""
        if self._store is None and self.recompute == "keep_attn":
            from ..utils.offload import LayerStore, choose_placements
            cfg, tp = self.cfg, self.tp.size
            nl = len(self.layers)
            rows = tokens * tp    # attention runs on the gathered rows with this rank's heads
            per_layer = rows * (cfg.heads_q // tp) * cfg.head_dim * 2
            qkvd = (cfg.heads_q + 2 * cfg.heads_kv) * cfg.head_dim // tp
            reserve = (nl * tokens * cfg.hidden * 2 + rows * 2 * (5 * cfg.hidden + 2 * qkvd + 6 * cfg.ffn // tp)
                       + (20 << 30 if cfg.vocab > 65536 else 2 << 30))
            if self.attn_store_placement is not None:
                where = [self.attn_store_placement] * (nl - 1)
            else:
                where = choose_placements(nl - 1, per_layer, self.device, reserve, host_copies)
            self._store_capacity = rows * ((cfg.heads_q // tp) * cfg.head_dim + 2 * (cfg.heads_q // tp))
            # page-lock the host part now: if the host refuses, those layers are recomputed instead, and the
            # agreement below sees it
            self._pinned = []
            n_host = sum(w == "host" for w in where)
            if n_host and self.device.type == "cuda":
                try:
                    self._pinned = [torch.empty(n_host, self._store_capacity, dtype=self.dtype, pin_memory=True)
                                    for _ in range(host_copies)]
                except RuntimeError:
                    self._pinned = []
                    where = [w if w != "host" else None for w in where]
            if self.store_sync_group is not None:
                # every rank of the job must agree on WHICH layers skip the attention recompute (a server
                # that recomputes waits for peers that would not take part): keep the common prefix
                import torch.distributed as dist
                k = torch.tensor([sum(w is not None for w in where)], dtype=torch.int64)
                dist.all_reduce(k, op=dist.ReduceOp.MIN, group=self.store_sync_group)
                where = [w if i < int(k.item()) else None for i, w in enumerate(where)]
            full = [None] * cfg.num_layers     # indexed by global layer number; the last local layer is never recomputed
            for layer, w in zip(self.layers[:-1], where):
                full[layer.index] = w
            # with several nano-batch stores this one only carries the placement (no pinned buffer)
            self._store = LayerStore(full, self.device, 0, self.dtype,
                                     host=self._pinned[0] if (self._pinned and host_copies == 1) else None)
            self._store.never_asked = cfg.num_layers - (nl - 1)
        return self._store

    def ensure_positions(self, longest_document: int) -> None:
        """Make sure the rotary table covers positions ``0 .. longest_document - 1``. A configuration whose
        ``max_position`` is shorter than the documents it is trained on (a Hugging Face config with
        ``max_position_embeddings`` 8192 and 128K-token documents, or documents elongated beyond the preset)
        gets a longer table here, before any kernel indexes it; the kernels themselves clamp and report
        an out-of-range position instead of reading past the table."""
        if longest_document > self.rope_table.shape[0]:
            rows = 1 << max(0, int(longest_document - 1)).bit_length()
            import logging
            logging.getLogger("distca_b200").warning(
                "documents of %d tokens exceed max_position %d: rotary table extended to %d rows",
                longest_document, self.rope_table.shape[0], rows)
            self.rope_table = ew.rope_table(rows, self.cfg.head_dim, self.cfg.rope_theta, self.device)

    def load_full_state(self, full: dict) -> None:
        """Load un-sharded tensors (this repository's row order), slicing for this tensor-parallel rank."""
        for name, _ in self.store.shapes:
            t = shard_full_tensor(name, full[name], self.cfg, self.tp.size, self.tp.rank)
            self.store.p[name].copy_(t.to(self.store.p[name].dtype))

    # ---- embedding ----
    def embed(self, ids):
        e = ew.embedding_fwd(ids, self.store.p["embedding.word_embeddings.weight"], self.vocab_start)
        if self.tp.size > 1:
            e = self.tp.reduce_scatter_rows(e)
        return e

    def embed_bwd(self, ids, dx):
        dxf = self.tp.all_gather_rows(dx)
        ew.embedding_bwd(ids, dxf, self.store.g["embedding.word_embeddings.weight"], self.vocab_start)

    # ---- final norm + LM head + cross entropy, forward and backward in token chunks ----
    def _lm_weight(self):
        name = "output_layer.weight" if "output_layer.weight" in self.store.p else "embedding.word_embeddings.weight"
        return self.store.p[name], self.store.g[name]

    def head_loss_and_grad(self, x, labels, num_valid_global: int, need_grad: bool = True):
        """x: [T(/tp), H] -> (sum of token losses on this rank / num_valid_global, dx)."""
        cfg = self.cfg
        w, gw = self._lm_weight()
        gln = self.store.g["decoder.final_layernorm.weight"]
        wln = self.store.p["decoder.final_layernorm.weight"]
        T = x.shape[0]
        dx = torch.empty_like(x) if need_grad else None
        scale = 1.0 / max(1, num_valid_global)
        loss_sum = torch.zeros((), dtype=torch.float32, device=x.device)
        chunk = max(128, self.lm_head_chunk // self.tp.size)
        nchunks = (T + chunk - 1) // chunk
        use_acc = need_grad and x.is_cuda and nchunks > 1 and gw.dtype != torch.float32
        if use_acc:
            if self._lm_acc is None:
                self._lm_acc = torch.empty(gw.shape, dtype=torch.float32, device=x.device)
            self._lm_acc.zero_()
        for c0 in range(0, T, chunk):
            c1 = min(T, c0 + chunk)
            xc = x[c0:c1]
            n, rstd = ew.rmsnorm_fwd(xc, wln, cfg.norm_eps)
            nf = self.tp.all_gather_rows(n)
            # the gathered chunk is (rank 0's rows c0:c1 | rank 1's rows c0:c1 | ...): pick the same labels
            if self.tp.size > 1:
                lab = torch.cat([labels[r * T + c0:r * T + c1] for r in range(self.tp.size)])
            else:
                lab = labels[c0:c1]
            if x.is_cuda:
                logits = torch.empty(nf.shape[0], self.vocab_local, dtype=torch.float32, device=x.device)
                gemm.gemm_raw(nf, w, logits, nf.shape[0], self.vocab_local, cfg.hidden, 0, 0)
            else:
                logits = nf @ w.t()
            stats = ew.ce_stats(logits, lab, self.vocab_start)
            stats_all = self.tp.all_gather_stats(stats)
            loss_tok, dlogits = ew.ce_grad(logits, lab, stats_all, scale, self.vocab_start)
            del logits
            loss_sum += loss_tok.sum() * scale
            if not need_grad:
                continue
            if use_acc:
                gemm.linear_wgrad(dlogits, nf, out=self._lm_acc, accumulate=True)
            else:
                gemm.linear_wgrad(dlogits, nf, out=gw, accumulate=True)
            dn = self.tp.reduce_scatter_rows(gemm.linear_dgrad(dlogits, w))
            del dlogits
            ew.rmsnorm_bwd(xc, wln, rstd, dn, gln, dx_out=dx[c0:c1])
        if use_acc:
            gw.add_(self._lm_acc.to(gw.dtype))
        return loss_sum, dx

    # ---- whole-stage passes ----
    def _finite(self, t, what: str, index: int) -> None:
        """Debug aid (``check_finite``): name the first layer pass that produced a NaN / Inf, like the reference's
        NaN hooks (playground/utils/nan_detector.py:165-444)."""
        if self.check_finite and t is not None and not bool(torch.isfinite(t).all()):
            raise FloatingPointError(f"non-finite values in the {what} of layer {index}")

    def forward_backward(self, batch: Batch, core_attn, *, x_in: torch.Tensor | None = None,
                         dy_in: torch.Tensor | None = None):
        """One micro-batch through this stage. Returns (loss or None, dx_to_previous_stage or None)."""
        assert self.first_stage and self.last_stage, "pipeline stages are driven by parallel.pipeline"
        x = self.embed(batch.ids)
        ctxs, inputs = [], []
        nl = len(self.layers)
        store = self._attn_store(x.shape[0]) if self.recompute == "keep_attn" else None
        for i, layer in enumerate(self.layers):
            keep = self.recompute == "none" or i == nl - 1
            inputs.append(x)
            with timers.layer("fwd", layer.index):
                x, ctx = layer.forward(x, batch.pos, self.rope_table, core_attn, keep,
                                       attn_store=store if store is not None and store.has(layer.index) else None)
            self._finite(x, "forward output", layer.index)
            ctxs.append(ctx)
        with timers.phase("lm_head"):
            loss, dx = self.head_loss_and_grad(x, batch.labels, batch.num_valid_global)
        del x
        if store is not None:
            store.prefetch(self.layers[nl - 2].index if nl > 1 else -1)
        for i in reversed(range(nl)):
            layer = self.layers[i]
            ctx = ctxs[i]
            ctxs[i] = None
            if ctx is None:
                saved = None
                if store is not None and store.has(layer.index):
                    saved = store.load(layer.index)
                    store.prefetch(self.layers[i - 1].index if i > 0 else -1)
                with timers.layer("recompute", layer.index):
                    _, ctx = layer.forward(inputs[i], batch.pos, self.rope_table, core_attn, True, saved_attn=saved,
                                           need_output=False)
                del saved
            inputs[i] = None
            with timers.layer("bwd", layer.index):
                dx = layer.backward(ctx, dx, batch.pos, self.rope_table, core_attn)
            self._finite(dx, "input gradient", layer.index)
            del ctx
            if self.grad_ready_hook is not None:
                self.grad_ready_hook(list(layer.names.values()))
        with timers.phase("embed_bwd"):
            self.embed_bwd(batch.ids, dx)
        return loss, None

    def forward_backward_nano(self, batches, cas):
        """One step over several nano-batches interleaved layer by layer (ping-pong). ``batches[k]`` is
        ``None`` when this rank has no tokens of nano-batch ``k``. Gradients of all nano-batches
        accumulate into the same buffers; returns the summed loss. With ``self.nano_streams`` every
        nano-batch runs on its own CUDA stream (see :meth:`LlamaLayer.forward_nano`)."""
        assert self.first_stage and self.last_stage
        n = len(batches)
        streams = None
        if self.nano_streams and self.device.type == "cuda":
            if self._nano_stream_objs is None or len(self._nano_stream_objs) != n:
                self._nano_stream_objs = [torch.cuda.Stream(self.device) for _ in range(n)]
            streams = self._nano_stream_objs
            main = torch.cuda.current_stream(self.device)
            for st_ in streams:
                st_.wait_stream(main)          # zero_grad and the host-to-device copies come first
        xs = []
        for k, b in enumerate(batches):
            with _on(streams, k):
                xs.append(self.embed(b.ids) if b is not None else None)
        poss = [b.pos if b is not None else None for b in batches]
        nl = len(self.layers)
        stores = None
        if self.recompute == "keep_attn":
            stores = self._attn_stores([x.shape[0] if x is not None else 0 for x in xs])
        ctxs, inputs = [], []
        pre = None
        for i, layer in enumerate(self.layers):
            keep = self.recompute == "none" or i == nl - 1
            inputs.append(xs)
            use = stores if stores is not None and stores[0].has(layer.index) else None
            nxt = self.layers[i + 1] if (self.fuse_ticks and i + 1 < nl) else None
            with timers.layer("fwd", layer.index):
                outs = layer.forward_nano(xs, poss, self.rope_table, cas, keep, stores=use, streams=streams,
                                          pre=pre, next_layer=nxt)
            outs, pre = outs if nxt is not None else (outs, None)
            xs = [o[0] for o in outs]
            ctxs.append([o[1] for o in outs] if keep else None)
        losses = []
        dxs = [None] * n
        done = None
        for k in range(n):
            if xs[k] is None:
                continue
            with _on(streams, k), timers.phase("lm_head"):
                if streams is not None and done is not None:
                    streams[k].wait_event(done)          # the LM head's gradient accumulators are shared
                l, dxs[k] = self.head_loss_and_grad(xs[k], batches[k].labels, batches[k].num_valid_global)
                losses.append(l)
                if streams is not None:
                    done = torch.cuda.Event()
                    done.record(streams[k])
        del xs
        for i in reversed(range(nl)):
            layer = self.layers[i]
            cs = ctxs[i]
            ctxs[i] = None
            if cs is None:
                saved = None
                if stores is not None and stores[0].has(layer.index):
                    saved = []
                    for k, st in enumerate(stores):
                        with _on(streams, k):
                            saved.append(st.load(layer.index) if inputs[i][k] is not None else None)
                            if i > 0 and inputs[i][k] is not None:
                                st.prefetch(self.layers[i - 1].index)
                with timers.layer("recompute", layer.index):
                    outs = layer.forward_nano(inputs[i], poss, self.rope_table, cas, True, saved=saved,
                                              need_output=False, streams=streams)
                cs = [o[1] for o in outs]
                del saved, outs
            inputs[i] = None
            with timers.layer("bwd", layer.index):
                dxs = layer.backward_nano(cs, dxs, poss, self.rope_table, cas, streams=streams)
            del cs
            if self.grad_ready_hook is not None:
                if streams is not None:
                    for st_ in streams:
                        torch.cuda.current_stream(self.device).wait_stream(st_)
                self.grad_ready_hook(list(layer.names.values()))
        done = None
        for k in range(n):
            if dxs[k] is None:
                continue
            with _on(streams, k), timers.phase("embed_bwd"):
                if streams is not None and done is not None:
                    streams[k].wait_event(done)
                self.embed_bwd(batches[k].ids, dxs[k])
                if streams is not None:
                    done = torch.cuda.Event()
                    done.record(streams[k])
        if streams is not None:
            for st_ in streams:
                torch.cuda.current_stream(self.device).wait_stream(st_)
        loss = torch.zeros((), dtype=torch.float32, device=self.device)
        for l in losses:
            loss = loss + l
        return loss, None

    def _attn_stores(self, tokens_per_nano: list):
        """One attention-output store per nano-batch with a common placement (the memory question is
        asked once, for the sum of the nano-batches)."""
        if self._stores is None:
            from ..utils.offload import LayerStore
            base = self._attn_store(max(1, sum(tokens_per_nano)), host_copies=len(tokens_per_nano))
            # either nano-batch may hold up to the whole sequence: same capacity for both
            self._stores = [LayerStore(list(base.where), self.device, self._store_capacity, self.dtype,
                                       host=self._pinned[k] if k < len(self._pinned) else None)
                            for k in range(len(tokens_per_nano))]
            for st in self._stores:
                st.never_asked = base.never_asked
        return self._stores

    # ---- pipeline-stage passes (forward and backward of one micro-batch at different times) ----
    def stage_forward(self, batch: Batch, core_attn, x_in: torch.Tensor | None, keep_last: bool = False):
        """Forward of this stage's layers. Returns ``(x_out, saved)``; ``saved`` is what
        :meth:`stage_backward` needs (layer inputs under full recompute, full contexts otherwise).
        ``keep_last`` keeps the last layer's context (only valid when its backward follows with no
        other core-attention call in between)."""
        x = self.embed(batch.ids) if self.first_stage else x_in
        inputs, ctxs = [], []
        nl = len(self.layers)
        # keep_attn: this micro-batch's attention outputs (+ statistics) wait in HBM for its backward slot,
        # which may run under a different core-attention plan (the servers keep nothing in between)
        store = _ListStore() if self.recompute == "keep_attn" else None
        for i, layer in enumerate(self.layers):
            keep = self.recompute == "none" or (keep_last and i == nl - 1)
            inputs.append(x)
            with timers.layer("fwd", layer.index):
                x, ctx = layer.forward(x, batch.pos, self.rope_table, core_attn, keep, attn_store=store)
            ctxs.append(ctx)
        return x, (inputs, ctxs, x if self.last_stage else None, store)

    def stage_backward(self, batch: Batch, core_attn, saved, dy: torch.Tensor | None, grads_final: bool = False):
        """Backward of this stage for one micro-batch. On the last stage ``dy`` is ignored and the
        loss head produces the gradient. ``grads_final``: this is the step's last micro-batch, so a layer's
        gradients are complete once its backward has run (the gradient-ready hook fires per layer).
        Returns ``(loss or None, dx for the previous stage or None)``."""
        inputs, ctxs, x_out, store = saved
        loss = None
        if self.last_stage:
            with timers.phase("lm_head"):
                loss, dx = self.head_loss_and_grad(x_out, batch.labels, batch.num_valid_global)
        else:
            dx = dy
        del x_out
        for i in reversed(range(len(self.layers))):
            layer = self.layers[i]
            ctx = ctxs[i]
            ctxs[i] = None
            if ctx is None:
                with timers.layer("recompute", layer.index):
                    _, ctx = layer.forward(inputs[i], batch.pos, self.rope_table, core_attn, True,
                                           saved_attn=store.load(layer.index) if store is not None else None,
                                           need_output=False)
            inputs[i] = None
            with timers.layer("bwd", layer.index):
                dx = layer.backward(ctx, dx, batch.pos, self.rope_table, core_attn)
            del ctx
            if grads_final and self.grad_ready_hook is not None:
                self.grad_ready_hook(list(layer.names.values()))
        if self.first_stage:
            with timers.phase("embed_bwd"):
                self.embed_bwd(batch.ids, dx)
            dx = None
        return loss, dx

    def stage_forward_nano(self, batches, cas, x_ins):
        """:meth:`stage_forward` for the nano-batches of one micro-batch, interleaved layer by layer (ping-pong
        inside a pipeline stage; the reference runs its ping-pong layers under the pipeline schedule the same
        way, distca/runtime/megatron/ping_pong/transformer_block.py:234-344 under
        forward_backward_func.py:117-519). ``batches[k]`` / ``x_ins[k]`` are ``None`` for a nano-batch this rank
        owns no tokens of (it still serves attention for it). Returns ``(x_outs, saved)``."""
        n = len(batches)
        xs = [None] * n
        for k, b in enumerate(batches):
            if b is not None:
                xs[k] = self.embed(b.ids) if self.first_stage else x_ins[k]
        poss = [b.pos if b is not None else None for b in batches]
        stores = [_ListStore() for _ in range(n)] if self.recompute == "keep_attn" else None
        inputs, ctxs = [], []
        pre, nl = None, len(self.layers)
        for i, layer in enumerate(self.layers):
            keep = self.recompute == "none"
            inputs.append(xs)
            nxt = self.layers[i + 1] if (self.fuse_ticks and i + 1 < nl) else None
            with timers.layer("fwd", layer.index):
                outs = layer.forward_nano(xs, poss, self.rope_table, cas, keep, stores=stores, pre=pre, next_layer=nxt)
            outs, pre = outs if nxt is not None else (outs, None)
            xs = [o[0] for o in outs]
            ctxs.append([o[1] for o in outs] if keep else None)
        return xs, (inputs, ctxs, xs if self.last_stage else None, stores)

    def stage_backward_nano(self, batches, cas, saved, dys, grads_final: bool = False):
        """:meth:`stage_backward` for the nano-batches of one micro-batch (see :meth:`stage_forward_nano`).
        Returns ``(summed loss or None, [dx per nano-batch] or None on the first stage)``."""
        inputs, ctxs, x_outs, stores = saved
        n = len(batches)
        poss = [b.pos if b is not None else None for b in batches]
        loss = None
        if self.last_stage:
            dxs = [None] * n
            for k, b in enumerate(batches):
                if b is None:
                    continue
                with timers.phase("lm_head"):
                    l, dxs[k] = self.head_loss_and_grad(x_outs[k], b.labels, b.num_valid_global)
                loss = l if loss is None else loss + l
        else:
            dxs = list(dys)
        del x_outs
        for i in reversed(range(len(self.layers))):
            layer = self.layers[i]
            cs = ctxs[i]
            ctxs[i] = None
            if cs is None:
                kept = None
                if stores is not None:
                    kept = [stores[k].load(layer.index) if inputs[i][k] is not None else None for k in range(n)]
                with timers.layer("recompute", layer.index):
                    outs = layer.forward_nano(inputs[i], poss, self.rope_table, cas, True, saved=kept, need_output=False)
                cs = [o[1] for o in outs]
                del kept, outs
            inputs[i] = None
            with timers.layer("bwd", layer.index):
                dxs = layer.backward_nano(cs, dxs, poss, self.rope_table, cas)
            del cs
            if grads_final and self.grad_ready_hook is not None:
                self.grad_ready_hook(list(layer.names.values()))
        if self.first_stage:
            for k, b in enumerate(batches):
                if b is not None:
                    with timers.phase("embed_bwd"):
                        self.embed_bwd(b.ids, dxs[k])
            dxs = None
        return loss, dxs

    def forward_loss(self, batch: Batch, core_attn) -> torch.Tensor:
        """Evaluation pass (no gradients)."""
        x = self.embed(batch.ids)
        for layer in self.layers:
            x, _ = layer.forward(x, batch.pos, self.rope_table, core_attn, False)
        loss, _ = self.head_loss_and_grad(x, batch.labels, batch.num_valid_global, need_grad=False)
        return loss
