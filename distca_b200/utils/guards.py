"""Host-side training guards: non-finite or spiking loss, exploding gradient norm, and a pre-flight
memory estimate. None of them touches the GPU beyond values the step already returns.

The reference gets the same checks from Megatron flags in its playground trainer
(``--check-for-nan-in-loss-and-grad``, ``--check-for-spiky-loss``, ``--check-for-large-grads``,
playground/simple_4d.py:465-466, and ``--distca-quit-if-maybe-oom``, :603-605).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

from ..models.config import ModelConfig, ParallelConfig


class TrainingFault(RuntimeError):
    pass


@dataclass
class TrainingGuards:
    check_nan: bool = True
    spiky_loss_factor: float = 0.0     # 0 = off; fault when loss > factor x running maximum of good steps
    large_grad_factor: float = 0.0     # 0 = off; fault when grad norm > factor x running maximum
    warmup_steps: int = 2              # steps that only feed the running statistics
    _max_loss: float = field(default=0.0, init=False)
    _max_grad: float = field(default=0.0, init=False)
    _seen: int = field(default=0, init=False)

    def check(self, step: int, loss: float, grad_norm: float | None = None) -> None:
        """Raises :class:`TrainingFault` with a one-line reason; otherwise updates the statistics."""
        if self.check_nan and not math.isfinite(loss):
            raise TrainingFault(f"step {step}: loss is {loss}")
        if self.check_nan and grad_norm is not None and not math.isfinite(grad_norm):
            raise TrainingFault(f"step {step}: gradient norm is {grad_norm}")
        if self._seen >= self.warmup_steps:
            if self.spiky_loss_factor and self._max_loss and loss > self.spiky_loss_factor * self._max_loss:
                raise TrainingFault(f"step {step}: loss {loss:.4f} is more than {self.spiky_loss_factor} x the "
                                    f"largest loss seen so far ({self._max_loss:.4f})")
            if (self.large_grad_factor and grad_norm is not None and self._max_grad
                    and grad_norm > self.large_grad_factor * self._max_grad):
                raise TrainingFault(f"step {step}: gradient norm {grad_norm:.3e} is more than "
                                    f"{self.large_grad_factor} x the largest seen so far ({self._max_grad:.3e})")
        self._max_loss = max(self._max_loss, loss)
        if grad_norm is not None:
            self._max_grad = max(self._max_grad, grad_norm)
        self._seen += 1


def estimate_memory_gb(cfg: ModelConfig, par: ParallelConfig, tokens_per_rank: int, *, recompute: str = "full",
                       cad: bool = True, comm_buffer_gb: float = 2.0, microbatches_in_flight: int = 1,
                       nano_batches: int = 1) -> dict:
    """Rough per-GPU high-water mark (GB) of one training step: parameters, gradients, optimizer
    shards, stored layer inputs, one layer's transient activations, the LM-head chunk and the
    core-attention arena. Within a few percent of the measured 177 GB of Llama-3-8B at 128K on one GPU: meant to refuse a configuration before it runs out of memory."""
    GB = 1e9
    layers = cfg.num_layers // par.pp
    params = cfg.num_params() / (par.tp * par.pp)
    weights = params * 2
    grads = params * (4 if microbatches_in_flight > 1 else 2)
    optim = params * 10 / par.dp                     # m, v fp32 + 16-bit master remainder, ZeRO-1
    T = tokens_per_rank
    rows_sp = T // par.tp                            # sequence-parallel rows between the linear blocks
    qkvd = cfg.qkv_dim // par.tp
    inputs = layers * rows_sp * cfg.hidden * 2 * microbatches_in_flight
    transient = 2 * (T * (4 * cfg.hidden + 2 * qkvd + 4 * cfg.ffn // par.tp))   # calibrated on the 128K run
    if recompute == "none":
        inputs = layers * transient / 2 * microbatches_in_flight
    head = 2 * 8192 * (cfg.vocab // par.tp) * 4 + (cfg.vocab // par.tp) * cfg.hidden * 4
    arena = 0.0
    if cad and par.dp * par.pp > 1:
        W = par.dp * par.pp
        q_b, kv_b = cfg.q_dim // par.tp * 2, cfg.kv_dim // par.tp * 2
        arena = (2 * T * q_b * 2 + max(comm_buffer_gb * 2**30 - 2 * T * q_b, 4 * T * kv_b) + T * q_b + T * qkvd * 2
                 + W * T * 2 * kv_b + 2 * T * (cfg.heads_q // par.tp) * 8) * nano_batches
    # peer arena of the tensor-parallel transports: one staging shard, tp reduce-scatter slots, tp gather slots
    tp_arena = rows_sp * cfg.hidden * 2 * (1 + 2 * par.tp) if par.tp > 1 else 0.0
    total = weights + grads + optim + inputs + transient + head + arena + tp_arena
    # keep_attn: the kept attention outputs go to whatever HBM is left and then to host memory, so they never make a
    # configuration fail; reported for information
    kept = layers * microbatches_in_flight * T * (cfg.q_dim // par.tp + 2 * cfg.heads_q // par.tp) * 2 if recompute == "keep_attn" else 0.0
    return {"weights": weights / GB, "gradients": grads / GB, "optimizer": optim / GB, "layer_inputs": inputs / GB,
            "transient": transient / GB, "lm_head": head / GB, "attention_arena": arena / GB,
            "tensor_parallel_arena": tp_arena / GB, "total": total / GB, "kept_attention_if_room": kept / GB}


def quit_if_maybe_oom(est: dict, capacity_gb: float, margin: float = 0.97) -> None:
    if est["total"] > capacity_gb * margin:
        parts = ", ".join(f"{k} {v:.1f}" for k, v in est.items() if k not in ("total", "kept_attention_if_room"))
        raise TrainingFault(f"estimated {est['total']:.1f} GB per GPU exceeds {capacity_gb:.0f} GB ({parts})")


def main() -> None:
    """``python -m distca_b200.utils.guards --model llama3-8b --tp 2 --pp 2 --dp 2 --tokens 131072``:
    per-GPU memory plan of a configuration (the reference's playground/estimate_memory.py what-if)."""
    import argparse
    import json

    from ..models.config import get_model_config
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--tokens", type=int, default=131072, help="tokens per rank and micro-batch")
    ap.add_argument("--recompute", default="full", choices=["none", "full", "keep_attn"])
    ap.add_argument("--no-cad", action="store_true")
    ap.add_argument("--comm-buffer-gb", type=float, default=2.0)
    ap.add_argument("--capacity-gb", type=float, default=180.0)
    a = ap.parse_args()
    par = ParallelConfig(a.tp, a.pp, a.dp)
    est = estimate_memory_gb(get_model_config(a.model), par, a.tokens, recompute=a.recompute, cad=not a.no_cad,
                             comm_buffer_gb=a.comm_buffer_gb, microbatches_in_flight=a.pp)
    est["fits"] = est["total"] <= a.capacity_gb * 0.97
    print(json.dumps({k: (round(v, 2) if isinstance(v, float) else v) for k, v in est.items()}))


if __name__ == "__main__":
    main()
