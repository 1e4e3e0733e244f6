"""Checkpoint save / load in the Megatron-LM directory and key layout.

    <dir>/latest_checkpointed_iteration.txt
    <dir>/iter_0000100/mp_rank_00/model_optim_rng.pt          (tp rank 0, no pipeline parallelism)
    <dir>/iter_0000100/mp_rank_01_002/model_optim_rng.pt      (tp rank 1, pp rank 2)
    <dir>/iter_0000100/mp_rank_00/distrib_optim_dp000.pt      (one optimizer shard per dp rank)

``model_optim_rng.pt`` holds ``args, checkpoint_version, iteration, model, optimizer,
opt_param_scheduler, rng_state`` with Megatron ``GPTModel`` parameter names. The fused QKV weight is
stored the Megatron way (per KV group: its query heads, then its key head, then its value head);
in memory this repository keeps [all Q | all K | all V] so that Q, K and V are column slices; the QKV bias
of Qwen2-style models is permuted the same way. Pipeline stages number their layers from 0 in the file
(``decoder.layers.0`` of ``mp_rank_00_001`` is the stage's first layer), as Megatron does, while the model
objects use global layer numbers. The random-number state saved with the model is restored on load, and the
entry point fast-forwards its data stream by the saved iteration count.

The reference's root script only saves per-rank ``torch.save`` files and has no load path
(pretrain_llama.py:677-706, 862-863); its playground forwards Megatron's ``--save/--load``
(playground/simple_4d.py:430-432), which is the layout reproduced here.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..models.config import ModelConfig

CHECKPOINT_VERSION = 3.0


def qkv_to_megatron(w: torch.Tensor, hq: int, hkv: int, D: int) -> torch.Tensor:
    """[all Q | all K | all V] rows -> per-KV-group interleaved rows (local heads of one tp rank)."""
    H = w.shape[1]
    g = hq // hkv
    q = w[:hq * D].reshape(hkv, g * D, H)
    k = w[hq * D:(hq + hkv) * D].reshape(hkv, D, H)
    v = w[(hq + hkv) * D:].reshape(hkv, D, H)
    return torch.cat([q, k, v], dim=1).reshape((hq + 2 * hkv) * D, H)


def qkv_from_megatron(w: torch.Tensor, hq: int, hkv: int, D: int) -> torch.Tensor:
    H = w.shape[1]
    g = hq // hkv
    x = w.reshape(hkv, (g + 2) * D, H)
    q = x[:, :g * D].reshape(hq * D, H)
    k = x[:, g * D:(g + 1) * D].reshape(hkv * D, H)
    v = x[:, (g + 1) * D:].reshape(hkv * D, H)
    return torch.cat([q, k, v], dim=0)


def rank_dir(root: str, iteration: int, tp_rank: int, pp_rank: int, pp_size: int) -> str:
    name = f"mp_rank_{tp_rank:02d}" if pp_size == 1 else f"mp_rank_{tp_rank:02d}_{pp_rank:03d}"
    return os.path.join(root, f"iter_{iteration:07d}", name)


def file_key(name: str, first_layer: int) -> str:
    """Key of a parameter in the checkpoint file: layer numbers are local to the pipeline stage."""
    prefix = "decoder.layers."
    if not name.startswith(prefix):
        return name
    num, rest = name[len(prefix):].split(".", 1)
    return f"{prefix}{int(num) - first_layer}.{rest}"


def _first_layer(model) -> int:
    return int(getattr(model, "layer_range", (0, 0))[0])


def model_state_dict(model, cfg: ModelConfig, tp: int) -> dict:
    hq, hkv, D = cfg.heads_q // tp, cfg.heads_kv // tp, cfg.head_dim
    first = _first_layer(model)
    sd = {}
    for name, _ in model.store.shapes:
        t = model.store.p[name].detach()
        if name.endswith("linear_qkv.weight"):
            t = qkv_to_megatron(t, hq, hkv, D)
        elif name.endswith("linear_qkv.bias"):
            t = qkv_to_megatron(t[:, None], hq, hkv, D)[:, 0]
        sd[file_key(name, first)] = t.cpu().clone()
    return sd


def load_model_state_dict(model, sd: dict, cfg: ModelConfig, tp: int) -> None:
    hq, hkv, D = cfg.heads_q // tp, cfg.heads_kv // tp, cfg.head_dim
    first = _first_layer(model)
    for name, _ in model.store.shapes:
        t = sd[file_key(name, first)]
        if name.endswith("linear_qkv.weight"):
            t = qkv_from_megatron(t, hq, hkv, D)
        elif name.endswith("linear_qkv.bias"):
            t = qkv_from_megatron(t[:, None], hq, hkv, D)[:, 0]
        model.store.p[name].copy_(t.to(model.store.p[name].dtype))


def save_checkpoint(root: str, iteration: int, model, optimizer, cfg: ModelConfig, *, tp_rank: int = 0,
                    tp_size: int = 1, pp_rank: int = 0, pp_size: int = 1, dp_rank: int = 0, args: dict | None = None) -> str:
    d = rank_dir(root, iteration, tp_rank, pp_rank, pp_size)
    os.makedirs(d, exist_ok=True)
    if dp_rank == 0:
        payload = {
            "args": dict(args or {}),
            "checkpoint_version": CHECKPOINT_VERSION,
            "iteration": iteration,
            "model": model_state_dict(model, cfg, tp_size),
            "optimizer": {"step": optimizer.step_count, "distributed": True,
                          "param_layout": [(file_key(n, _first_layer(model)), list(s)) for n, s in model.store.shapes]},
            "opt_param_scheduler": {"lr": optimizer.cfg.lr, "num_steps": optimizer.step_count},
            "rng_state": [{"random_rng_state": None, "torch_rng_state": torch.get_rng_state(),
                           "cuda_rng_state": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}],
        }
        torch.save(payload, os.path.join(d, "model_optim_rng.pt"))
    opt_sd = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in optimizer.state_dict().items()}
    torch.save(opt_sd, os.path.join(d, f"distrib_optim_dp{dp_rank:03d}.pt"))
    if dist.is_initialized():
        dist.barrier()
    if (not dist.is_initialized()) or dist.get_rank() == 0:
        with open(os.path.join(root, "latest_checkpointed_iteration.txt"), "w") as f:
            f.write(str(iteration))
    return d


def latest_iteration(root: str) -> int | None:
    p = os.path.join(root, "latest_checkpointed_iteration.txt")
    if not os.path.exists(p):
        return None
    with open(p) as f:
        return int(f.read().strip())


def load_checkpoint(root: str, model, optimizer, cfg: ModelConfig, *, tp_rank: int = 0, tp_size: int = 1,
                    pp_rank: int = 0, pp_size: int = 1, dp_rank: int = 0, iteration: int | None = None) -> int:
    it = latest_iteration(root) if iteration is None else iteration
    if it is None:
        raise FileNotFoundError(f"no checkpoint under {root}")
    d = rank_dir(root, it, tp_rank, pp_rank, pp_size)
    payload = torch.load(os.path.join(d, "model_optim_rng.pt"), map_location="cpu", weights_only=False)
    load_model_state_dict(model, payload["model"], cfg, tp_size)
    opt_path = os.path.join(d, f"distrib_optim_dp{dp_rank:03d}.pt")
    if optimizer is not None and os.path.exists(opt_path):
        optimizer.load_state_dict(torch.load(opt_path, map_location="cpu", weights_only=False))
    elif optimizer is not None and hasattr(optimizer, "resync_master"):
        optimizer.resync_master()     # weights only: rebuild the fp32 master copy from them
    rng = (payload.get("rng_state") or [None])[0]
    if rng:
        if rng.get("torch_rng_state") is not None:
            torch.set_rng_state(rng["torch_rng_state"])
        if rng.get("cuda_rng_state") is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(rng["cuda_rng_state"])
    return int(payload["iteration"])
