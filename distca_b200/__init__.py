"""distca_b200: long-context training with core-attention disaggregation on B200.

The names a user of the reference looks for, by their place here (imported on first use, so that
``import distca_b200`` stays cheap and works on a machine without a GPU):

    Planner, PlannerConfig, AsyncPlanner          planner (reference: distca/planner/planner.py:550-829)
    default_cost_model, default_time_model        cost tables of the B200 kernels (distca/timemodule/compute.py:75-118)
    ModelConfig, ParallelConfig, TrainConfig, get_model_config
    Trainer, PipelineTrainer, BatchSource, init_distributed     workers (distca/utils/worker.py, training_utils.py)
    CadRuntime, GlooCadRuntime                    dispatch / serve / return (distca/runtime/dispatch_fn.py,
                                                  distca/runtime/megatron/ops/fused_comm_attn.py)
    PeerArena, SignalBoard                        symmetric buffers + signals (distca/runtime/attn_kernels/dispatch.py)
    save_checkpoint, load_checkpoint              Megatron-layout checkpoints
"""
from __future__ import annotations

import importlib

__version__ = "0.2.0"

_EXPORTS = {
    "Planner": ".planner", "PlannerConfig": ".planner", "AsyncPlanner": ".planner",
    "default_cost_model": ".planner", "default_time_model": ".planner",
    "ModelConfig": ".models.config", "ParallelConfig": ".models.config", "TrainConfig": ".models.config",
    "get_model_config": ".models.config",
    "Trainer": ".runtime.trainer", "BatchSource": ".runtime.trainer", "init_distributed": ".runtime.trainer",
    "PipelineTrainer": ".parallel.pipeline",
    "CadRuntime": ".parallel.cad", "GlooCadRuntime": ".parallel.cad_cpu",
    "PeerArena": ".parallel.p2p", "SignalBoard": ".parallel.p2p",
    "save_checkpoint": ".utils.checkpoint", "load_checkpoint": ".utils.checkpoint",
}

__all__ = sorted(_EXPORTS) + ["__version__"]


def __getattr__(name: str):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(importlib.import_module(mod, __name__), name)
    globals()[name] = value
    return value


def __dir__():
    return __all__
