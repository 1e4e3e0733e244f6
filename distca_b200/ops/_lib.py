"""ctypes access to ``_kernels.so`` (the sm_100a kernels) and the per-device status word.

The kernels never trap: a wait that runs out or a failed bounds check writes a code into a
device-resident status word and returns. :func:`check_status` reads it back and raises.
On a machine with a GPU a missing library is an error, never a silent fallback.

The reference binds its CUDA library through torch custom ops (csrc/bindings/bindings.cpp, csrc/bindings/all_to_all.cpp) and
ends the process on a CUDA error (csrc/core/cuda_utils.h:11-18); here launchers return error codes.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_ROOT = Path(__file__).resolve().parent.parent
_LIB = None
_STATUS: dict[int, torch.Tensor] = {}

STATUS_NAMES = {0: "ok", 1: "mbarrier wait ran out", 2: "peer signal wait ran out",
                3: "bounds check failed"}

ERR_NAMES = {-1: "bad argument (shape/alignment)", -2: "CUDA driver entry point unavailable",
             -3: "tensor map encoding failed", -4: "size beyond the supported maximum"}


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """Load (building first if the sources are newer and nvcc exists) the kernel library."""
    global _LIB
    if _LIB is None:
        path = Path(os.environ["DISTCA_KERNELS_SO"]) if os.environ.get("DISTCA_KERNELS_SO") else _ROOT / "_kernels.so"
        if os.environ.get("DISTCA_KERNELS_SO"):
            pass        # an explicitly named build of the same sources (e.g. with other -D switches): never rebuilt here
        elif not path.exists() or os.environ.get("DISTCA_REBUILD", "0") == "1":
            from .. import build
            build.build_kernels()
        if not path.exists():
            raise KernelError(f"{path} is missing; run `python -m distca_b200.build`")
        _LIB = ctypes.CDLL(str(path))
    return _LIB


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    if dev is None:
        dev = torch.cuda.current_device()
    t = _STATUS.get(dev)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=f"cuda:{dev}")
        _STATUS[dev] = t
    return t


def check_status(device=None, what: str = "kernel") -> None:
    """Synchronising read of the status word; raises :class:`KernelError` when non-zero."""
    t = status_word(device)
    v = int(t[0].item())
    if v != 0:
        t.zero_()
        raise KernelError(f"{what}: device status {v} ({STATUS_NAMES.get(v, 'unknown')})")


LAUNCHES = 0  # kernels of this library launched so far (counted per successful launcher call)
_KERNELS_PER_CALL = {"flash_bwd": 3, "rmsnorm_bwd": 2}


def check_rc(rc: int, what: str) -> None:
    global LAUNCHES
    if rc == 0:
        LAUNCHES += _KERNELS_PER_CALL.get(what, 1)
        return
    if rc in ERR_NAMES:
        raise KernelError(f"{what}: {ERR_NAMES[rc]}")
    raise KernelError(f"{what}: CUDA error {rc} (the library printed its name to stderr)")


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


c_int = ctypes.c_int
c_long = ctypes.c_long
c_float = ctypes.c_float
c_void_p = ctypes.c_void_p
