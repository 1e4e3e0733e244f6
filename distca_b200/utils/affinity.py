"""CPU binding per local rank and the per-rank environment record.

Every rank runs a training thread, a planning thread and a heartbeat thread; eight ranks on one host otherwise
wander over all cores. ``bind(local_rank, local_world)`` gives each rank its own contiguous slice of the CPUs the
job is allowed to use (contiguous slices follow the sockets on hosts that number cores socket by socket, so a
rank's threads stay near its GPU's host memory). ``dump_environment`` writes what the reference's launcher
wrapper records per rank: the environment and the GPU topology.

Reference: playground/utils/cpu_affinity.py:10-58 (fixed 16 cores per process), utils/bind_and_exec.sh:11-45
(per-rank log files, ``env`` dump, ``nvidia-smi topo``), tests/check_cpu_binding.py.
"""
from __future__ import annotations

import os
import shutil
import subprocess


def allowed_cpus() -> list[int]:
    if hasattr(os, "sched_getaffinity"):
        return sorted(os.sched_getaffinity(0))
    return list(range(os.cpu_count() or 1))


def plan_affinity(local_rank: int, local_world: int, cpus: list[int] | None = None, per_proc: int | None = None) -> list[int]:
    """The CPUs of ``local_rank``: slice ``local_rank`` of ``local_world`` equal contiguous slices of ``cpus``
    (default: the CPUs this process may use), at most ``per_proc`` of them. With fewer CPUs than ranks, ranks share
    (round robin) instead of failing."""
    cpus = sorted(cpus if cpus is not None else allowed_cpus())
    if not 0 <= local_rank < local_world:
        raise ValueError(f"local rank {local_rank} outside 0..{local_world - 1}")
    n = len(cpus) // local_world
    if n == 0:
        return [cpus[local_rank % len(cpus)]]
    mine = cpus[local_rank * n:(local_rank + 1) * n]
    return mine[:per_proc] if per_proc else mine


def format_cpus(cpus: list[int]) -> str:
    """``[0, 1, 2, 3, 8, 9]`` -> ``"0-3,8-9"``."""
    out, i = [], 0
    cpus = sorted(cpus)
    while i < len(cpus):
        j = i
        while j + 1 < len(cpus) and cpus[j + 1] == cpus[j] + 1:
            j += 1
        out.append(str(cpus[i]) if i == j else f"{cpus[i]}-{cpus[j]}")
        i = j + 1
    return ",".join(out)


def bind(local_rank: int, local_world: int, per_proc: int | None = None, logger=None) -> list[int]:
    """Bind this process (and the threads it starts later) to its slice; returns the CPUs. No-op where the
    platform has no ``sched_setaffinity``."""
    mine = plan_affinity(local_rank, local_world, per_proc=per_proc)
    if hasattr(os, "sched_setaffinity"):
        os.sched_setaffinity(0, mine)
    if logger is not None:
        logger.info("cpu affinity of local rank %d: %s", local_rank, format_cpus(mine))
    return mine


def dump_environment(out_dir: str, rank: int, local_rank: int) -> str:
    """``<out_dir>/envs/<host>.r<rank>.lr<local>.env``: environment variables, CPU binding and (local rank 0, when
    ``nvidia-smi`` exists) the GPU topology matrix. Reading only: no GPU setting is touched."""
    host = os.uname().nodename
    d = os.path.join(out_dir, "envs")
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"{host}.r{rank}.lr{local_rank}.env")
    with open(path, "w") as f:
        for k in sorted(os.environ):
            f.write(f"{k}={os.environ[k]}\n")
        f.write(f"# cpus: {format_cpus(allowed_cpus())}\n")
        smi = shutil.which("nvidia-smi")
        if smi and local_rank == 0:
            try:
                topo = subprocess.run([smi, "topo", "-m"], capture_output=True, text=True, timeout=30).stdout
                f.write("# nvidia-smi topo -m\n" + "".join(f"# {ln}\n" for ln in topo.splitlines()))
            except Exception as e:  # the record is best effort
                f.write(f"# nvidia-smi topo failed: {e!r}\n")
    return path
