"""Multi-node launcher: one ``torchrun`` per node, each driving that node's GPUs.

    python -m distca_b200.launch --nodes nodeA,nodeB --gpus-per-node 8 --output-dir runs/x -- \\
        pretrain_llama.py --tp-size 2 --pp-size 2 --num-tokens 131072 ...

Nodes are reached with ``ssh`` (the first one is the rendezvous host); ``--nodes localhost`` or no
``--nodes`` runs in place without ssh. ``{hostname}`` in the command is replaced per node and each node's
output is streamed and, with ``--output-dir``, saved as ``<hostname>.log``. ``--dry-run`` prints the
commands only. ``--nsys PREFIX`` wraps every node's ``torchrun`` in ``nsys profile -o PREFIX.<hostname>
--trace=cuda,nvtx`` (the reference's ``ENABLE_NSYS`` switch, pretrain_llama.sh:243-246; run the script with
``--nvtx`` to get per-tick / per-layer / per-phase ranges; ``nsys`` itself must be installed on the nodes).
The reference does the same job with one Ray task per 8-GPU node
(distca/ray_launch.py:11-137); Ray is not a dependency here.
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys
import threading


def build_commands(nodes: list[str], gpus_per_node: int, script_args: list[str], port: int = 29500,
                   workdir: str | None = None, python: str = sys.executable, nsys: str | None = None
                   ) -> list[tuple[str, str]]:
    """(node, shell command) per node."""
    master = "127.0.0.1" if nodes == ["localhost"] else nodes[0]
    out = []
    for rank, node in enumerate(nodes):
        args = [a.replace("{hostname}", node) for a in script_args]
        cmd = [python, "-m", "torch.distributed.run", f"--nnodes={len(nodes)}", f"--node-rank={rank}",
               f"--nproc-per-node={gpus_per_node}", "--master-addr", master, "--master-port", str(port), *args]
        if nsys:
            cmd = ["nsys", "profile", "-o", f"{nsys}.{node}", "--trace=cuda,nvtx", "--force-overwrite=true", *cmd]
        line = " ".join(shlex.quote(c) for c in cmd)
        if workdir:
            line = f"cd {shlex.quote(workdir)} && {line}"
        if node != "localhost":
            line = f"ssh -o BatchMode=yes {shlex.quote(node)} {shlex.quote(line)}"
        out.append((node, line))
    return out


def _stream(node: str, proc: subprocess.Popen, log_path: str | None, quiet: bool) -> None:
    log = open(log_path, "w") if log_path else None
    for line in proc.stdout:
        if not quiet:
            sys.stdout.write(f"[{node}] {line}")
        if log:
            log.write(line)
    if log:
        log.close()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--nodes", default="localhost", help="comma-separated host names")
    ap.add_argument("--gpus-per-node", type=int, default=8)
    ap.add_argument("--port", type=int, default=29500)
    ap.add_argument("--workdir", default=os.getcwd())
    ap.add_argument("--output-dir", default=None)
    ap.add_argument("--no-duplicate-log", action="store_true", help="print only the first node's output")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--nsys", default=None, metavar="PREFIX", help="profile every node's run with nsys into PREFIX.<hostname>")
    ap.add_argument("script", nargs=argparse.REMAINDER, help="-- script.py args...")
    a = ap.parse_args(argv)
    script = a.script[1:] if a.script and a.script[0] == "--" else a.script
    if not script:
        ap.error("nothing to launch")
    nodes = [n for n in a.nodes.split(",") if n]
    cmds = build_commands(nodes, a.gpus_per_node, script, a.port, a.workdir, nsys=a.nsys)
    if a.dry_run:
        for node, c in cmds:
            print(f"[{node}] {c}")
        return 0
    if a.output_dir:
        os.makedirs(a.output_dir, exist_ok=True)
    procs, threads = [], []
    for i, (node, c) in enumerate(cmds):
        p = subprocess.Popen(c, shell=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, bufsize=1)
        t = threading.Thread(target=_stream, daemon=True, args=(
            node, p, os.path.join(a.output_dir, f"{node}.log") if a.output_dir else None,
            a.no_duplicate_log and i > 0))
        t.start()
        procs.append(p)
        threads.append(t)
    rc = 0
    for p, t in zip(procs, threads):
        rc = p.wait() or rc
        t.join()
    return rc


if __name__ == "__main__":
    sys.exit(main())
