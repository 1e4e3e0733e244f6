"""The multi-rank self-checks (``python -m distca_b200.runtime.selfcheck``) as two gloo ranks on the CPU: the same
program that compares the GPU paths with one another, here on the CPU restatements of the kernels, so its own
logic (batch sources, comparisons, exit codes) is pinned without a GPU."""
import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(check, extra):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), "-m", "distca_b200.runtime.selfcheck", check, "--model", "tiny",
           "--tokens", "1024", "--steps", "2", *extra]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


def test_spanning_documents_against_per_document_cp_on_two_gloo_ranks():
    res = _run("span", [])
    assert res["ok"] and res["longest_document"] > res["tokens_per_rank"], res
    assert all(abs(x - y) < 1e-4 for x, y in zip(res["loss_percp"], res["loss_span"])), res


@pytest.mark.parametrize("extra", [["--pp", "2", "--microbatches", "2", "--nano", "2", "--recompute", "keep_attn"]],
                         ids=["pp2-pingpong"])
def test_cad_against_local_attention_on_two_gloo_ranks(extra):
    res = _run("cad", extra)
    assert res["ok"] and res["worst_tensor_rel_err"] < 1e-4, res
