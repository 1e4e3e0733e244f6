"""The regression-sweep runner (``python -m distca_b200.sweep``): case parsing, the command it builds for every
case, and a real two-case sweep of the entry point on two gloo ranks (CAD and the per-document CP baseline on
the same documents must report the same loss)."""
import json
import os
import subprocess
import sys

import pytest

from distca_b200 import sweep

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_case_parsing_and_arguments():
    c = sweep.Case.parse("llama3-8b 2 1 4 131072 distca 2 2 4 'distca subopt-mem'")
    assert (c.nodes, c.microbatches, c.tokens, c.mode, c.dp, c.pp, c.tp) == (2, 4, 131072, "distca", 2, 2, 4)
    assert c.world == 16 and c.comment == "distca subopt-mem"
    a = sweep.script_args(c, "prolong", 0.3, "out/x", steps=5, gpus_per_node=8, extra=["--nvtx"])
    s = " ".join(a)
    assert "--tp-size 4 --pp-size 2 --dp-size 2" in s and "--num-microbatch 4" in s and "--cad" in s
    assert "--sample-name prolong --change-long-doc-ratio 0.3" in s and "--elongate-factor 2" in s
    assert a[-1] == "--nvtx" and "--max-sample-id 5" in s
    b = sweep.Case.parse("llama3-8b 1 1 1 65536 wlbllm 4 1 2")
    assert "--baseline-mode percp" in " ".join(sweep.script_args(b, "wlbllm", 0.0, "o", 3, 8, []))
    with pytest.raises(ValueError):
        sweep.Case.parse("llama3-8b 1 1 1 65536 ping 4 1 2")
    with pytest.raises(ValueError):
        sweep.Case.parse("llama3-8b 1 1")
    with pytest.raises(ValueError):                              # 8 ranks asked, one node of 4 GPUs given
        sweep.script_args(b, "wlbllm", 0.0, "o", 3, 4, [])
    with pytest.raises(ValueError):                              # the baseline has no pipeline stages
        sweep.script_args(sweep.Case.parse("llama3-8b 1 1 4 65536 baseline 2 2 2"), "mixture", 0.0, "o", 3, 8, [])


def test_dry_run_prints_one_launch_per_case(capsys):
    rc = sweep.main(["--dry-run", "--gpus-per-node", "8", "--case", "llama3-8b 1 1 4 131072 distca 2 2 2 a",
                     "--case", "llama3-8b 1 1 1 131072 baseline 4 1 2 b", "--dist", "mixture 0.0", "--dist", "prolong 0.3"])
    out = capsys.readouterr().out
    assert rc == 0 and out.count("torch.distributed.run") == 4 and out.count("--baseline-mode percp") == 2


def test_two_case_sweep_on_gloo_ranks(tmp_path):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "distca_b200.sweep", "--gpus-per-node", "2", "--steps", "2", "--output-dir", str(tmp_path),
           "--port", "29720", "--case", "tiny 1 1 1 1024 distca 2 1 1 cad", "--case", "tiny 1 1 1 1024 baseline 2 1 1 percp",
           "--dist", "loguniform 0.0"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    rows = [json.loads(l) for l in open(tmp_path / "sweep.jsonl")]
    assert [x["mode"] for x in rows] == ["distca", "baseline"] and all(x["rc"] == 0 for x in rows)
    a, b = (x["result"]["last_loss"] for x in rows)
    assert abs(a - b) < 1e-4, (a, b)
    assert "tokens/s" in r.stdout and "percp" in r.stdout


def test_collective_micro_benchmark_on_gloo_ranks_feeds_the_network_model():
    from distca_b200.planner import NetworkModel
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", "-m", "distca_b200.utils.net_bench", "--sizes-mb", "1", "4", "--iters", "2", "--warmup", "1",
           "--ops", "all_gather", "all_reduce", "all_to_all", "push_all_gather"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rows = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert {x["op"] for x in rows} == {"all_gather", "all_reduce", "all_to_all"}      # the peer-store kernel needs GPUs
    assert all(x["world"] == 2 and x["ms"] > 0 and x["bus_gbs"] > 0 for x in rows) and len(rows) == 6
    net = NetworkModel.from_sweep(r.stdout.splitlines())
    assert net.ms("all_gather", 2, rows[0]["bytes_per_rank"]) == rows[0]["ms"]
