"""The benchmark program end to end on CPU ranks (tiny model, gloo, stand-ins for the CUDA timing calls): the
JSON contract of the headline path at 1 and 2 ranks, with ping-pong nano-batches, and of the per-document CP arm."""
import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNER = os.path.join(ROOT, "tests", "bench_cpu_runner.py")
KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
        "dtype", "data", "config", "e2e", "gpu_launches", "clocks"}


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(world, extra):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
    if world == 1:
        cmd = [sys.executable, RUNNER, *extra]
        env.update(WORLD_SIZE="1", RANK="0", LOCAL_RANK="0")
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
               "127.0.0.1", "--master-port", str(_port()), RUNNER, *extra]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, lines                      # rank 0 prints ONE line
    return json.loads(lines[0])


def test_headline_line_on_one_rank():
    out = _run(1, [])
    assert KEYS <= set(out) and out["n_gpus"] == 1 and out["steps"] == 1 and out["warmup"] == 1
    assert out["value"] > 0 and out["e2e"]["value"] > 0 and out["e2e"]["h2d_bytes_per_step"] == 1024 * 20
    assert out["config"]["parallelism"] == "dp1" and out["config"]["seq_len"] == 1024 and out["scaling"] == "weak"
    assert "roofline" not in out and "cad" not in out


@pytest.mark.parametrize("extra", [[], ["--nano-batches", "2"]], ids=["cad", "pingpong"])
def test_headline_line_on_two_ranks_with_disaggregation(extra):
    out = _run(2, extra)
    assert KEYS <= set(out) and out["n_gpus"] == 2 and out["config"]["parallelism"] == "dp2-cad"
    assert out["config"]["global_batch"] == 2 and out["config"]["nano_batches"] == (2 if extra else 1)
    assert set(out["roofline"]["paths"]) == {"qkv_gemm_rope_dispatch", "attention_forward_with_output_return",
                                             "attention_backward_with_gradient_return",
                                             "gradient_reduce_scatter_adam_all_gather"} and "error" not in out["roofline"]
    assert out["cad"]["planned_imbalance_after"] <= out["cad"]["planned_imbalance_before"] + 1e-9
    assert abs(out["loss_first_last"][0] - 10.4) < 0.2


def test_per_document_cp_arm_on_the_headline_layout():
    out = _run(2, ["--baseline-mode", "percp"])
    assert out["config"]["parallelism"] == "tp1-cp2-percp" and out["n_gpus"] == 2 and out["value"] > 0
    assert out["percp"]["kv_bytes_received_per_layer_and_rank"] > 0 and "cad" not in out


@pytest.mark.parametrize("extra,parallelism", [
    (["--config", "4d_128k", "--nano-batches", "2"], "tp2-pp2-dp2-cad"),
    (["--config", "4d_128k", "--baseline-mode", "percp"], "tp2-cp4-percp"),
    (["--config", "tp8_64k", "--model", "tiny-8kv"], "tp8-pp1-dp1"),
    (["--config", "34b_256k", "--model", "tiny-8kv"], "tp4-pp2-dp1-cad"),
], ids=["4d-pingpong", "4d-percp", "tp8", "tp4-pp2"])
def test_fixed_eight_rank_layouts_run_end_to_end_on_small_models(extra, parallelism):
    """The fixed 8-rank layouts of ``bench.py --config`` (tensor x pipeline x data parallel with disaggregation and
    ping-pong, its per-document CP baseline, TP=8, TP=4 x PP=2 with full recompute) through the same program on
    eight CPU ranks with a small model in place of the layout's own."""
    out = _run(8, extra)
    assert KEYS <= set(out) and out["n_gpus"] == 8 and out["config"]["parallelism"] == parallelism
    assert out["value"] > 0 and out["e2e"]["value"] > 0 and all(x == x for x in out["loss_first_last"])
    if "pp2" in parallelism:
        assert out["pipeline"]["ticks"] == 4 and abs(out["pipeline"]["bubble_fraction"] - 1 / 3) < 1e-9
    if extra[-2:] == ["--nano-batches", "2"]:
        assert out["config"]["nano_batches"] == 2
