"""End-to-end CLI run on CPU: train, write artifacts, save a Megatron-layout checkpoint, resume."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, cwd):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", WORLD_SIZE="1", RANK="0", LOCAL_RANK="0")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "pretrain_llama.py"), *args], cwd=cwd, env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def test_cli_train_save_resume(tmp_path):
    out = str(tmp_path / "run")
    ck = str(tmp_path / "ckpt")
    base = ["--model", "tiny", "--num-layers", "1", "--num-tokens", "256", "--sample-name", "loguniform64",
            "--output-dir", out, "--lr", "1e-3"]
    _run(base + ["--max-sample-id", "2", "--save", ck, "--save-interval", "2", "--log-memory"], str(tmp_path))
    assert os.path.exists(os.path.join(out, "config.json"))
    recs = [json.loads(l) for l in open(os.path.join(out, "benchmark.raw.jsonl"))]
    assert len(recs) == 2 and all(r["loss"] == r["loss"] for r in recs)
    assert os.path.exists(os.path.join(out, "benchmark.json"))
    assert open(os.path.join(ck, "latest_checkpointed_iteration.txt")).read().strip() == "2"
    f = os.path.join(ck, "iter_0000002", "mp_rank_00", "model_optim_rng.pt")
    payload = torch.load(f, map_location="cpu", weights_only=False)
    assert {"args", "checkpoint_version", "iteration", "model", "optimizer", "opt_param_scheduler", "rng_state"} <= set(payload)
    assert "decoder.layers.0.self_attention.linear_qkv.weight" in payload["model"]
    assert os.path.exists(os.path.join(ck, "iter_0000002", "mp_rank_00", "distrib_optim_dp000.pt"))
    log = _run(base + ["--max-sample-id", "1", "--load", ck], str(tmp_path))
    assert "resumed from" in log and "iteration 2" in log


def test_qkv_layout_roundtrip():
    from distca_b200.utils.checkpoint import qkv_from_megatron, qkv_to_megatron
    hq, hkv, D, H = 8, 2, 4, 6
    w = torch.arange((hq + 2 * hkv) * D * H, dtype=torch.float32).reshape(-1, H)
    m = qkv_to_megatron(w, hq, hkv, D)
    assert torch.equal(qkv_from_megatron(m, hq, hkv, D), w)
    # first group: its 4 query heads, then key head 0, then value head 0
    g = hq // hkv
    assert torch.equal(m[:g * D], w[:g * D])
    assert torch.equal(m[g * D:(g + 1) * D], w[hq * D:hq * D + D])
    assert torch.equal(m[(g + 1) * D:(g + 2) * D], w[(hq + hkv) * D:(hq + hkv) * D + D])


def test_pipeline_stage_and_qkv_bias_checkpoints_use_megatron_keys():
    """Round trip against a hand-built state dict with Megatron keys: a pipeline stage's file numbers its
    layers from 0, and the QKV bias of a Qwen2-style model is stored per KV group like the weight."""
    from distca_b200.models.config import ModelConfig
    from distca_b200.models.llama import LlamaModel
    from distca_b200.utils.checkpoint import (file_key, load_model_state_dict, model_state_dict, qkv_from_megatron,
                                              qkv_to_megatron)
    cfg = ModelConfig(name="q", num_layers=4, hidden=32, heads_q=4, heads_kv=2, head_dim=8, ffn=48, vocab=64,
                      qkv_bias=True, max_position=64)
    hq, hkv, D = cfg.heads_q, cfg.heads_kv, cfg.head_dim
    # second stage of two: global layers 2 and 3
    stage = LlamaModel(cfg, "cpu", layer_range=(2, 4), first_stage=False, last_stage=True, dtype=torch.float32, seed=3)
    sd = model_state_dict(stage, cfg, tp=1)
    assert "decoder.layers.0.self_attention.linear_qkv.weight" in sd and "decoder.layers.1.mlp.linear_fc2.weight" in sd
    assert not any(k.startswith("decoder.layers.2.") or k.startswith("decoder.layers.3.") for k in sd)
    assert file_key("decoder.layers.3.mlp.linear_fc1.weight", 2) == "decoder.layers.1.mlp.linear_fc1.weight"
    assert file_key("output_layer.weight", 2) == "output_layer.weight"
    # the bias is permuted exactly like the rows of the weight
    b = stage.store.p["decoder.layers.2.self_attention.linear_qkv.bias"]
    w = stage.store.p["decoder.layers.2.self_attention.linear_qkv.weight"]
    assert torch.equal(sd["decoder.layers.0.self_attention.linear_qkv.bias"], qkv_to_megatron(b[:, None], hq, hkv, D)[:, 0])
    g = hq // hkv
    assert torch.equal(sd["decoder.layers.0.self_attention.linear_qkv.bias"][g * D:(g + 1) * D], b[hq * D:hq * D + D])
    assert torch.equal(sd["decoder.layers.0.self_attention.linear_qkv.weight"], qkv_to_megatron(w, hq, hkv, D))
    # a state dict written by hand with Megatron keys loads into the right global layers
    hand = {k: torch.randn_like(v) for k, v in sd.items()}
    other = LlamaModel(cfg, "cpu", layer_range=(2, 4), first_stage=False, last_stage=True, dtype=torch.float32, seed=9)
    load_model_state_dict(other, hand, cfg, tp=1)
    torch.testing.assert_close(other.store.p["decoder.layers.3.mlp.linear_fc2.weight"], hand["decoder.layers.1.mlp.linear_fc2.weight"])
    torch.testing.assert_close(other.store.p["decoder.layers.2.self_attention.linear_qkv.bias"],
                               qkv_from_megatron(hand["decoder.layers.0.self_attention.linear_qkv.bias"][:, None], hq, hkv, D)[:, 0])
    for k, v in model_state_dict(other, cfg, tp=1).items():
        torch.testing.assert_close(v, hand[k])


def test_checkpoint_restores_rng_state(tmp_path):
    from distca_b200.models.config import ModelConfig, TrainConfig
    from distca_b200.models.llama import LlamaModel
    from distca_b200.parallel.optimizer import ShardedAdam
    from distca_b200.utils.checkpoint import load_checkpoint, save_checkpoint
    cfg = ModelConfig(name="r", num_layers=1, hidden=32, heads_q=2, heads_kv=1, head_dim=16, ffn=48, vocab=64, max_position=64)
    m = LlamaModel(cfg, "cpu", dtype=torch.float32)
    opt = ShardedAdam(m.store, TrainConfig())
    torch.manual_seed(1234)
    torch.rand(3)
    save_checkpoint(str(tmp_path), 5, m, opt, cfg)
    want = torch.rand(4)
    torch.manual_seed(99)
    assert load_checkpoint(str(tmp_path), m, opt, cfg) == 5
    assert torch.equal(torch.rand(4), want)


def test_bench_named_configs_are_the_contract_layouts():
    """bench.py --config: the three fixed 8-GPU layouts (TP=8 at 64K with 8 sequences per step; TP=2 x PP=2 x DP=2
    at 128K; 34B shape at TP=4 x PP=2 and 256K with full recompute)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_mod", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    from distca_b200.models.config import get_model_config
    c = bench.NAMED_CONFIGS
    assert set(c) == {"tp8_64k", "4d_128k", "34b_256k"}
    for v in c.values():
        assert v["tp"] * v["pp"] * v["dp"] == 8
        cfg = get_model_config(v["model"])
        assert cfg.heads_kv % v["tp"] == 0 and cfg.num_layers % v["pp"] == 0
        assert v["pp"] == 1 or v["microbatches"] >= v["pp"]
    assert (c["tp8_64k"]["seq_len"], c["tp8_64k"]["seqs_per_rank"]) == (65536, 8)
    assert (c["4d_128k"]["tp"], c["4d_128k"]["pp"], c["4d_128k"]["dp"], c["4d_128k"]["seq_len"]) == (2, 2, 2, 131072)
    m = get_model_config("codellama-34b")
    assert (m.num_layers, m.hidden, m.heads_q, m.heads_kv, m.ffn, m.vocab) == (48, 8192, 64, 8, 22016, 32000)
    assert c["34b_256k"]["recompute"] == "full" and c["34b_256k"]["seq_len"] == 262144


def test_cli_call_trace_and_profile_of_one_step(tmp_path):
    """--trace-calls-step writes the Python calls of this package during that step (which rank is where),
    --torch-profile-step a chrome trace of that step."""
    out = str(tmp_path / "run")
    _run(["--model", "tiny", "--num-layers", "1", "--num-tokens", "256", "--sample-name", "loguniform64", "--output-dir", out,
          "--max-sample-id", "2", "--trace-calls-step", "1", "--torch-profile-step", "1"], str(tmp_path))
    calls = open(os.path.join(out, "calls.rank0.log")).read()
    assert "-> train_step (trainer.py:" in calls and "<- train_step" in calls and "forward_backward" in calls
    trace = json.load(open(os.path.join(out, "trace.rank0.json")))
    assert trace["traceEvents"]
