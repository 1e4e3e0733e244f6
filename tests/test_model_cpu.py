"""Hand-written layer/model backward against autograd on CPU (fp64): engine logic without a GPU."""
import numpy as np
import pytest
import torch

from distca_b200.models.config import ModelConfig
from distca_b200.models.llama import Batch, LlamaModel, LocalCoreAttention
from distca_b200.models.reference import reference_loss
from distca_b200.ops.attention import AttnPlan, AttnTasks


def _batch(cfg, doc_lens, seed=0):
    g = torch.Generator().manual_seed(seed)
    T = sum(doc_lens)
    ids = torch.randint(0, cfg.vocab, (T,), generator=g)
    labels = torch.roll(ids, -1)
    pos = torch.cat([torch.arange(L, dtype=torch.int32) for L in doc_lens])
    ends = np.cumsum(doc_lens) - 1
    labels[ends] = -100
    return Batch(ids, labels, pos, int((labels >= 0).sum()))


@pytest.mark.parametrize("recompute", ["none", "full", "keep_attn"])
def test_manual_backward_matches_autograd(recompute):
    cfg = ModelConfig(name="t", num_layers=2, hidden=64, heads_q=4, heads_kv=2, head_dim=16, ffn=96, vocab=128,
                      max_position=512)
    doc_lens = [40, 7, 81]
    model = LlamaModel(cfg, "cpu", dtype=torch.float64, recompute=recompute, lm_head_chunk=50)
    batch = _batch(cfg, doc_lens)
    tasks = AttnTasks.from_doc_lens(doc_lens)
    ca = LocalCoreAttention(cfg)
    ca.set_batch(AttnPlan(tasks, "cpu", need_backward=False))
    model.store.zero_grad()
    loss, _ = model.forward_backward(batch, ca)

    params = {n: t.detach().clone().requires_grad_(True) for n, t in model.store.p.items()}
    ref = reference_loss(cfg, params, batch.ids, batch.labels, batch.pos, tasks, batch.num_valid_global)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-6
    for n, t in params.items():
        torch.testing.assert_close(model.store.g[n], t.grad, rtol=1e-4, atol=1e-7, msg=lambda m: f"{n}: {m}")
    ev = model.forward_loss(batch, ca)
    assert abs(ev.item() - ref.item()) < 1e-6


def test_qkv_bias_model_matches_autograd():
    """Qwen2-style architecture: bias on the Q/K/V projection (added before RoPE), hand-written
    backward including the bias gradient."""
    cfg = ModelConfig(name="q", num_layers=2, hidden=64, heads_q=4, heads_kv=2, head_dim=16, ffn=96, vocab=128,
                      max_position=512, qkv_bias=True)
    doc_lens = [33, 95]
    model = LlamaModel(cfg, "cpu", dtype=torch.float64, recompute="keep_attn", lm_head_chunk=50)
    assert any(n.endswith("linear_qkv.bias") for n, _ in model.store.shapes)
    batch = _batch(cfg, doc_lens)
    tasks = AttnTasks.from_doc_lens(doc_lens)
    ca = LocalCoreAttention(cfg)
    ca.set_batch(AttnPlan(tasks, "cpu", need_backward=False))
    model.store.zero_grad()
    loss, _ = model.forward_backward(batch, ca)
    params = {n: t.detach().clone().requires_grad_(True) for n, t in model.store.p.items()}
    ref = reference_loss(cfg, params, batch.ids, batch.labels, batch.pos, tasks, batch.num_valid_global)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-6
    for n, t in params.items():
        torch.testing.assert_close(model.store.g[n], t.grad, rtol=1e-4, atol=1e-7, msg=lambda m: f"{n}: {m}")


def test_hf_config_mapping_llama_and_qwen2():
    base = {"num_hidden_layers": 4, "hidden_size": 512, "num_attention_heads": 8, "num_key_value_heads": 2,
            "intermediate_size": 1376, "vocab_size": 1000, "rms_norm_eps": 1e-6, "rope_theta": 1e6}
    llama = ModelConfig.from_hf({**base, "architectures": ["LlamaForCausalLM"]})
    qwen = ModelConfig.from_hf({**base, "architectures": ["Qwen2ForCausalLM"], "tie_word_embeddings": True})
    assert not llama.qkv_bias and qwen.qkv_bias and qwen.tie_embeddings and llama.head_dim == 64
    assert qwen.num_params() == llama.num_params() + 4 * llama.qkv_dim - 1000 * 512


def test_rotary_table_grows_for_documents_longer_than_max_position():
    """The host guard in front of the RoPE kernels: a document longer than the configuration's
    ``max_position`` extends the table before anything indexes it, and the result equals a model that
    was configured with the longer table from the start."""
    kw = dict(name="t", num_layers=1, hidden=32, heads_q=2, heads_kv=1, head_dim=16, ffn=48, vocab=64)
    short = LlamaModel(ModelConfig(max_position=32, **kw), "cpu", dtype=torch.float64)
    long_ = LlamaModel(ModelConfig(max_position=128, **kw), "cpu", dtype=torch.float64)
    assert short.rope_table.shape[0] == 32
    short.ensure_positions(20)
    assert short.rope_table.shape[0] == 32           # still fits: untouched
    short.ensure_positions(100)
    assert short.rope_table.shape[0] == 128
    torch.testing.assert_close(short.rope_table, long_.rope_table)
    doc_lens = [100, 12]
    batch = _batch(short.cfg, doc_lens)
    losses = []
    for m in (short, long_):
        ca = LocalCoreAttention(m.cfg)
        ca.set_batch(AttnPlan(AttnTasks.from_doc_lens(doc_lens), "cpu", need_backward=False))
        losses.append(m.forward_loss(batch, ca).item())
    assert abs(losses[0] - losses[1]) < 1e-9


def test_finite_check_names_the_layer_that_produced_the_first_nan():
    cfg = ModelConfig(name="t", num_layers=3, hidden=64, heads_q=4, heads_kv=2, head_dim=16, ffn=96, vocab=128,
                      max_position=512)
    doc_lens = [40, 24]
    model = LlamaModel(cfg, "cpu", dtype=torch.float64, recompute="full", lm_head_chunk=50)
    batch = _batch(cfg, doc_lens)
    ca = LocalCoreAttention(cfg)
    ca.set_batch(AttnPlan(AttnTasks.from_doc_lens(doc_lens), "cpu", need_backward=False))
    model.check_finite = True
    model.store.zero_grad()
    loss, _ = model.forward_backward(batch, ca)            # clean weights: nothing raised
    assert torch.isfinite(loss)
    model.store.p["decoder.layers.1.mlp.linear_fc2.weight"][0, 0] = float("nan")
    with pytest.raises(FloatingPointError, match="forward output of layer 1"):
        model.forward_backward(batch, ca)
    model.check_finite = False
    loss, _ = model.forward_backward(batch, ca)            # without the check the NaN only shows in the loss
    assert not torch.isfinite(loss)
