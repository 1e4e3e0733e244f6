"""Model and parallelism configuration.

Built-in shapes cover the models the reference's scripts name (Llama-3-8B via
DeepSeek-R1-Distill-Llama-8B and CodeLlama-34B, benchmarks/example-4d-parallel/run4d.sh:34-55) plus
tiny shapes for tests. ``ModelConfig.from_hf`` accepts a HuggingFace ``config.json`` dict the way the
reference maps ``AutoConfig`` fields (distca/utils/megatron_test_utils.py:281-398).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field


@dataclass
class ModelConfig:
    name: str = "tiny"
    num_layers: int = 2
    hidden: int = 256
    heads_q: int = 4
    heads_kv: int = 2
    head_dim: int = 64
    ffn: int = 688
    vocab: int = 32000
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    tie_embeddings: bool = False
    qkv_bias: bool = False      # Qwen2-style bias on the Q/K/V projections (no other linear has a bias)
    init_std: float = 0.02
    max_position: int = 131072

    @property
    def q_dim(self) -> int:
        return self.heads_q * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.heads_kv * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def num_params(self) -> int:
        per_layer = (self.qkv_dim * self.hidden + self.hidden * self.q_dim + 3 * self.ffn * self.hidden
                     + 2 * self.hidden + (self.qkv_dim if self.qkv_bias else 0))
        emb = self.vocab * self.hidden
        return self.num_layers * per_layer + emb * (1 if self.tie_embeddings else 2) + self.hidden

    def flops_per_token_linear(self) -> float:
        """Forward multiply-add FLOPs (x2) per token of every GEMM incl. the LM head."""
        per_layer = 2.0 * (self.qkv_dim * self.hidden + self.hidden * self.q_dim + 3 * self.ffn * self.hidden)
        return self.num_layers * per_layer + 2.0 * self.vocab * self.hidden

    @staticmethod
    def from_hf(cfg: dict, name: str = "hf") -> "ModelConfig":
        heads = cfg["num_attention_heads"]
        return ModelConfig(
            name=name, num_layers=cfg["num_hidden_layers"], hidden=cfg["hidden_size"], heads_q=heads,
            heads_kv=cfg.get("num_key_value_heads", heads),
            head_dim=cfg.get("head_dim") or cfg["hidden_size"] // heads,
            ffn=cfg["intermediate_size"], vocab=cfg["vocab_size"],
            rope_theta=float(cfg.get("rope_theta", 10000.0)), norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
            tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            # Qwen2ForCausalLM has biases on q/k/v only; Llama exposes the switch as attention_bias
            qkv_bias=bool(cfg.get("attention_bias", False)) or "Qwen2" in str(cfg.get("architectures", "")),
            max_position=int(cfg.get("max_position_embeddings", 131072)))

    @staticmethod
    def from_path(path: str) -> "ModelConfig":
        p = os.path.join(path, "config.json") if os.path.isdir(path) else path
        with open(p) as f:
            return ModelConfig.from_hf(json.load(f), name=os.path.basename(os.path.dirname(p)) or "hf")

    def with_layers(self, n: int | None) -> "ModelConfig":
        """Depth override (the reference's ``--num-layers`` / ``NUM_LAYERS``)."""
        if n is None:
            return self
        d = asdict(self)
        d["num_layers"] = n
        return ModelConfig(**d)


PRESETS: dict[str, ModelConfig] = {
    # CPU/gloo fp32 configuration: 2 layers, hidden 256, 4 q heads / 2 kv heads of 64, FFN 688
    "tiny": ModelConfig(name="tiny"),
    # same depth with head_dim 128 (the tcgen05 attention kernels are specialised for 128)
    "tiny-128": ModelConfig(name="tiny-128", num_layers=2, hidden=512, heads_q=4, heads_kv=2, head_dim=128,
                            ffn=1024, vocab=4096, rope_theta=10000.0),
    "small-128": ModelConfig(name="small-128", num_layers=4, hidden=1024, heads_q=8, heads_kv=2, head_dim=128,
                             ffn=2816, vocab=32000, rope_theta=500000.0),
    # Qwen2-shaped small model (QKV bias), the reference's second supported architecture
    "qwen2-tiny": ModelConfig(name="qwen2-tiny", num_layers=2, hidden=256, heads_q=4, heads_kv=2, head_dim=64,
                              ffn=688, vocab=32000, rope_theta=1000000.0, qkv_bias=True),
    # the head layout of the large models in small (8 KV heads: divisible by every tensor-parallel size of one box)
    "tiny-8kv": ModelConfig(name="tiny-8kv", num_layers=2, hidden=512, heads_q=16, heads_kv=8, head_dim=64,
                            ffn=1024, vocab=4096, rope_theta=500000.0),
    "llama3-8b": ModelConfig(name="llama3-8b", num_layers=32, hidden=4096, heads_q=32, heads_kv=8, head_dim=128,
                             ffn=14336, vocab=128256, rope_theta=500000.0, max_position=131072),
    "codellama-34b": ModelConfig(name="codellama-34b", num_layers=48, hidden=8192, heads_q=64, heads_kv=8,
                                 head_dim=128, ffn=22016, vocab=32000, rope_theta=1000000.0,
                                 max_position=262144),
}


def get_model_config(name_or_path: str, num_layers: int | None = None) -> ModelConfig:
    if name_or_path in PRESETS:
        cfg = PRESETS[name_or_path]
    elif os.path.exists(name_or_path):
        cfg = ModelConfig.from_path(name_or_path)
    else:
        low = name_or_path.lower()
        if "34b" in low:
            cfg = PRESETS["codellama-34b"]
        elif "8b" in low:
            cfg = PRESETS["llama3-8b"]
        else:
            raise ValueError(f"unknown model {name_or_path!r}; presets: {sorted(PRESETS)}")
    return cfg.with_layers(num_layers)


@dataclass
class ParallelConfig:
    """World layout. ``dp`` is the reference's ``--cp-size`` ("dpcp": ranks that hold different tokens
    of the global batch and serve each other's core attention); order of ranks is tp-fastest, then
    dp, then pp (the reference builds attention-server groups over dp x pp for each tp index,
    distca/runtime/megatron/create_group.py:43-67)."""
    tp: int = 1
    pp: int = 1
    dp: int = 1

    @property
    def world(self) -> int:
        return self.tp * self.pp * self.dp

    def coords(self, rank: int) -> tuple[int, int, int]:
        """rank -> (tp_rank, dp_rank, pp_rank)."""
        return rank % self.tp, (rank // self.tp) % self.dp, rank // (self.tp * self.dp)

    def rank_of(self, tp_rank: int, dp_rank: int, pp_rank: int) -> int:
        return tp_rank + self.tp * (dp_rank + self.dp * pp_rank)

    def describe(self) -> str:
        parts = [f"{k}{v}" for k, v in (("tp", self.tp), ("pp", self.pp), ("dp", self.dp)) if v > 1]
        return "-".join(parts) if parts else "single"


@dataclass
class TrainConfig:
    lr: float = 1e-5
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.01
    clip_grad: float = 1.0
    recompute: str = "full"        # none | full | keep_attn (recompute all but core attention)
    grad_dtype: str = "bf16"       # bf16 | fp32
    lm_head_chunk: int = 8192
    cad: bool = True
    pingpong: bool = True
    comm_buffer_gb: float = 2.0
    extra: dict = field(default_factory=dict)
