"""``PackedSeqParams`` with the public fields of Megatron-LM's dataclass of the same name."""
from dataclasses import dataclass
from typing import Any


@dataclass
class PackedSeqParams:
    qkv_format: str = None
    cu_seqlens_q: Any = None
    cu_seqlens_kv: Any = None
    cu_seqlens_q_padded: Any = None
    cu_seqlens_kv_padded: Any = None
    max_seqlen_q: Any = None
    max_seqlen_kv: Any = None
