"""Stand-in package so that the reference's pure-Python planner and metadata modules import without
Megatron-LM (absent offline). Only ``megatron.core.packed_seq_params.PackedSeqParams`` is provided: a
plain dataclass with the fields the reference reads (distca/runtime/compute_metadata.py:5, 326-365).
Used by the differential planner tests and by the reference arm of the dispatch micro-benchmark; never
on this framework's own path."""
