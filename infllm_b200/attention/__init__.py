"""Attention-forward registry with the reference's names (inf_llm/attention/__init__.py:8-13;
the misspelt ATTN_FORWRAD is the reference's public name)."""
from .context_manager import ContextManager, device_store_info, device_store_release, device_store_reserve
from .dot_production_attention import CudaMultiStageDotProductionAttention, get_multi_stage_dot_production_attention
from .head_groups import HeadGroupComm
from .inf_llm import inf_llm_forward
from .rope import RotaryEmbeddingESM
from .sink_window import infinite_lm_forward, stream_llm_forward
from .sharded_decode import PeerMailbox, ShardedDecodeMemory, UnitRangeShard, global_topk, unit_range

ATTN_FORWRAD = {
    "inf-llm": inf_llm_forward,
    "infinite-lm": infinite_lm_forward,
    "stream-llm": stream_llm_forward,
}
ATTN_FORWARD = ATTN_FORWRAD

__all__ = ["RotaryEmbeddingESM", "ATTN_FORWRAD", "ATTN_FORWARD", "ContextManager", "inf_llm_forward", "infinite_lm_forward", "stream_llm_forward",
           "CudaMultiStageDotProductionAttention", "get_multi_stage_dot_production_attention",
           "HeadGroupComm", "device_store_reserve", "device_store_release", "device_store_info", "PeerMailbox", "ShardedDecodeMemory", "UnitRangeShard", "global_topk", "unit_range"]
