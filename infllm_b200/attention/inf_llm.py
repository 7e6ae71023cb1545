"""inf_llm_forward with the signature of the reference (inf_llm/attention/inf_llm.py:5-80)."""
from typing import Optional

import torch

from .context_manager import ContextManager


def inf_llm_forward(n_local, n_init, topk, block_size, max_cached_block, exc_block_size, fattn,
                    repr_topk: int = 1, cache_strategy="lru", score_decay=None, chunk_topk_calc=None,
                    async_global_stream=True, pin_memory=False, faiss=False, perhead=False, *args,
                    head_group_comm=None, device_store_mb=0, **kwargs):
    """Returns forward(self, query, key_value, position_bias, use_cache, past_key_value, project_q,
    project_k, project_v, attention_out, dim_head, num_heads, num_heads_kv) -> (o, past_key_value).
    Unknown keyword arguments are swallowed like in the reference (inf_llm.py:17).  `head_group_comm` (a
    HeadGroupComm, not in the reference) says that the projections and head counts passed to forward() are this
    rank's slice of a KV-head-group sharding; the caller sums the ranks' attention_out results.  `device_store_mb`
    (not in the reference): see ContextManager."""

    def forward(self, query: torch.Tensor, key_value: torch.Tensor, position_bias: Optional[torch.Tensor],
                use_cache: bool, past_key_value, project_q, project_k, project_v, attention_out, dim_head,
                num_heads, num_heads_kv):
        batch_size, len_q, len_k = query.size(0), query.size(1), key_value.size(1)
        assert use_cache  # inf_llm.py:33
        # head-major views of the projections; the kernels take strides, so nothing is copied here
        h_q = project_q(query).view(batch_size, len_q, num_heads, dim_head).permute(0, 2, 1, 3)
        h_k = project_k(key_value).view(batch_size, len_k, num_heads_kv, dim_head).permute(0, 2, 1, 3)
        h_v = project_v(key_value).view(batch_size, len_k, num_heads_kv, dim_head).permute(0, 2, 1, 3)
        if past_key_value is None:  # inf_llm.py:45-58
            past_key_value = ContextManager(
                position_bias, n_init, n_local, block_size, max_cached_block, topk, exc_block_size, score_decay,
                fattn, repr_topk, cache_strategy, chunk_topk_calc, async_global_stream, pin_memory, faiss, perhead,
                head_group_comm=head_group_comm, device_store_mb=device_store_mb)
        o = past_key_value.append(h_q, h_k, h_v, h_q, h_k, h_v)
        o = o.view(batch_size, num_heads, len_q, dim_head).permute(0, 2, 1, 3)
        o = o.reshape(batch_size, len_q, dim_head * num_heads)
        o = attention_out(o)
        if use_cache:
            return o, past_key_value
        return o

    return forward
