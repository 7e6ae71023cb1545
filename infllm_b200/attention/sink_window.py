"""The reference's two sink + window attention types on the CUDA kernels: "infinite-lm" (LM-Infinite,
inf_llm/attention/infinite_lm.py:6-100) and "stream-llm" (StreamingLLM, inf_llm/attention/stream_llm.py:6-111).

Both keep the first n_init tokens (the sink) and the last n_local tokens (the window).  A query attends to its
window with window-relative rotary positions, and to the sink tokens that have left its window with all queries at
one fixed position; the two parts are normalised jointly by the multi-stage attention (a window-masked stage and a
stage with the complement mask — the one caller of the boundary that uses a complement mask that actually hides
pairs).  They differ in the positions of the sink stage:

    infinite-lm   sink keys un-rotated, queries at position n_local - 1
    stream-llm    sink keys at positions 0..n_init-1, queries at position n_local + n_init - 1

Same factory and forward signatures as the reference; the cache object returned as past_key_value is the
reference's tuple (K of [sink | window], V, tokens seen).
"""
import torch

from .dot_production_attention import get_multi_stage_dot_production_attention


def _sink_window_forward(n_local, n_init, fattn, stream_positions):
    Attn, _ = get_multi_stage_dot_production_attention(fattn)

    def forward(self, query, key_value, position_bias, use_cache, past_key_value, project_q, project_k, project_v,
                attention_out, dim_head, num_heads, num_heads_kv):
        batch, len_q, len_new = query.size(0), query.size(1), key_value.size(1)

        def heads(x, n, length):  # (B, L, n*D) -> (B, n, L, D)
            return x.view(batch, length, n, dim_head).permute(0, 2, 1, 3).contiguous()

        q = heads(project_q(query), num_heads, len_q)
        k = heads(project_k(key_value), num_heads_kv, len_new)
        v = heads(project_v(key_value), num_heads_kv, len_new)
        seen = len_new
        if past_key_value is not None:
            k = torch.cat((past_key_value[0], k), dim=-2)
            v = torch.cat((past_key_value[1], v), dim=-2)
            seen += past_key_value[2]
        cache = None
        if use_cache:  # everything while the history is short, then [first n_init | last n_local]
            if seen <= n_local + n_init:
                cache = (k, v, seen)
            else:
                tail = max(0, k.size(-2) - n_local)
                cache = (torch.cat((k[:, :, :n_init], k[:, :, tail:]), dim=2),
                         torch.cat((v[:, :, :n_init], v[:, :, tail:]), dim=2), seen)
        # window stage over the last len_q + n_local keys
        wk, wv = k, v
        if len_q + n_local < k.size(-2):
            cut = k.size(-2) - len_q - n_local
            wk, wv = k[:, :, cut:].contiguous(), v[:, :, cut:].contiguous()
        wq, wk = position_bias(q, wk)
        # sink stage: only once some token has left the window
        if seen > n_local:
            sk, sv = k[:, :, :n_init].contiguous(), v[:, :, :n_init].contiguous()
            if stream_positions:
                sq = position_bias.apply_rotary_pos_emb_one_angle(q, n_local + n_init)
                sk = position_bias.apply_rotary_pos_emb(sk, sk.size(-2), sk.size(-2), None, None)
            else:
                sq = position_bias.apply_rotary_pos_emb_one_angle(q, n_local)
        else:
            sq = q
            sk = torch.empty((batch, num_heads_kv, 0, dim_head), device=k.device, dtype=k.dtype)
            sv = torch.empty_like(sk)
        attn = Attn(wq.shape, wq.dtype, wq.device)
        attn.append(wq, wk, wv, sliding_window=n_local)
        attn.append(sq, sk, sv, end=True, sliding_window=(seen - len_q, n_local), complement_sliding_window=True)
        o, _ = attn.get_result()
        o = o.view(batch, num_heads, len_q, dim_head).permute(0, 2, 1, 3).reshape(batch, len_q, num_heads * dim_head)
        o = attention_out(o)
        return (o, cache) if use_cache else o

    return forward


def infinite_lm_forward(n_local, n_init, fattn: bool = False, *args, **kwargs):
    """ATTN_FORWRAD["infinite-lm"] (inf_llm/attention/infinite_lm.py:6)."""
    return _sink_window_forward(n_local, n_init, fattn, stream_positions=False)


def stream_llm_forward(n_local, n_init, fattn: bool = False, *args, **kwargs):
    """ATTN_FORWRAD["stream-llm"] (inf_llm/attention/stream_llm.py:6)."""
    return _sink_window_forward(n_local, n_init, fattn, stream_positions=True)
