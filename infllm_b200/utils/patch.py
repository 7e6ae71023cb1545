"""patch_hf for current transformers (5.x): put an ATTN_FORWRAD attention type behind the self-attention modules
of a Hugging Face Llama / Mistral / Qwen2 causal LM.

The reference's patch (inf_llm/utils/patch.py:33-172) replaces the attention module's forward and the decoder's
forward of transformers 4.3x, whose signatures no longer exist.  Here only the attention modules are touched:
their forward keeps the 5.x signature `(hidden_states, position_embeddings, attention_mask, past_key_values,
**kwargs) -> (output, None)`, ignores the rotary tables and the mask it is handed (the attention types rotate
and mask themselves) and keeps its own per-layer cache object — the `past_key_value` of the reference's forward —
on the module.  `model.infllm_reset()` starts a new sequence.  Call the model with `use_cache=False`: the cache
that matters is the one on the attention modules, and transformers' own KV cache would only duplicate the keys.
"""
import types

from ..attention import ATTN_FORWRAD, RotaryEmbeddingESM


def _attention_modules(model):
    decoder = getattr(model, "model", model)
    layers = getattr(decoder, "layers", None)
    if layers is None or not hasattr(layers[0], "self_attn"):
        raise ValueError("patch_hf supports decoder-only models with model.layers[i].self_attn (llama, mistral, qwen2)")
    return [layer.self_attn for layer in layers]


def patch_hf(model, attn_type: str = "inf-llm", attn_kwargs: dict = None, base=None, distance_scale=None, **kwargs):
    """Same arguments as the reference's patch_hf (patch.py:33-40).  `attn_type` is a key of ATTN_FORWRAD
    ("inf-llm", "infinite-lm", "stream-llm"; the reference's yaml files spell the first one "inf_llm" too)."""
    attn_kwargs = dict(attn_kwargs or {})
    attn_kwargs.update(kwargs)
    attn_type = {"inf_llm": "inf-llm", "infinite_lm": "infinite-lm", "stream_llm": "stream-llm"}.get(attn_type, attn_type)
    forward = ATTN_FORWRAD[attn_type](**attn_kwargs)
    cfg = model.config
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    if base is None:
        rp = getattr(cfg, "rope_parameters", None) or {}
        base = rp.get("rope_theta") or getattr(cfg, "rope_theta", None) or 10000.0
    rope = RotaryEmbeddingESM(head_dim, base, 1.0 if distance_scale is None else distance_scale)
    modules = _attention_modules(model)

    def attention_forward(self, hidden_states, position_embeddings=None, attention_mask=None, past_key_values=None,
                          **_):
        o, self._infllm_past = forward(self, hidden_states, hidden_states, rope, True, self._infllm_past, self.q_proj,
                                       self.k_proj, self.v_proj, self.o_proj, head_dim, cfg.num_attention_heads,
                                       cfg.num_key_value_heads)
        return o, None

    for m in modules:
        m._infllm_past = None
        m._old_forward = m.forward
        m.forward = types.MethodType(attention_forward, m)

    def infllm_reset():
        for m in modules:
            m._infllm_past = None

    model.infllm_reset = infllm_reset
    model.position_bias = rope
    return model
