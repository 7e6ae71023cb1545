"""patch_hf on a small random-init Llama of the installed transformers: while the sequence fits the local
window, InfLLM's attention is plain causal attention, so the patched model must reproduce the unpatched one's
logits; then a longer prompt runs through chunked prefill and greedy decoding."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _model():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, vocab_size=2000, rope_theta=1e6, max_position_embeddings=1 << 20,
                      attn_implementation="sdpa")
    return LlamaForCausalLM(cfg).to(DEV, torch.bfloat16).eval()


def test_patched_llama_matches_plain_attention_inside_the_window():
    from infllm_b200.utils import patch_hf

    model = _model()
    ids = torch.randint(0, 2000, (1, 300), generator=torch.Generator().manual_seed(1)).to(DEV)
    with torch.inference_mode():
        want = model(input_ids=ids, use_cache=False).logits.float()
        patch_hf(model, "inf-llm", n_local=512, n_init=128, topk=4, block_size=128, max_cached_block=8, exc_block_size=128,
                 fattn=True, repr_topk=4)
        got = model(input_ids=ids, use_cache=False).logits.float()
        # the same prompt in two pieces and then token by token: the memory carries over
        model.infllm_reset()
        a = model(input_ids=ids[:, :200], use_cache=False).logits.float()
        b = model(input_ids=ids[:, 200:299], use_cache=False).logits.float()
        c = model(input_ids=ids[:, 299:], use_cache=False).logits.float()
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= 0.05 * scale
    assert (torch.cat((a, b, c), dim=1) - want).abs().max().item() <= 0.05 * scale
    assert (got.argmax(-1) == want.argmax(-1)).float().mean().item() > 0.97


def test_chunked_prefill_and_greedy_decoding():
    from infllm_b200.utils import GreedySearch, patch_hf

    model = patch_hf(_model(), "inf-llm", n_local=512, n_init=128, topk=4, block_size=128, max_cached_block=8,
                     exc_block_size=128, fattn=True, repr_topk=4)
    ids = torch.randint(0, 2000, (1, 3000), generator=torch.Generator().manual_seed(2)).to(DEV)
    searcher = GreedySearch(model)
    one = searcher.generate(ids, max_length=8, chunk_size=1024)
    two = searcher.generate(ids, max_length=8, chunk_size=1024)
    assert len(one) == 8 and one == two  # deterministic, and clear() starts from scratch
    past = model.model.layers[0].self_attn._infllm_past
    assert past.size() == 3000 + 7 and past.num_global_block > 0
