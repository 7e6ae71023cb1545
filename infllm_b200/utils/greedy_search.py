"""Chunked prefill + greedy decoding over a patched model (the job of inf_llm/utils/greedy_search.py:35-105):
the prompt is fed in chunks of `chunk_size` tokens so that activations stay bounded, the attention modules keep
the context memory, and only the last position's logits are ever materialised."""
import torch


class GreedySearch:
    def __init__(self, model, tokenizer=None):
        self.model, self.tokenizer = model, tokenizer
        model.eval()

    def clear(self):
        self.model.infllm_reset()

    @torch.inference_mode()
    def _step(self, ids):
        out = self.model(input_ids=ids, use_cache=False, logits_to_keep=1)
        return out.logits[:, -1]

    @torch.inference_mode()
    def generate(self, input_ids, max_length=64, chunk_size=8192, eos_token_id=None):
        """input_ids (1, L) -> list of generated token ids (at most max_length)."""
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        self.clear()
        logits = None
        for st in range(0, input_ids.size(1), chunk_size):
            logits = self._step(input_ids[:, st:st + chunk_size])
        generated = []
        for i in range(max_length):
            nxt = logits.argmax(dim=-1)
            generated.append(int(nxt))
            if (eos_token_id is not None and generated[-1] == eos_token_id) or i == max_length - 1:
                break
            logits = self._step(nxt[:, None])
        return generated
