"""A minimal Llama-shaped decoder over the attention-forward API, tensor-parallel by KV-head groups.

The reference patches a Hugging Face model and runs it on one GPU (inf_llm/utils/patch.py:33-172,
inf_llm/utils/greedy_search.py:35-105).  This module is the smallest caller of the same API that can be spread over
GPUs: every rank holds the query/key/value projection rows of its heads, the matching columns of the output
projection, and a column/row slice of the feed-forward matrices; the two partial sums of a layer (attention output,
feed-forward output) are all-reduced.  The context memories see only their rank's heads and share the retrieval
scores through a `HeadGroupComm` (infllm_b200/attention/head_groups.py), so all ranks retrieve the same units.

Weights are random (there are no checkpoints to load here): every matrix is drawn whole from a generator seeded by
(seed, layer, matrix) and then sliced, so a model split over N ranks has exactly the weights of the same model on one.
"""
import zlib

import torch

from ..attention import ATTN_FORWRAD, RotaryEmbeddingESM


def _rms_norm(x, weight, eps):
    v = x.float()
    v = v * torch.rsqrt(v.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (v * weight.float()).to(x.dtype)


class HeadGroupDecoder:
    """n_layers x (RMSNorm, context-memory attention, RMSNorm, SwiGLU feed-forward), final norm, LM head.

    `comm` is a HeadGroupComm when world > 1 (collective construction), `group` the torch.distributed group of the
    all-reduces.  `attn_kwargs` are the keyword arguments of ATTN_FORWRAD["inf-llm"] (n_local, n_init, topk, ...)."""

    def __init__(self, n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, attn_kwargs, rank=0, world=1,
                 comm=None, group=None, seed=0, dtype=torch.bfloat16, device=None, rope_base=500000.0, eps=1e-5,
                 init_std=0.02):
        assert n_heads % world == 0 and n_kv_heads % world == 0 and ffn % world == 0
        assert world == 1 or comm is not None
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.n_layers, self.hidden, self.head_dim, self.vocab, self.eps = n_layers, hidden, head_dim, vocab, eps
        self.heads, self.kv_heads = n_heads // world, n_kv_heads // world
        self.rank, self.world, self.group, self.dtype = rank, world, group, dtype
        self.rope = RotaryEmbeddingESM(head_dim, rope_base, 1.0)
        kwargs = dict(attn_kwargs)
        if world > 1:
            kwargs["head_group_comm"] = comm
        self.forward = ATTN_FORWRAD["inf-llm"](**kwargs)

        def draw(rows, cols, *key):  # the whole matrix, the same on every rank
            g = torch.Generator(device=self.device).manual_seed(zlib.crc32(repr((seed,) + key).encode()))
            return (torch.randn((rows, cols), generator=g, device=self.device, dtype=torch.float32) * init_std).to(dtype)

        nq, nk, nf = self.heads * head_dim, self.kv_heads * head_dim, ffn // world
        self.embed = draw(vocab, hidden, "embed")
        self.lm_head = draw(vocab, hidden, "lm_head")
        self.final_norm = torch.ones(hidden, dtype=dtype, device=self.device)
        self.layers = []
        for i in range(n_layers):
            wq, wk, wv = draw(n_heads * head_dim, hidden, i, "q"), draw(n_kv_heads * head_dim, hidden, i, "k"), \
                draw(n_kv_heads * head_dim, hidden, i, "v")
            wo = draw(hidden, n_heads * head_dim, i, "o")
            gate, up, down = draw(ffn, hidden, i, "gate"), draw(ffn, hidden, i, "up"), draw(hidden, ffn, i, "down")
            self.layers.append(dict(
                wq=wq[rank * nq:(rank + 1) * nq].contiguous(), wk=wk[rank * nk:(rank + 1) * nk].contiguous(),
                wv=wv[rank * nk:(rank + 1) * nk].contiguous(), wo=wo[:, rank * nq:(rank + 1) * nq].contiguous(),
                gate=gate[rank * nf:(rank + 1) * nf].contiguous(), up=up[rank * nf:(rank + 1) * nf].contiguous(),
                down=down[:, rank * nf:(rank + 1) * nf].contiguous(),
                norm1=torch.ones(hidden, dtype=dtype, device=self.device),
                norm2=torch.ones(hidden, dtype=dtype, device=self.device), past=None))
            del wq, wk, wv, wo, gate, up, down

    def _sum(self, x):
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(x, group=self.group)
        return x

    def reset(self):
        for layer in self.layers:
            if layer["past"] is not None:
                layer["past"].reset()

    @torch.inference_mode()
    def step(self, ids):
        """ids (1, L) -> logits (1, vocab) of the last position; the context memories advance by L tokens."""
        lin = torch.nn.functional.linear
        h = self.embed[ids]
        for layer in self.layers:
            x = _rms_norm(h, layer["norm1"], self.eps)
            o, layer["past"] = self.forward(
                None, x, x, self.rope, True, layer["past"], lambda t: lin(t, layer["wq"]), lambda t: lin(t, layer["wk"]),
                lambda t: lin(t, layer["wv"]), lambda t: self._sum(lin(t, layer["wo"])), self.head_dim, self.heads,
                self.kv_heads)
            h = h + o
            x = _rms_norm(h, layer["norm2"], self.eps)
            h = h + self._sum(lin(torch.nn.functional.silu(lin(x, layer["gate"])) * lin(x, layer["up"]), layer["down"]))
        last = _rms_norm(h[:, -1], self.final_norm, self.eps)
        return lin(last, self.lm_head).float()

    @torch.inference_mode()
    def generate(self, input_ids, max_length=64, chunk_size=8192):
        """Chunked prefill of input_ids (1, L), then greedy decoding.  Returns (generated ids, logits of every
        generated position (max_length, vocab))."""
        self.reset()
        logits = None
        for st in range(0, input_ids.size(1), chunk_size):
            logits = self.step(input_ids[:, st:st + chunk_size])
        out, trail = [], []
        for i in range(max_length):
            trail.append(logits[0].clone())
            nxt = logits.argmax(dim=-1)
            out.append(int(nxt))
            if i == max_length - 1:
                break
            logits = self.step(nxt[:, None])
        return out, torch.stack(trail)
