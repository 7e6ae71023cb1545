"""CPU oracle (test infrastructure) for the reference's sink + window attention types.

Restates inf_llm/attention/infinite_lm.py:6-100 ("infinite-lm", LM-Infinite) and
inf_llm/attention/stream_llm.py:6-111 ("stream-llm", StreamingLLM) in fp32 torch ops, on top of the RoPE and
multi-stage attention functions of infllm_oracle.py.  Both keep the first n_init tokens (the sink) and the last
n_local tokens (the window); a query attends to its window with window-relative rotary positions and to the sink
tokens that have left its window with every query at one fixed position:

    infinite-lm   sink keys un-rotated, queries at position n_local - 1            (infinite_lm.py:64-71)
    stream-llm    sink keys at positions 0..n_init-1, queries at n_local + n_init - 1   (stream_llm.py:68-76)

Pinned against recordings of the reference itself (tests/golden/sink_window.npz, written by
tests/golden/make_golden.py).  Only tests import this file.
"""
from dataclasses import dataclass, field
from typing import Optional

import torch

from .infllm_oracle import Stage, multi_stage_attention, rope_apply, rope_cos_sin, rope_local, rope_one_angle


@dataclass
class SinkWindowMemory:
    """What survives between calls: K/V of [sink | window] (one contiguous history while it is short) and the
    number of tokens seen (the reference's cache tuple, infinite_lm.py:41-50)."""

    n_local: int
    n_init: int
    dim: int
    base: float
    kind: str  # "infinite-lm" | "stream-llm"
    k: Optional[torch.Tensor] = None  # (H_kv, n, D)
    v: Optional[torch.Tensor] = None
    length: int = 0
    outputs: list = field(default_factory=list)

    def append(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """q (H, L, D), k and v (H_kv, L, D) of L new tokens -> attention output (H, L, D)."""
        lq = q.size(-2)
        if self.k is not None:
            k, v = torch.cat((self.k, k), dim=-2), torch.cat((self.v, v), dim=-2)
        total = self.length + lq
        # the cache for the next call: everything while short, else first n_init + last n_local  (:41-48)
        if total <= self.n_local + self.n_init:
            self.k, self.v = k, v
        else:
            keep = max(0, k.size(-2) - self.n_local)
            self.k = torch.cat((k[:, : self.n_init], k[:, keep:]), dim=-2)
            self.v = torch.cat((v[:, : self.n_init], v[:, keep:]), dim=-2)
        self.length = total
        # window stage: the last lq + n_local keys, window-relative rotation, window mask  (:55-62, :83)
        lk, lv = k, v
        if lq + self.n_local < k.size(-2):
            lk, lv = k[:, k.size(-2) - lq - self.n_local:], v[:, v.size(-2) - lq - self.n_local:]
        rq, rk = rope_local(q, lk, self.dim, self.base, 1.0)
        stages = [Stage(rq, rk, lv, sliding_window=self.n_local)]
        # sink stage: the tokens that left the window, complement mask  (:64-85)
        if total > self.n_local:
            sink_k, sink_v = k[:, : self.n_init], v[:, : self.n_init]
            if self.kind == "infinite-lm":
                sq = rope_one_angle(q, self.n_local, self.dim, self.base, 1.0)
            else:
                sq = rope_one_angle(q, self.n_local + self.n_init, self.dim, self.base, 1.0)
                cos, sin = rope_cos_sin(self.dim, self.base, 1.0, self.n_init)
                n = sink_k.size(-2)
                sink_k = rope_apply(sink_k, cos[:n], sin[:n])
        else:
            sq, sink_k, sink_v = q, k[:, :0], v[:, :0]
        stages.append(Stage(sq, sink_k, sink_v, sliding_window=(total - lq, self.n_local), complement=True))
        out, _ = multi_stage_attention(stages)
        return out
