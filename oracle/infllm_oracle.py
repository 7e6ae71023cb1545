"""CPU oracle for InfLLM's per-layer context-memory attention.  TEST INFRASTRUCTURE.

This file restates, on the host in fp32 torch ops, the algorithm of the reference's
context-memory attention path so that the CUDA path can be checked against it.  It
is not part of the product: only tests/, __graft_entry__.smoke() and the
cpu_baseline / --impl reference legs of bench.py may import it.

Parity pin: the reference has no tests or golden vectors of its own.  The oracle is
pinned against outputs of the reference itself (imported from its checkout through
tests/golden/ref_shim.py, which only rewrites device literals) on seeded inputs;
the recorded vectors live in tests/golden/*.npz and tests/test_oracle_golden.py
replays them.

Each function cites the reference file:line it follows (paths relative to the
reference repository root).  The restatement keeps the reference's arithmetic but
not its data structures: tokens live in one absolute-indexed log, and the cursors
of the reference (local window, remainder, init sink, sealed blocks) are integers
over that log.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- RoPE
def rope_inv_freq(dim: int, base: float) -> torch.Tensor:
    """inf_llm/attention/rope.py:22-24 — fp32 inverse frequencies."""
    return 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))


def rope_cos_sin(dim: int, base: float, scale: float, length: int):
    """inf_llm/attention/rope.py:49-65 — fp32 tables, angle = (t*scale) * inv_freq, duplicated halves."""
    t = torch.arange(length).to(torch.float32)
    freqs = torch.outer(t * scale, rope_inv_freq(dim, base))
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    """inf_llm/attention/rope.py:31-33."""
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat((-x2, x1), dim=-1)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """inf_llm/attention/rope.py:35-47 — fp32 math, cast back to x's dtype.
    x: (..., L, D); cos/sin: (L, D) or (1, D)."""
    return ((x.float() * cos) + (_rotate_half(x).float() * sin)).to(x.dtype)


def rope_local(q, k, dim, base, scale):
    """inf_llm/attention/rope.py:107-112 — window-relative positions: keys 0..Lk-1, queries Lk-Lq..Lk-1."""
    lq, lk = q.size(-2), k.size(-2)
    cos, sin = rope_cos_sin(dim, base, scale, lk)
    return rope_apply(q, cos[lk - lq : lk], sin[lk - lq : lk]), rope_apply(k, cos, sin)


def rope_one_angle(x, index, dim, base, scale):
    """inf_llm/attention/rope.py:89-104 — every row rotated to the single position index-1."""
    cos, sin = rope_cos_sin(dim, base, scale, index)
    return rope_apply(x, cos[index - 1 : index], sin[index - 1 : index])


# ------------------------------------------------------- multi-stage attention
@dataclass
class Stage:
    """One append() of the reference's multi-stage attention
    (inf_llm/attention/dot_production_attention/base.py:18-26)."""

    q: torch.Tensor  # (H, Lq, D)
    k: torch.Tensor  # (H_kv, Lk, D)
    v: torch.Tensor  # (H_kv, Lk, D)
    sliding_window: Optional[object] = None  # None | int | (offset, size)
    complement: bool = False
    get_score: bool = False


def stage_mask(lq: int, lk: int, sliding_window, complement: bool) -> torch.Tensor:
    """inf_llm/attention/dot_production_attention/torch_impl.py:60-78."""
    if sliding_window is None:
        return torch.ones((lq, lk), dtype=torch.bool)
    if isinstance(sliding_window, int):
        sliding_window = (lk - lq, sliding_window)
    off, size = sliding_window
    dist = torch.arange(lq)[:, None] - torch.arange(lk)[None, :] + off
    if complement:
        return dist >= size
    return (dist < size) & (dist >= 0)


def multi_stage_attention(stages: Sequence[Stage]):
    """Jointly normalised attention over several (q, k, v, mask) stages.

    inf_llm/attention/dot_production_attention/torch_impl.py:15-36 (finalize) and :39-96
    (append): logits per stage, masked with -inf, scaled by 1/sqrt(D), concatenated over
    stages, ONE softmax, then per stage the masked probabilities give the per-key score
    (sum over queries) and p @ v is accumulated into the result.
    Returns (out (H, Lq, D) in q dtype, [score (H, Lk_stage) or None per stage]).
    """
    logits, masks = [], []
    h = stages[0].q.size(0)
    for s in stages:
        g = h // s.k.size(0)
        k = s.k.repeat_interleave(g, dim=0) if g > 1 else s.k
        m = stage_mask(s.q.size(-2), s.k.size(-2), s.sliding_window, s.complement)
        lg = torch.matmul(s.q, k.transpose(-1, -2))
        lg = lg.masked_fill(~m[None], float("-inf"))
        lg = lg * (1.0 / math.sqrt(s.q.size(-1)))
        logits.append(lg)
        masks.append(m)
    p = torch.softmax(torch.cat(logits, dim=-1), dim=-1)
    out = torch.zeros_like(stages[0].q)
    scores, st = [], 0
    for s, m in zip(stages, masks):
        lk = s.k.size(-2)
        ps = p[:, :, st : st + lk].masked_fill(~m[None], 0)
        g = h // s.v.size(0)
        v = s.v.repeat_interleave(g, dim=0) if g > 1 else s.v
        scores.append(ps.sum(dim=-2) if s.get_score else None)
        out += torch.matmul(ps, v)
        st += lk
    return out, scores


# ----------------------------------------------------------------- LRU bookkeeping
class LruTable:
    """The per-unit `cached_blocks` dict of the reference: block id -> stamp, iteration in
    insertion order (a Python dict), which decides ties at eviction.
    inf_llm/attention/context_manager.py:246-265 (eviction), :495-515 (stamping)."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.entries: dict = {}

    def plan(self, wanted: Sequence[int]) -> List[int]:
        """Evict what the reference evicts before loading `wanted`; returns evicted ids in order.
        context_manager.py:496-502 then :253-265: num_remove = len - capacity + misses;
        candidates in ascending stamp order (stable over insertion order); `wanted` is protected."""
        num_remove = len(self.entries) - self.capacity
        for b in wanted:
            if b not in self.entries:
                num_remove += 1
        evicted: List[int] = []
        if num_remove <= 0:
            return evicted
        order = sorted(self.entries.items(), key=lambda kv: kv[1])
        for bid, _ in order:
            if bid not in wanted:
                del self.entries[bid]
                evicted.append(bid)
            if len(evicted) >= num_remove:
                break
        return evicted

    def stamp(self, wanted: Sequence[int], value) -> None:
        """context_manager.py:504-513 — written in the raw (descending score) top-k order."""
        for b in wanted:
            self.entries[b] = value


# ------------------------------------------------------------- the context memory
@dataclass
class ExecBlockTrace:
    """What one execution block did; the quantities the CUDA path is compared on."""

    q_start: int  # absolute index of the block's first query token
    q_end: int
    topk_raw: List[int]  # retrieval result in the order the scorer returned it
    n_blocks_visible: int  # sealed blocks that existed when this exec block ran
    init_len: int
    overflow_len: int
    evicted: List[int]
    cached_after: List[Tuple[int, float]]  # LRU table items in dict order
    block_scores: Optional[torch.Tensor] = None  # fp32 (n_blocks,) or None when not scored


class OracleContextMemory:
    """One batch element (one `unit`) of the reference's ContextManager
    (inf_llm/attention/context_manager.py:196-816) for cache_strategy "lru" / "lru-s",
    fattn=False, faiss=False, perhead=False, with or without chunk_topk_calc.

    A batch of B sequences is B independent instances: the reference shares only the cursor
    arithmetic between units, and that depends on lengths alone."""

    def __init__(self, n_init, n_local, block_size, max_cached_block, topk, exc_block_size,
                 repr_topk=1, rope_base=10000.0, rope_scale=1.0, cache_strategy="lru",
                 score_decay=None, keep_scores=False, chunk_topk_calc=None):
        assert exc_block_size <= n_local  # context_manager.py:219
        assert cache_strategy in ("lru", "lru-s")  # :238
        self.n_init, self.n_local, self.bs = n_init, n_local, block_size
        self.max_cached, self.topk, self.exc = max_cached_block, topk, exc_block_size
        self.repr_topk, self.base, self.scale = repr_topk, rope_base, rope_scale
        self.strategy, self.decay = cache_strategy, score_decay
        self.keep_scores = keep_scores
        # chunk_topk_calc (:749-757, 548-610): a call of more than one token is cut into chunks of this many tokens
        # and every exec block of a chunk is ranked when the chunk starts, i.e. over the units sealed by then
        self.chunk_topk_calc = chunk_topk_calc
        self._unit_limit: Optional[int] = None
        self.length = 0  # tokens consumed (context_manager.py:211, :793)
        self.k_log: Optional[torch.Tensor] = None  # (H_kv, T, D) un-rotated keys of every token
        self.v_log: Optional[torch.Tensor] = None
        self.acc: Optional[torch.Tensor] = None  # (H, T) accumulated local attention mass (S5)
        self.init_len = 0  # tokens [0, init_len) form the attention sink
        self.init_full = False
        self.block_k: List[torch.Tensor] = []  # representative key row (H*D,) per sealed block
        self.frontier = 0  # first token not yet moved to the sink or sealed
        self.lru = LruTable(max_cached_block)
        self.load_count = 0
        self.resident: set = set()  # which blocks hold a cache slot (must mirror lru.entries)
        self.trace: List[ExecBlockTrace] = []

    # -- helpers
    @property
    def num_blocks(self) -> int:
        return len(self.block_k)

    def _block_range(self, b: int) -> Tuple[int, int]:
        st = self.n_init + b * self.bs
        return st, st + self.bs

    def _retrieve(self, gq: torch.Tensor):
        """context_manager.py:366-383 and VectorTensor.get_topk :159-163."""
        n = self.num_blocks if self._unit_limit is None else self._unit_limit  # :553-559 for a chunk
        if n <= self.topk:
            return list(range(n)), None
        qbar = gq.mean(dim=1).reshape(-1)  # (H*D,)
        scores = torch.matmul(torch.stack(self.block_k[:n]), qbar[:, None]).squeeze(-1)
        return scores.topk(self.topk, dim=0).indices.tolist(), scores

    def _seal(self, end: int) -> None:
        """context_manager.py:614-679 after one exec block that ended at absolute token `end`."""
        rem = end - self.frontier
        if not self.init_full and rem > self.n_local:  # :628-646
            take = min(self.n_init - self.init_len, rem - self.n_local)
            self.init_len += take
            self.frontier += take
            rem -= take
            if self.init_len == self.n_init:
                self.init_full = True
        h = self.acc.size(0)
        g = h // self.k_log.size(0)
        while rem - self.bs >= self.n_local:  # :649-676
            rem -= self.bs
            st = self.frontier
            kblk = self.k_log[:, st : st + self.bs]  # (H_kv, bs, D)
            kblk = kblk.repeat_interleave(g, dim=0) if g > 1 else kblk  # :280-289
            idx = self.acc[:, st : st + self.bs].topk(self.repr_topk, dim=-1).indices  # :274
            rep = torch.gather(kblk, 1, idx[:, :, None].expand(h, self.repr_topk, kblk.size(-1)))
            self.block_k.append(rep.mean(dim=1).reshape(-1))  # :669-670
            self.frontier += self.bs

    # -- the path
    def append(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """context_manager.py:682-813.  q (H, L, D); k, v (H_kv, L, D), un-rotated; returns (H, L, D).
        The reference passes the same tensors as the local and the global inputs
        (inf_llm/attention/inf_llm.py:61-67)."""
        h, L, d = q.shape
        if self.k_log is None:
            self.k_log, self.v_log = k.clone(), v.clone()
            self.acc = torch.zeros((h, L), dtype=k.dtype)
        else:
            self.k_log = torch.cat((self.k_log, k), dim=1)
            self.v_log = torch.cat((self.v_log, v), dim=1)
            self.acc = torch.cat((self.acc, torch.zeros((h, L), dtype=k.dtype)), dim=1)
        t0 = self.length
        rem_start = self.frontier  # first token of the reference's remainder tensor in this call
        rem_total = t0 + L - rem_start  # its length after the cat at :728-731
        gq_all = rope_one_angle(q, self.n_local, d, self.base, self.scale)  # :744-747
        outs = []
        chunk = None
        if self.chunk_topk_calc is not None and L > 1:  # :749-757
            chunk = (self.chunk_topk_calc // self.exc) * self.exc
        self._unit_limit = None
        for st in range(0, L, self.exc):  # :762
            ed = min(st + self.exc, L)
            if chunk is not None and st % chunk == 0:
                self._unit_limit = self.num_blocks  # :764-770: ranked now for the whole chunk
            s_abs, e_abs = t0 + st, t0 + ed
            ks = max(s_abs - self.n_local, 0)  # :772-773 in absolute token indices
            lq, lk = rope_local(q[:, st:ed], self.k_log[:, ks:e_abs], d, self.base, self.scale)  # :480
            local = Stage(lq, lk, self.v_log[:, ks:e_abs], sliding_window=self.n_local, get_score=True)

            gq = gq_all[:, st:ed]
            topk_raw, scores = self._retrieve(gq)  # :493
            evicted = self.lru.plan(topk_raw)  # :495-502
            for b in evicted:
                self.resident.discard(b)
            if self.strategy == "lru":  # :504-513
                self.load_count += 1
                self.lru.stamp(topk_raw, self.load_count)
            else:
                self.lru.stamp(topk_raw, 0)
            for b in topk_raw:  # MemoryUnit.load -> CudaCache.alloc (:76, :18-22)
                if b not in self.resident:
                    assert len(self.resident) < self.max_cached, "cache slots exhausted (context_manager.py:19)"
                    self.resident.add(b)

            # gathered global keys: [retrieved blocks | init sink | overflow]  (:386-451)
            blocks = sorted(topk_raw)  # :402; attention is order independent
            ovf = max(e_abs - self.frontier - self.n_local, 0)  # :391
            segs = [self._block_range(b) for b in blocks]
            segs.append((0, self.init_len))
            segs.append((self.frontier, self.frontier + ovf))
            gk = torch.cat([self.k_log[:, a:b] for a, b in segs], dim=1)
            gv = torch.cat([self.v_log[:, a:b] for a, b in segs], dim=1)
            rmd_st = len(blocks) * self.bs + self.init_len
            glob = Stage(gq, gk, gv, sliding_window=(rem_total + rmd_st, self.n_local),  # :437
                         complement=True, get_score=self.strategy == "lru-s")
            o, sc = multi_stage_attention([local, glob])  # :486-533
            outs.append(o)

            if self.strategy == "lru-s" and sc[1] is not None:  # :454-470
                per_block = sc[1][:, : len(blocks) * self.bs].reshape(h, len(blocks), self.bs).sum(-1).sum(0)
                for b in list(self.lru.entries):
                    self.lru.entries[b] = self.lru.entries[b] * self.decay
                # the reference pairs the scores with its buffer slot order; the per-block sums are
                # the same set of (block, score) pairs, so pairing by sorted id is equivalent.
                for b, sval in zip(blocks, per_block.tolist()):
                    self.lru.entries[b] += sval

            self.acc[:, ks:e_abs] += sc[0]  # :623-625
            self.trace.append(ExecBlockTrace(
                s_abs, e_abs, list(topk_raw), self.num_blocks, self.init_len, ovf, evicted,
                list(self.lru.entries.items()),
                scores.clone() if (scores is not None and self.keep_scores) else None))
            self._seal(e_abs)  # :784-785
        self._unit_limit = None
        self.length += L
        return torch.cat(outs, dim=1)

    def size(self) -> int:
        return self.length
