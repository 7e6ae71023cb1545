"""Single-sequence decode over a context memory that is sharded by memory-unit range across GPUs.

The reference keeps a whole layer's memory on one GPU (inf_llm/attention/context_manager.py); it has no
multi-GPU path.  Here rank r of G owns the sealed units [N*r/G, N*(r+1)/G) — their K/V in pinned host memory,
their representative keys, and a GPU cache of max_cached_block units with its own LRU order — while the local
window, the init sink and the un-sealed remainder (a few thousand tokens) are kept by every rank.  One token:

1. every rank scores its own representative keys and takes its local top-k        (calc_block_topk, :366-383)
2. all-gather of the (score, id) pairs, 8 bytes each -> the same global top-k on every rank
3. every rank runs split-K attention over the retrieved units it owns, its 1/G share of the window, and
   (rank 0) the sink / (last rank) the overflow tokens, and reduces that to one (o, lse) partial
4. all-gather of the partials, (D + 1) floats per head -> log-sum-exp merge on every rank   (_append, :474-545)
5. every rank adds its share of the token's local attention row to the accumulated scores; when a unit
   seals (append_global, :614-679) the ranks all-reduce that unit's 128 score columns, pick the same
   representative tokens, and the last rank, which owns every unit sealed after the load, stores it.

A `UnitRangeShard` is one rank's state and drives the kernels through the C ABI; `ShardedDecodeMemory` runs the
five steps over the shards that live in this process (one per process under torch.distributed; all of them in one
process when the ranks are emulated on a single GPU) and the collectives between processes.
"""
import ctypes

import numpy as np
import torch

from .. import _lib

F32 = 2  # INFLLM_F32: fp32 output of infllm_lse_merge


def unit_range(n_total, rank, world):
    """Units owned by `rank` at load time: [lo, hi).  Units sealed later all go to the last rank."""
    return (n_total * rank) // world, (n_total * (rank + 1)) // world


def global_topk(scores, ids, k):
    """The k best of the gathered candidates: descending score, ties to the lower id (the order of the
    single-GPU scorer).  `ids` < 0 mark padding.  Host tensors in, a list of at most k ids out."""
    scores = scores.reshape(-1).numpy()
    ids = ids.reshape(-1).numpy()
    order = np.lexsort((ids, -scores))  # last key first: by score descending, then by id ascending
    return [int(ids[i]) for i in order if ids[i] >= 0][:k]


class UnitRangeShard:
    """One rank's share of the memory and its decode kernels."""

    def __init__(self, rank, world, position_embedding, n_init, n_local, block_size, max_cached_block, topk, repr_topk,
                 n_heads, n_kv_heads, head_dim, dtype=torch.bfloat16, device=None, spare_units=64):
        if head_dim != 128:
            raise NotImplementedError("the decode kernels are built for head_dim 128")
        if max_cached_block < topk:  # CudaCache.alloc would assert (context_manager.py:19)
            raise _lib.InfLLMCapacityError(_lib.E_CAPACITY, "max_cached_block < topk")
        self.rank, self.world = rank, world
        self.pe = position_embedding
        self.n_init, self.n_local, self.bs = n_init, n_local, block_size
        self.max_cached, self.topk, self.repr_topk = max_cached_block, topk, repr_topk
        self.H, self.HKV, self.D = n_heads, n_kv_heads, head_dim
        self.dtype, self.code = dtype, _lib.dtype_code(dtype)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.spare = spare_units
        self.cap = n_local + max(4096, 2 * block_size)  # token slots: window + remainder + room before a compaction
        dev, H, HKV, D = self.device, n_heads, n_kv_heads, head_dim
        self.k_raw = torch.zeros((HKV, self.cap, D), dtype=dtype, device=dev)
        self.k_rot = torch.zeros_like(self.k_raw)
        self.v = torch.zeros_like(self.k_raw)
        self.score = torch.zeros((H, self.cap), dtype=torch.float32, device=dev)
        self.q_loc = torch.empty((H, D), dtype=dtype, device=dev)
        self.q_glb = torch.empty((H, D), dtype=dtype, device=dev)
        self.qbar = torch.empty((H * D,), dtype=torch.float32, device=dev)
        self.cos = torch.empty((self.cap, D // 2), dtype=torch.float32, device=dev)
        self.sin = torch.empty_like(self.cos)
        inv = (1.0 / (float(self.pe.base) ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).contiguous()
        arr = (ctypes.c_float * (D // 2))(*inv.tolist())
        _lib.check(_lib.lib.infllm_rope_table(arr, float(self.pe.distance_scale), D, self.cap, self.cos.data_ptr(),
                                              self.sin.data_ptr(), _lib.stream_ptr()))
        self.cache = torch.zeros((max_cached_block, 2, HKV, block_size, D), dtype=dtype, device=dev)
        self.lru = ctypes.c_void_p()
        _lib.check(_lib.lib.infllm_lru_create(max_cached_block, ctypes.byref(self.lru)))
        # the cache's bookkeeping lives in one structure that infllm_shard_refill works on: which slot holds which
        # owned unit, the stack of free slots, the LRU table, the counters
        self._free_arr = np.arange(max_cached_block - 1, -1, -1, dtype=np.int32)
        self._slot_arr = np.full((1,), -1, dtype=np.int32)
        cs = self._cs = _lib.ShardCache()
        cs.lru, cs.n_free, cs.free_slots = self.lru, max_cached_block, self._free_arr.ctypes.data
        cs.slot_of = self._slot_arr.ctypes.data
        max_keys = n_local + topk * block_size + n_init + block_size
        self.max_parts = int(_lib.lib.infllm_attn_decode_max_parts(topk + 3, max_keys))
        self.part_o = torch.empty((self.max_parts, H, D), dtype=torch.float32, device=dev)
        self.part_lse = torch.empty((self.max_parts, H), dtype=torch.float32, device=dev)
        self.logits = torch.empty((H, n_local + 1), dtype=torch.float32, device=dev)
        # [o (H, D) | lse (H) | miss word | pad]: the message a rank sends to its peers
        self.pack = torch.zeros((H * (D + 1) + 4,), dtype=torch.float32, device=dev)
        # [global retrieval ranked on the device (topk) | exchange error | any miss | pad]: read by the host per token
        self.d_status = torch.zeros((topk + 4,), dtype=torch.int32, device=dev)
        self.d_status[:topk] = -1
        self.h_status = torch.zeros((topk + 4,), dtype=torch.int32).pin_memory()
        self._status_np, self._status_ptr = self.h_status.numpy(), self.h_status.data_ptr()
        self.slot_table = None
        self.lse = torch.empty((H,), dtype=torch.float32, device=dev)
        self.cand = torch.empty((2, topk), dtype=torch.int32, device=dev)         # [score bits | ids]
        self.scores_buf = None
        self.profile = False  # when set, CUDA events bracket the scoring and the attention of every token
        self.flag_in_data = True  # the candidate exchange of run_token: words that carry their own arrival flag
        self.stamps, self.stamp_row = None, 0  # (rows, 8) int64 on the device: see infllm_shard_token.d_stamps
        self._events = {"topk": [], "decode": []}
        self.t0 = self.length = self.frontier = self.n_total = self.lo = self.n_owned = 0
        self.block_k = self.host_units = self.init_k = self.init_v = None
        self._share = (0, 0)
        self._token_args = None
        # raw addresses of the buffers the per-token calls pass on (tensor indexing costs microseconds a piece)
        self._p = {name: getattr(self, name).data_ptr() for name in
                   ("k_raw", "k_rot", "v", "score", "q_loc", "q_glb", "qbar", "cos", "sin", "cache", "part_o", "part_lse",
                    "logits", "pack", "lse", "cand", "d_status")}
        self.unit_bytes = 2 * n_kv_heads * block_size * head_dim * self.k_raw.element_size()
        self._stream = None
        m = topk + 3  # retrieved units + window share + sink + overflow
        self._seg_arrays = ((ctypes.c_void_p * m)(), (ctypes.c_void_p * m)(), (ctypes.c_int64 * m)(),
                            (ctypes.c_int32 * m)(), (ctypes.c_int32 * m)())
        self._unit_seg_arrays = ((ctypes.c_void_p * m)(), (ctypes.c_void_p * m)(), (ctypes.c_int64 * m)(),
                                 (ctypes.c_int32 * m)(), (ctypes.c_int32 * m)())
        for i in range(topk):
            self._unit_seg_arrays[2][i], self._unit_seg_arrays[3][i], self._unit_seg_arrays[4][i] = (
                block_size * head_dim, block_size, 1)

    def __del__(self):
        if getattr(self, "lru", None):
            _lib.lib.infllm_lru_destroy(self.lru)
            self.lru = None

    @property
    def slot_of(self):
        """{owned unit id: cache slot} (a copy, for callers off the per-token path)."""
        a = self._slot_arr[:self.n_owned]
        return {self.lo + int(i): int(a[i]) for i in np.nonzero(a >= 0)[0]}

    hits = property(lambda self: self._cs.hits, lambda self, v: setattr(self._cs, "hits", v))
    misses = property(lambda self: self._cs.misses, lambda self, v: setattr(self._cs, "misses", v))
    load_count = property(lambda self: self._cs.load_count, lambda self, v: setattr(self._cs, "load_count", v))

    def _sync_cache_state(self):
        """The structure follows the tensors it points into (after a load or a growth of the store)."""
        cs, room = self._cs, self.block_k.shape[0]
        if self._slot_arr.shape[0] < room:
            grown = np.full((room,), -1, dtype=np.int32)
            grown[:self._slot_arr.shape[0]] = self._slot_arr
            self._slot_arr = grown
        cs.slot_of = self._slot_arr.ctypes.data
        cs.id_lo, cs.n_owned = self.lo, self.n_owned
        cs.d_cache, cs.h_units, cs.unit_bytes = self._p["cache"], self.host_units.data_ptr(), self.unit_bytes
        cs.d_slot_table, cs.d_ptr_table = self.slot_table.data_ptr(), self.ptr_table.data_ptr()

    # ------------------------------------------------------------------ state
    def load_synthetic(self, n_total, units, block_k, init_k, init_v, win_k, win_v):
        """Install a memory of n_total sealed units of which this rank receives its own range: `units`
        (n_owned, 2, H_kv, bs, D) and `block_k` (n_owned, H*D) on the host, plus the replicated sink
        (H_kv, n_init, D) x2 and window (H_kv, n_local, D) x2."""
        lo, hi = unit_range(n_total, self.rank, self.world)
        n_owned = hi - lo
        assert units.shape[0] == n_owned and block_k.shape[0] == n_owned
        room = n_owned + (self.spare if self.rank == self.world - 1 else 0)
        self.host_units = torch.empty((max(room, 1),) + tuple(units.shape[1:]), dtype=self.dtype).pin_memory()
        self.host_units[:n_owned].copy_(units)
        self.block_k = torch.zeros((max(room, 1), self.H * self.D), dtype=self.dtype, device=self.device)
        self.block_k[:n_owned].copy_(block_k)
        self.scores_buf = torch.empty((max(room, 1),), dtype=torch.float32, device=self.device)
        self.slot_table = torch.full((max(room, 1),), -1, dtype=torch.int32, device=self.device)
        # where every owned unit lives right now: its cache slot, else its place in the pinned host store (which the
        # attention reads in place over PCIe, so that no token waits for a refill)
        self.ptr_table = self._store_addresses(max(room, 1))
        self.ticket = torch.zeros((4,), dtype=torch.int32, device=self.device)
        self.init_k, self.init_v = init_k.to(self.device).contiguous(), init_v.to(self.device).contiguous()
        self._store_pointers()
        self.n_total, self.lo, self.n_owned = n_total, lo, n_owned
        self._sync_cache_state()
        self.frontier = self.n_init + n_total * self.bs
        self.length = self.frontier + self.n_local
        self.t0 = self.frontier
        n = self.n_local
        self.k_raw[:, :n].copy_(win_k)
        self.v[:, :n].copy_(win_v)
        self.score.zero_()
        self._rotate(0, n)

    def _store_addresses(self, room):
        base = self.host_units.data_ptr()
        return (base + torch.arange(room, dtype=torch.int64) * self.unit_bytes).to(self.device)

    def _store_pointers(self):
        self._p.update(block_k=self.block_k.data_ptr(), host_units=self.host_units.data_ptr(),
                       slot_table=self.slot_table.data_ptr(), ptr_table=self.ptr_table.data_ptr(),
                       ticket=self.ticket.data_ptr(),
                       scores_buf=self.scores_buf.data_ptr(), init_k=self.init_k.data_ptr(), init_v=self.init_v.data_ptr())

    def _rope(self, x, x_hs, x_ts, out, o_hs, o_ts, heads, length, pos0, step):
        _lib.check(_lib.lib.infllm_rope_apply(x, x_hs, x_ts, out, o_hs, o_ts, heads, length, self.D, self.cos.data_ptr(),
                                              self.sin.data_ptr(), self.cap, pos0, step, self.code, _lib.stream_ptr()))

    def _rotate(self, slot0, n):
        """k_rot[slot] = RoPE(k_raw[slot]) at position `slot` (token - t0) for slots [slot0, slot0 + n)."""
        off = slot0 * self.D * self.k_raw.element_size()
        self._rope(self.k_raw.data_ptr() + off, self.cap * self.D, self.D, self.k_rot.data_ptr() + off,
                   self.cap * self.D, self.D, self.HKV, n, slot0, 1)

    def _compact(self):
        """Move the live tokens [frontier, length) to slot 0 and rotate them anew."""
        live, s0 = self.length - self.frontier, self.frontier - self.t0
        for buf in (self.k_raw, self.v):
            buf[:, :live] = buf[:, s0:s0 + live].clone()
        self.score[:, :live] = self.score[:, s0:s0 + live].clone()
        self.t0 = self.frontier
        self._rotate(0, live)

    # ------------------------------------------------------------------ step 1
    def begin(self, q, k, v):
        """Ingest one token (q (H, 1, D), k and v (H_kv, 1, D)); returns this rank's candidates as an int32
        tensor (2, topk): the scores' bit patterns and the global unit ids, padded with (-inf, -1)."""
        if self.length - self.t0 >= self.cap:
            self._compact()
        T, at, D, p = self.length, self.length - self.t0, self.D, self._p
        row = at * D * 2
        self._stream = stream = _lib.stream_ptr()
        # copies, the three rotations (keys and queries window-relative, queries at the one global angle), the
        # query "mean" of the one-token exec block (context_manager.py:373-375) and the new score column
        _lib.check(_lib.lib.infllm_ingest_token(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), p["q_loc"], p["q_glb"], D,
            p["qbar"], p["k_raw"] + row, p["k_rot"] + row, p["v"] + row, self.cap * D, p["score"] + at * 4, self.cap,
            self.H, self.HKV, D, p["cos"], p["sin"], self.cap, T - self.t0, self.n_local - 1, self.code, stream))
        if self.n_owned < self.topk:  # fewer units than a retrieval takes: pad the candidates
            self.cand[0].view(torch.float32).fill_(float("-inf"))
            self.cand[1].fill_(-1)
        if self.n_owned > 0:
            kk = min(self.topk, self.n_owned)
            ev = self._mark("topk")
            _lib.check(_lib.lib.infllm_block_topk(p["block_k"], self.n_owned, self.H * D, p["qbar"], p["scores_buf"], kk,
                                                  self.lo, p["cand"] + 4 * self.topk, p["cand"], self.code, stream))
            self._mark("topk", ev)
        return self.cand

    def _mark(self, slot, begin=None):
        if not self.profile:
            return None
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        if begin is not None:
            self._events[slot].append((begin, e))
        return e

    def get_profile(self):
        """{slot: (milliseconds, launches)} of the bracketed kernels since the last call; synchronises."""
        torch.cuda.synchronize(self.device)
        out = {k: (sum(a.elapsed_time(b) for a, b in v), len(v)) for k, v in self._events.items()}
        self._events = {k: [] for k in self._events}
        return out

    # ------------------------------------------------------------------ step 3
    def attend(self, ids):
        """Partial attention of this rank for the global retrieval `ids` (host list); returns the packed
        fp32 tensor [o (H, D) | lse (H)]."""
        E, G, r = self.length + 1, self.world, self.rank
        owned = [b for b in ids if self.lo <= b < self.lo + self.n_owned]
        self._refill(owned)
        segs = []  # (k pointer, v pointer, head stride, length, query variant)
        esz, D, p = 2, self.D, self._p
        for b in owned:
            base = p["cache"] + self.slot_of[b] * self.unit_bytes
            segs.append((base, base + self.unit_bytes // 2, self.bs * D, self.bs, 1))
        wlo = max(E - self.n_local, 0)
        W = E - wlo
        a, b_ = wlo + (W * r) // G, wlo + (W * (r + 1)) // G
        self._share = (a, b_)
        logit_seg = -1
        if b_ > a:
            off = (a - self.t0) * D * esz
            logit_seg = len(segs)
            segs.append((p["k_rot"] + off, p["v"] + off, self.cap * D, b_ - a, 0))
        if r == 0 and self.n_init > 0:
            segs.append((p["init_k"], p["init_v"], self.n_init * D, self.n_init, 1))
        if r == G - 1 and wlo > self.frontier:  # tokens between the last sealed unit and the window
            off = (self.frontier - self.t0) * D * esz
            segs.append((p["k_raw"] + off, p["v"] + off, self.cap * D, wlo - self.frontier, 1))
        if not segs:
            self.pack[:self.H * D].zero_()
            self.pack[self.H * D:self.H * (D + 1)].fill_(float("-inf"))
            return self.pack
        n = len(segs)
        kp, vp, hs, ln, qs = self._seg_arrays
        for i, sg in enumerate(segs):
            kp[i], vp[i], hs[i], ln[i], qs[i] = sg
        n_parts = ctypes.c_int()
        self.keys_last = sum(s[3] for s in segs)
        ev = self._mark("decode")
        _lib.check(_lib.lib.infllm_attn_decode(p["q_loc"], p["q_glb"], self.H, self.HKV, D, n, kp, vp, hs, ln, qs,
                                               p["part_o"], p["part_lse"], self.max_parts, ctypes.byref(n_parts),
                                               logit_seg, p["logits"], self.code, self._stream))
        _lib.check(_lib.lib.infllm_lse_merge(p["part_o"], p["part_lse"], n_parts.value, self.H, D, p["pack"], D,
                                             p["pack"] + self.H * D * 4, F32, self._stream))
        self._mark("decode", ev)
        return self.pack

    def _refill(self, ids, n=None):
        """LRU plan for the owned part of a retrieval (context_manager.py:246-265, 495-515) and the copies of the
        units that are not cached, from the pinned store into free slots: one call into the library.  `ids`: a list,
        or the address of n int32 (entries that are negative or another rank's are skipped)."""
        if n is None:
            n = len(ids)
            ids = (ctypes.c_int32 * max(n, 1))(*ids)
        _lib.check(_lib.lib.infllm_shard_refill(ctypes.byref(self._cs), ids, n, self._stream))

    def run_token(self, q, k, v, out, mb):
        """One token through infllm_shard_token_run: every launch of it in one call (see the header).  Leaves the
        merged output in `out` and the retrieval + status words in h_status once the stream has drained."""
        if self.length - self.t0 >= self.cap:
            self._compact()
        a, p = self._token_args, self._p
        if a is None:
            a = self._token_args = _lib.ShardToken()
            for name in ("q_loc", "q_glb", "qbar", "k_raw", "k_rot", "v", "score", "cos", "sin", "cand", "part_o",
                         "part_lse", "logits", "pack", "lse", "cache"):
                setattr(a, "d_" + name, p[name])
            a.d_status, a.h_status = p["d_status"], self.h_status.data_ptr()
            a.cap, a.n_heads, a.n_kv_heads, a.head_dim, a.dtype = self.cap, self.H, self.HKV, self.D, self.code
            a.n_local, a.block_size, a.topk, a.unit_bytes, a.max_parts = (self.n_local, self.bs, self.topk,
                                                                          self.unit_bytes, self.max_parts)
            a.cand_off, a.cand_slot, a.cand_bytes = mb.cand_off, mb.cand_slot, mb.cand_bytes
            a.part_off, a.part_slot, a.part_bytes = mb.part_off, mb.part_slot, mb.part_bytes
            a.flag1_off, a.flag2_off, a.wait_us = mb.flag1, mb.flag2, mb.wait_us
            a.ll_cand_off, a.ll_cand_slot = (mb.ll_cand_off, mb.ll_cand_slot) if self.flag_in_data else (0, 0)
            a.ll_part_off, a.ll_part_slot = (mb.ll_part_off, mb.ll_part_slot) if self.flag_in_data else (0, 0)
            # (the store's addresses change only when it grows, which drops this block)
            a.d_block_k, a.d_scores, a.d_slot_table = p["block_k"], p["scores_buf"], p["slot_table"]
            a.d_unit_ptrs, a.d_ticket = p["ptr_table"], p["ticket"]
            first = self.rank == 0 and self.n_init > 0
            a.d_init_k, a.d_init_v, a.init_len = (p["init_k"], p["init_v"], self.n_init) if first else (None, None, 0)
        E, G, r = self.length + 1, self.world, self.rank
        wlo = max(E - self.n_local, 0)
        W = E - wlo
        lo_, hi_ = wlo + (W * r) // G, wlo + (W * (r + 1)) // G
        self._share = (lo_, hi_)
        a.d_q, a.d_k, a.d_vin, a.q_hs, a.k_hs, a.v_hs = q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), k.stride(0), v.stride(0)
        a.at = self.length - self.t0
        a.n_owned, a.id_lo = self.n_owned, self.lo
        a.share_at, a.share_len = lo_ - self.t0, hi_ - lo_
        last = r == G - 1 and wlo > self.frontier
        a.ovf_at, a.ovf_len = (self.frontier - self.t0, wlo - self.frontier) if last else (0, 0)
        a.d_out, a.seq = out.data_ptr(), mb.seq
        if self.stamps is not None:  # a profiling pass: one row of 8 device timestamps per token
            a.d_stamps = self.stamps.data_ptr() + 64 * (self.stamp_row % self.stamps.shape[0])
            self.stamp_row += 1
        else:
            a.d_stamps = None
        self._stream = _lib.stream_ptr()
        _lib.check(_lib.lib.infllm_shard_token_run(ctypes.byref(a), mb.handle, self._stream))

    def attend_device(self):
        """attend() for a retrieval that exists only on the device so far (d_gids): the owned units are found through
        the device table of unit addresses — in their cache slots, or in place in the pinned store.  The message
        [o | lse | miss word] is left in `pack` (the miss word stays 0: every owned unit has an address)."""
        E, G, r = self.length + 1, self.world, self.rank
        esz, D, p = 2, self.D, self._p
        kp, vp, hs, ln, qs = self._unit_seg_arrays  # the first topk entries are placeholders the kernel resolves
        n = self.topk
        wlo = max(E - self.n_local, 0)
        W = E - wlo
        a, b_ = wlo + (W * r) // G, wlo + (W * (r + 1)) // G
        self._share = (a, b_)
        logit_seg = -1
        if b_ > a:
            off = (a - self.t0) * D * esz
            logit_seg = n
            kp[n], vp[n], hs[n], ln[n], qs[n] = p["k_rot"] + off, p["v"] + off, self.cap * D, b_ - a, 0
            n += 1
        if r == 0 and self.n_init > 0:
            kp[n], vp[n], hs[n], ln[n], qs[n] = p["init_k"], p["init_v"], self.n_init * D, self.n_init, 1
            n += 1
        if r == G - 1 and wlo > self.frontier:
            off = (self.frontier - self.t0) * D * esz
            kp[n], vp[n], hs[n], ln[n], qs[n] = p["k_raw"] + off, p["v"] + off, self.cap * D, wlo - self.frontier, 1
            n += 1
        n_parts = ctypes.c_int()
        miss = p["pack"] + self.H * (D + 1) * 4
        ev = self._mark("decode")
        _lib.check(_lib.lib.infllm_attn_decode_units(
            p["q_loc"], p["q_glb"], self.H, self.HKV, D, n, kp, vp, hs, ln, qs, 0, self.topk, p["d_status"], p["ptr_table"],
            self.lo, self.n_owned, None, self.unit_bytes, miss, p["part_o"], p["part_lse"], self.max_parts,
            ctypes.byref(n_parts), logit_seg, p["logits"], self.code, self._stream))
        _lib.check(_lib.lib.infllm_lse_merge(p["part_o"], p["part_lse"], n_parts.value, self.H, D, p["pack"], D,
                                             p["pack"] + self.H * D * 4, F32, self._stream))
        self._mark("decode", ev)

    # ------------------------------------------------------------------ step 5
    def merge(self, parts):
        """Step 4 and the first half of step 5 on this rank: log-sum-exp merge of the gathered partials
        (G, H*(D+1)) fp32 rows [o | lse] into the token's output (H, D), and this rank's share of the token's local
        attention row added to the accumulated scores, in one launch."""
        return self.merge_raw(parts.data_ptr(), parts.stride(0), parts.shape[0], None)

    def merge_raw(self, base, stride, n, skip):
        """merge() over n messages `stride` floats apart at device address `base`; `skip`: address of a device
        word that voids the call when it is non-zero (or None)."""
        H, D, p = self.H, self.D, self._p
        out = torch.empty((H, D), dtype=self.dtype, device=self.device)
        a, b = self._share
        _lib.check(_lib.lib.infllm_lse_merge_ex(
            base, stride, base + H * D * 4, stride, n, H, D, out.data_ptr(), D, p["lse"], self.code,
            p["logits"] if b > a else None, b - a, p["score"] + (a - self.t0) * 4, self.cap, skip, self._stream))
        return out

    def finish(self):
        """Count the token in.  Returns the (H, bs) score columns of the unit that seals now — this rank's
        partial sums, to be all-reduced — or None."""
        self.length += 1
        if self.length - self.frontier - self.bs >= self.n_local:  # context_manager.py:649
            s0 = self.frontier - self.t0
            return self.score[:, s0:s0 + self.bs].contiguous()
        return None

    def seal(self, scores):
        """Seal the oldest un-sealed 128 tokens as a unit, given their all-reduced score columns (H, bs)."""
        s0, D = self.frontier - self.t0, self.D
        self.score[:, s0:s0 + self.bs] = scores
        if self.rank == self.world - 1:
            if self.n_owned >= self.block_k.shape[0]:
                self._grow()
            row = self.block_k[self.n_owned]
            _lib.check(_lib.lib.infllm_repr_select(self.k_raw.data_ptr(), self.cap * D, D, self.score.data_ptr(), self.cap,
                                                   s0, 1, self.bs, self.repr_topk, self.H, self.HKV, D, row.data_ptr(),
                                                   self.code, _lib.stream_ptr()))
            unit = self.host_units[self.n_owned]
            unit[0].copy_(self.k_raw[:, s0:s0 + self.bs], non_blocking=True)
            unit[1].copy_(self.v[:, s0:s0 + self.bs], non_blocking=True)
            self.n_owned += 1
            self._cs.n_owned = self.n_owned
        self.frontier += self.bs
        self.n_total += 1

    def _grow(self):
        room = self.block_k.shape[0] + max(self.spare, 1)
        torch.cuda.current_stream().synchronize()  # copies into the old store have landed
        host = torch.empty((room,) + tuple(self.host_units.shape[1:]), dtype=self.dtype).pin_memory()
        host[:self.n_owned].copy_(self.host_units[:self.n_owned])
        self.host_units = host
        bk = torch.zeros((room, self.H * self.D), dtype=self.dtype, device=self.device)
        bk[:self.n_owned].copy_(self.block_k[:self.n_owned])
        self.block_k = bk
        self.scores_buf = torch.empty((room,), dtype=torch.float32, device=self.device)
        table = torch.full((room,), -1, dtype=torch.int32, device=self.device)
        table[:self.slot_table.shape[0]].copy_(self.slot_table)
        self.slot_table = table
        ptrs = self._store_addresses(room)  # the store moved: cached units keep their slots
        for b, slot in self.slot_of.items():
            ptrs[b - self.lo] = self._p["cache"] + slot * self.unit_bytes
        self.ptr_table = ptrs
        self._store_pointers()
        self._sync_cache_state()
        self._token_args = None


class PeerMailbox:
    """This rank's mailbox in device memory, writable by every rank of the node (CUDA IPC), for the two
    exchanges of a token: the retrieval candidates and the attention partials.  Collective: every rank of
    `group` constructs it.  Layout: [flags of exchange 1 | flags of exchange 2 | candidate slots | partial slots].
    """

    def __init__(self, topk, n_heads, head_dim, group=None, device=None, wait_us=2000000):
        import torch.distributed as dist

        self.group, self.rank, self.world = group, dist.get_rank(group), dist.get_world_size(group)
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.wait_us = wait_us
        self.flag1, self.flag2 = 0, 256
        self.cand_off, self.cand_bytes = 512, 2 * topk * 4
        self.cand_slot = (self.cand_bytes + 15) // 16 * 16
        self.part_off = (self.cand_off + self.world * self.cand_slot + 255) // 256 * 256
        self.part_bytes = (n_heads * (head_dim + 1) + 4) * 4  # [o | lse | miss word | pad]
        self.part_slot = (self.part_bytes + 15) // 16 * 16
        self.miss_off = n_heads * (head_dim + 1) * 4
        # a second candidate region for the exchange whose words carry their own arrival flag (8 bytes per word)
        self.ll_cand_off = (self.part_off + self.world * self.part_slot + 255) // 256 * 256
        self.ll_cand_slot = 2 * topk * 8
        self.ll_part_off = (self.ll_cand_off + self.world * self.ll_cand_slot + 255) // 256 * 256
        self.ll_part_slot = self.part_bytes // 4 * 8
        total = self.ll_part_off + self.world * self.ll_part_slot
        n = int(_lib.lib.infllm_mailbox_handle_bytes())
        mine = (ctypes.c_ubyte * n)()
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(_lib.lib.infllm_mailbox_create(total, self.rank, self.world, mine, ctypes.byref(self.handle)))
            if self.world > 1:
                local = torch.tensor(list(mine), dtype=torch.uint8, device=device)
                every = torch.empty((self.world, n), dtype=torch.uint8, device=device)
                dist.all_gather_into_tensor(every, local[None], group=group)
                flat = every.cpu().reshape(-1).tolist()
                _lib.check(_lib.lib.infllm_mailbox_open(self.handle, (ctypes.c_ubyte * len(flat))(*flat)))
                dist.barrier(group=group)  # nobody writes before everybody has mapped
        self.local = int(_lib.lib.infllm_mailbox_local(self.handle))
        self.seq = 0

    def close(self):
        if getattr(self, "handle", None):
            _lib.lib.infllm_mailbox_destroy(self.handle)
            self.handle = None

    def __del__(self):
        self.close()


class ShardedDecodeMemory:
    """Runs one token through the shards of this process and the collectives between processes.

    shards: the UnitRangeShard objects that live in this process, in rank order — one under torch.distributed
    (pass `group`, or leave None for the default group), or all G of them when the ranks share one process.
    """

    def __init__(self, shards, distributed=False, group=None, mailbox=None):
        self.shards, self.distributed, self.group = list(shards), distributed, group
        # with a PeerMailbox the two exchanges of a token run inside kernels over peer memory and the retrieval is
        # ranked on the device; the collectives below remain for the rare token that has to be redone (a retrieved
        # unit was not cached) and for the score columns of a sealing
        self.mailbox = mailbox if (distributed and mailbox is not None and mailbox.world > 1) else None
        self.redone = 0  # tokens that had to be run again (none since retrieved units are read wherever they live)
        self._pending = None  # the event behind the status copy of the token whose retrieval is not applied yet
        self._events = None
        self._last_ids = []
        if not distributed:
            assert [s.rank for s in self.shards] == list(range(self.shards[0].world)), "emulation needs every rank"

    @property
    def last_ids(self):
        """The global retrieval of the last token (applies it to the cache tables first if that is still due)."""
        self._settle()
        if self._last_ids is None:
            self._last_ids = [int(b) for b in self._last_status if b >= 0]
        return self._last_ids

    @last_ids.setter
    def last_ids(self, ids):
        self._last_ids = ids

    def _settle(self):
        """The token launched last ran ahead of the host: read its retrieval and status words now (they left the
        device right behind its kernels), check the exchange status and advance this rank's LRU order; a retrieved
        unit that is not cached is refilled on the token stream — the token itself read it in place."""
        if self._pending is None:
            return
        s = self.shards[0]
        self._pending.synchronize()
        self._pending = None
        st = s._status_np
        if st[s.topk]:
            s.d_status[s.topk:].zero_()
            raise _lib.InfLLMError(_lib.E_TIMEOUT, f"rank {int(st[s.topk]) - 1} did not arrive at an exchange of the "
                                                   "sharded decode within the limit")
        self._last_ids = None
        self._last_status = st[:s.topk].copy()
        s._refill(s._status_ptr, s.topk)

    def _all_gather(self, local):
        """local: (n_local_shards, ...) -> (world, ...) in rank order."""
        if not self.distributed:
            return local
        import torch.distributed as dist

        out = torch.empty((dist.get_world_size(self.group),) + tuple(local.shape[1:]), dtype=local.dtype,
                          device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=self.group)
        return out

    def _all_reduce(self, t):
        if self.distributed:
            import torch.distributed as dist

            dist.all_reduce(t, group=self.group)
        return t

    def append(self, q, k, v):
        """q (H, 1, D), k and v (H_kv, 1, D) of one new token -> attention output (H, 1, D)."""
        s0 = self.shards[0]
        if self.mailbox is not None and s0.n_total > s0.topk:
            return self._append_peer(q, k, v)
        cand = self._all_gather(self._stack([s.begin(q, k, v) for s in self.shards]))  # (G, 2, topk) int32
        if s0.n_total <= s0.topk:  # every unit, in id order, no scoring (context_manager.py:370-371)
            ids = list(range(s0.n_total))
        else:  # the ids go to the host anyway (cache plans); rank the G * topk candidates there
            c = cand.cpu()
            ids = global_topk(c[:, 0].contiguous().view(torch.float32), c[:, 1], s0.topk)
        self.last_ids = ids
        parts = self._all_gather(self._stack([s.attend(ids) for s in self.shards]))  # (G, H*(D+1)) fp32
        outs = [s.merge(parts) for s in self.shards]  # the same on every rank
        sealing = [s.finish() for s in self.shards]
        if sealing[0] is not None:
            total = self._all_reduce(sealing[0] if len(sealing) == 1 else torch.stack(sealing).sum(dim=0))
            for s in self.shards:
                s.seal(total)
        return outs[0].view(s0.H, 1, s0.D)

    def _append_peer(self, q, k, v):
        """append() with both exchanges inside kernels: candidates and partials are written straight into the
        peers' mailboxes, the global top-k is ranked on the device and the attention resolves the retrieved units
        it owns through the device copy of its slot table.  The host reads the retrieval afterwards, for the LRU
        order, and redoes the token through the collectives if any rank reports a unit that was not cached."""
        s, mb, lib = self.shards[0], self.mailbox, _lib.lib
        p, H, D = s._p, s.H, s.D
        if self._events is None:
            self._events = (torch.cuda.Event(), torch.cuda.Event())
        if mb.seq == 0 and self.distributed:  # the first exchange: nobody waits on a rank that is still setting up
            import torch.distributed as dist

            dist.barrier(group=self.group)
        self._settle()  # the previous token's retrieval: LRU order, refills (stream-ordered ahead of this token)
        mb.seq += 1
        if s.n_owned >= s.topk:  # the whole token in one call into the library
            out = torch.empty((H, D), dtype=s.dtype, device=s.device)
            s.run_token(q, k, v, out, mb)
        else:  # fewer owned units than a retrieval takes: the candidate message needs padding; piece by piece
            s.begin(q, k, v)
            st = s._stream
            err, any_miss = p["d_status"] + 4 * s.topk, p["d_status"] + 4 * s.topk + 4
            miss_word = p["pack"] + H * (D + 1) * 4
            _lib.check(lib.infllm_mailbox_put(mb.handle, p["cand"], mb.cand_bytes, mb.cand_off, mb.cand_slot, mb.flag1,
                                              mb.seq, st))
            _lib.check(lib.infllm_mailbox_wait(mb.handle, mb.flag1, mb.seq, mb.wait_us, err, 0, 0, -1, None, miss_word,
                                               st))
            _lib.check(lib.infllm_topk_pairs(mb.local + mb.cand_off, mb.cand_slot // 4, mb.world, s.topk, p["d_status"],
                                             err, st))
            s.attend_device()
            _lib.check(lib.infllm_mailbox_put(mb.handle, p["pack"], mb.part_bytes, mb.part_off, mb.part_slot, mb.flag2,
                                              mb.seq, st))
            _lib.check(lib.infllm_mailbox_wait(mb.handle, mb.flag2, mb.seq, mb.wait_us, err, mb.part_off, mb.part_slot,
                                               mb.miss_off, any_miss, None, st))
            out = s.merge_raw(mb.local + mb.part_off, mb.part_slot // 4, mb.world, any_miss)
            s.h_status.copy_(s.d_status, non_blocking=True)
        # the host does not wait: the status words and the retrieval are read when the next token arrives (or when
        # somebody asks for last_ids), and the LRU order is advanced then
        self._pending = self._events[mb.seq & 1]
        self._pending.record()
        sealing = s.finish()
        if sealing is not None:
            s.seal(self._all_reduce(sealing))
        return out.view(H, 1, D)

    @staticmethod
    def _stack(tensors):
        return tensors[0].unsqueeze(0) if len(tensors) == 1 else torch.stack(tensors)
