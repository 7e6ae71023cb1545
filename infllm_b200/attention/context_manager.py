"""ContextManager with the interface of the reference (inf_llm/attention/context_manager.py:196-816).

The state and the exec-block loop live in libinfllm_b200 (one native context per batch element,
see include/infllm_b200.h); this class validates arguments the way the reference does, feeds
tensors in and exposes the reference's observable attributes."""
import ctypes
import json
from typing import Optional

import torch

from .. import _lib


# Test hook: {field of infllm_config: value} written into the native configuration of every context created while
# it is set (debug_flags selects kernel families and turns look-ahead off, look_depth sets the look-ahead depth).
# The test-suite sets it with monkeypatch; nothing else does.
TEST_OVERRIDES: dict = {}


def device_store_reserve(mib: int, device=None):
    """Reserve `mib` MiB of device memory on `device` for device copies of the stores (ContextManager(...,
    device_store_mb=...)).  This is the only allocation the device copy makes: contexts take 128 MiB slabs from this
    pool as their stores grow, give them back on reset, and keep refilling from the host when it is empty."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    _lib.check(_lib.lib.infllm_device_store_reserve(int(dev), int(mib) << 20))


def device_store_release(device=None):
    """Free the pool's slabs that no context holds."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    _lib.check(_lib.lib.infllm_device_store_release(int(dev)))


def device_store_info(device=None):
    """(MiB reserved, MiB handed out to contexts) of the device's pool."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    tot, used = ctypes.c_int64(), ctypes.c_int64()
    _lib.check(_lib.lib.infllm_device_store_info(int(dev), ctypes.byref(tot), ctypes.byref(used)))
    return tot.value >> 20, used.value >> 20


class ContextManager:
    """Per-layer context memory: sliding local window, init sink, sealed memory units with
    representative keys, top-k retrieval, a GPU cache of max_cached_block units with LRU
    replacement over a pinned host store.

    Constructor arguments are those of the reference (context_manager.py:197-209).  `fattn` and
    `async_global_stream` are accepted and ignored: there is one attention implementation, and the
    host store always refills on a side stream.  `faiss` is not built.

    `device_store_mb` (not in the reference; default 0) keeps up to that many MiB of this memory's sealed units in
    device memory as well, taken from the pool of device_store_reserve(): refills of those units are
    device-to-device copies.  With 0 every refill comes from the pinned host store, as in the reference."""

    def __init__(self, position_embedding, n_init, n_local, block_size, max_cached_block, topk, exc_block_size,
                 score_decay: Optional[float] = None, fattn: bool = False, repr_topk: int = 1,
                 cache_strategy="lru", chunk_topk_calc: Optional[int] = None, async_global_stream: bool = False,
                 pin_memory: bool = False, faiss: bool = False, perhead: bool = False, head_group_comm=None,
                 device_store_mb: int = 0):
        self.length = 0
        self.device_store_mb = int(device_store_mb)
        self.head_group_comm = head_group_comm  # HeadGroupComm: the heads given to append() are this rank's slice
        self.position_embedding = position_embedding
        self.n_init = n_init
        self.n_local = n_local
        self.block_size = block_size
        self.max_cached_block = max_cached_block
        self.exc_block_size = exc_block_size
        self.score_decay = score_decay
        assert exc_block_size <= n_local  # context_manager.py:219
        self.topk = topk
        self.fattn = fattn
        self.initialized = False
        self.repr_topk = repr_topk
        self.cache_strategy = cache_strategy
        self.chunk_topk_calc = chunk_topk_calc
        self.async_global_stream = async_global_stream
        self.pin_memory = pin_memory
        self.faiss = faiss
        self.perhead = perhead
        assert cache_strategy in ["lru", "lru-s"]  # context_manager.py:238
        if faiss:
            raise NotImplementedError("faiss retrieval is not built (the reference needs the faiss package for it)")
        if chunk_topk_calc is not None and chunk_topk_calc < exc_block_size:
            raise ValueError("chunk_topk_calc must hold at least one exec block")  # the reference divides by zero
        self.chunk_topk_calc = chunk_topk_calc
        self._ctx = []  # native contexts, one per unit

    # -- native contexts
    def _init(self, q, k):
        batch, heads, _, dim = q.shape
        heads_kv = k.size(1)
        self.batch_size, self.num_heads, self.num_heads_kv, self.dim_head = batch, heads, heads_kv, dim
        if self.perhead:  # context_manager.py:690-704: every head is its own unit
            self.num_units, self.unit_size, self.unit_size_kv = batch * heads, 1, 1
        else:
            self.num_units, self.unit_size, self.unit_size_kv = batch, heads, heads_kv
        self.dtype = q.dtype
        self.device = q.device
        pe = self.position_embedding
        cfg = _lib.Config(
            n_heads=self.unit_size, n_kv_heads=self.unit_size_kv, head_dim=dim, n_init=self.n_init,
            n_local=self.n_local, block_size=self.block_size, max_cached_block=self.max_cached_block, topk=self.topk,
            exc_block_size=self.exc_block_size, repr_topk=self.repr_topk,
            cache_strategy=_lib.CACHE_LRU if self.cache_strategy == "lru" else _lib.CACHE_LRU_S,
            dtype=_lib.dtype_code(q.dtype), score_decay=float(self.score_decay or 0.0), rope_base=float(pe.base),
            rope_scale=float(pe.distance_scale), device=q.device.index if q.device.index is not None else
            torch.cuda.current_device(), shard_rank=0, shard_world=1)
        if self.chunk_topk_calc is not None:
            cfg.chunk_topk_calc = int(self.chunk_topk_calc)  # context_manager.py:749-770
        cfg.device_store_mb = int(self.device_store_mb)
        for name, value in TEST_OVERRIDES.items():  # empty outside the test-suite
            setattr(cfg, name, int(value))
        for _ in range(self.num_units):
            h = ctypes.c_void_p()
            _lib.check(_lib.lib.infllm_ctx_create(ctypes.byref(cfg), ctypes.byref(h)))
            if self.head_group_comm is not None:
                _lib.check(_lib.lib.infllm_ctx_set_comm(h, self.head_group_comm.handle))
            self._ctx.append(h)
            if getattr(self, "_profile", False):
                _lib.check(_lib.lib.infllm_ctx_profile(h, 1))
        self.initialized = True

    def __del__(self):
        try:
            for h in self._ctx:
                _lib.lib.infllm_ctx_destroy(h)
        except Exception:
            pass
        self._ctx = []

    # -- the path
    def append(self, local_q, local_k, local_v, global_q, global_k, global_v):
        """context_manager.py:682-813.  q (B, H, L, D); k, v (B, H_kv, L, D); returns (B, H, L, D).
        The global tensors must be the local ones (inf_llm/attention/inf_llm.py:58-59 passes the same
        projections twice); the kernels rotate them per stage themselves."""
        if self.initialized and local_q.shape[2] == 1 and not self.perhead and local_q.shape[0] == 1 and local_q.is_cuda:
            return self._append_token(local_q, local_k, local_v, global_q)
        for t in (local_q, local_k, local_v):
            _lib.require_cuda(t, "ContextManager.append input")
        if global_q is not local_q and global_q.data_ptr() != local_q.data_ptr():
            raise NotImplementedError("distinct global_q/k/v tensors are not supported: pass the local ones")
        assert local_q.dim() == 4
        batch, heads, length, dim = local_q.shape
        for t in (local_q, local_k, local_v):  # context_manager.py:301-306
            assert t.size(0) == batch and t.size(2) == length and t.size(3) == dim
        if not self.initialized:
            self._init(local_q, local_k)
        assert heads == self.num_heads and local_k.size(1) == self.num_heads_kv and batch == self.batch_size
        q, k, v = local_q, local_k, local_v
        if q.stride(-1) != 1:
            q = q.contiguous()
        if k.stride(-1) != 1 or k.stride() != v.stride():
            k, v = k.contiguous(), v.contiguous()
        out = torch.empty((batch, heads, length, dim), dtype=q.dtype, device=q.device)
        stream = _lib.stream_ptr(q.device)
        if self.perhead:
            g = heads // self.num_heads_kv
            for b in range(batch):
                for h in range(heads):
                    qq, kk, vv, oo = q[b, h:h + 1], k[b, h // g:h // g + 1], v[b, h // g:h // g + 1], out[b, h:h + 1]
                    self._append_unit(self._ctx[b * heads + h], qq, kk, vv, oo, length, stream)
        else:
            for b in range(batch):
                self._append_unit(self._ctx[b], q[b], k[b], v[b], out[b], length, stream)
        self.length += length
        return out

    def _append_token(self, q, k, v, global_q):
        """One token of one sequence: the same call with the checks that cannot fail for this shape left out (the
        host's share of a decode step is a few tens of microseconds, of the order of the GPU's)."""
        if global_q is not q and global_q.data_ptr() != q.data_ptr():
            raise NotImplementedError("distinct global_q/k/v tensors are not supported: pass the local ones")
        if q.shape[1] != self.num_heads or k.shape[1] != self.num_heads_kv or q.dtype != self.dtype or \
                q.stride(-1) != 1 or k.stride(-1) != 1 or k.stride() != v.stride() or not (k.is_cuda and v.is_cuda):
            raise ValueError("ContextManager.append: a one-token call with other shapes, strides or dtype than the memory's")
        out = torch.empty_like(q, memory_format=torch.contiguous_format)
        rc = _lib.lib.infllm_ctx_append(
            self._ctx[0], q.data_ptr(), q.stride(1), q.stride(2), k.data_ptr(), k.stride(1), k.stride(2), v.data_ptr(),
            v.stride(1), v.stride(2), out.data_ptr(), out.stride(1), out.stride(2), 1,
            torch.cuda.current_stream(q.device).cuda_stream)
        if rc:
            _lib.check(rc)
        self.length += 1
        return out

    @staticmethod
    def _append_unit(ctx, q, k, v, o, length, stream):
        _lib.check(_lib.lib.infllm_ctx_append(
            ctx, q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1), v.data_ptr(),
            v.stride(0), v.stride(1), o.data_ptr(), o.stride(0), o.stride(1), length, stream))

    def size(self, *args, **kwargs):
        return self.length

    # -- what the reference keeps as attributes
    def info(self, u=0):
        info = _lib.CtxInfo()
        _lib.check(_lib.lib.infllm_ctx_get_info(self._ctx[u], ctypes.byref(info)))
        return {n: getattr(info, n) for n, _ in _lib.CtxInfo._fields_}

    @property
    def num_global_block(self):
        return self.info()["num_blocks"] if self._ctx else 0

    @property
    def cached_blocks(self):
        """[{block id: stamp}] per unit, in the reference's dict order (context_manager.py:318)."""
        out = []
        for h in self._ctx:
            cap = self.max_cached_block + self.topk
            ids, st, n = (ctypes.c_int32 * cap)(), (ctypes.c_double * cap)(), ctypes.c_int()
            _lib.check(_lib.lib.infllm_ctx_get_cached(h, ids, st, cap, ctypes.byref(n)))
            out.append({int(ids[i]): st[i] for i in range(n.value)})
        return out

    def last_topk(self, u=0):
        """Retrieved ids of every exec block of the last append, in scorer order."""
        n_eb = self.info(u)["exec_blocks"]
        out = []
        for eb in range(n_eb):
            ids, n = (ctypes.c_int32 * max(self.topk, 1))(), ctypes.c_int()
            _lib.check(_lib.lib.infllm_ctx_get_topk(self._ctx[u], eb, ids, self.topk, ctypes.byref(n)))
            out.append([int(ids[i]) for i in range(n.value)])
        return out

    def block_k_rows(self, u=0):
        """Representative keys (num_blocks, H*D) of unit u as a host tensor."""
        n = self.info(u)["num_blocks"]
        t = torch.empty((n, self.unit_size * self.dim_head), dtype=self.dtype)
        if n:
            _lib.check(_lib.lib.infllm_ctx_get_block_k(self._ctx[u], 0, n, t.data_ptr()))
        return t

    def profile(self, enable=True):
        """Time the hot kernels with CUDA events on their stream (off by default)."""
        self._profile = bool(enable)
        for h in self._ctx:
            _lib.check(_lib.lib.infllm_ctx_profile(h, int(enable)))

    def get_profile(self):
        """{slot: (device ms, algorithmic work, launches)} summed over units since the last call."""
        names = ("attn", "colsum", "decode", "topk")
        tot = {n: [0.0, 0.0, 0] for n in names}
        for h in self._ctx:
            ms, work = (ctypes.c_double * _lib.PROF_SLOTS)(), (ctypes.c_double * _lib.PROF_SLOTS)()
            n = (ctypes.c_int64 * _lib.PROF_SLOTS)()
            _lib.check(_lib.lib.infllm_ctx_get_profile(h, ms, work, n))
            for i, name in enumerate(names):
                tot[name][0] += ms[i]
                tot[name][1] += work[i]
                tot[name][2] += n[i]
        return {k: tuple(v) for k, v in tot.items()}

    def trace(self, enable=True, u=0):
        """Event trace of the exec-block loop (off by default): CUDA events at fixed points of every stream."""
        _lib.check(_lib.lib.infllm_ctx_trace(self._ctx[u], int(enable)))

    def get_trace(self, u=0, cap=65536):
        """[(label, exec block, ms since the first mark)] in record order; clears the trace.  Labels as in
        include/infllm_b200.h (0/1 attention begin/end, 7/8 staged refill copies, 11/12 refill copies waited for)."""
        labels, ebs, ms, n = (ctypes.c_int32 * cap)(), (ctypes.c_int64 * cap)(), (ctypes.c_float * cap)(), ctypes.c_int()
        _lib.check(_lib.lib.infllm_ctx_get_trace(self._ctx[u], labels, ebs, ms, cap, ctypes.byref(n)))
        return [(int(labels[i]), int(ebs[i]), float(ms[i])) for i in range(n.value)]

    @staticmethod
    def refill_overlap(trace):
        """From a trace: how the refill copies of the cache overlapped the attention kernels.

        Returns dict(copy_ms, staged_ms, late_ms, under_attention_ms, overlap_frac, hidden_frac): copy_ms is the time
        refill copies were running (staged ahead on the copy stream + waited for on the urgent stream),
        under_attention_ms the part of it during which an exec-block attention kernel was running, overlap_frac
        their ratio, and hidden_frac the share of the copy time that no exec block waited for."""
        def intervals(begin, end):
            out, open_at = [], None
            for label, _, t in trace:
                if label == begin:
                    open_at = t
                elif label == end and open_at is not None:
                    out.append((open_at, t))
                    open_at = None
            return out

        attn = sorted(intervals(0, 1))
        staged, late = intervals(7, 8), intervals(11, 12)

        def under(iv):
            a, b = iv
            return sum(max(0.0, min(b, y) - max(a, x)) for x, y in attn if y > a and x < b)

        staged_ms, late_ms = sum(b - a for a, b in staged), sum(b - a for a, b in late)
        copy_ms = staged_ms + late_ms
        hidden = sum(under(iv) for iv in staged) + sum(under(iv) for iv in late)
        return dict(copy_ms=copy_ms, staged_ms=staged_ms, late_ms=late_ms, under_attention_ms=hidden,
                    overlap_frac=(hidden / copy_ms if copy_ms > 0 else None),
                    hidden_frac=(staged_ms / copy_ms if copy_ms > 0 else None))

    def host_timers(self, u=0):
        """Host microseconds per phase of the exec-block loop since the last call (diagnostics)."""
        us = (ctypes.c_double * 8)()
        _lib.check(_lib.lib.infllm_ctx_get_host_timers(self._ctx[u], us))
        names = ("rank_sync", "plan", "lookahead_launch", "attn_launch", "lookahead_stage", "seal", "cand_wait")
        return {n: us[i] for i, n in enumerate(names)}

    def load_synthetic(self, units, block_k, init_k, init_v, win_k, win_v):
        """Install a ready-made memory without running a prefill (decode-only workloads and tests).

        units (n, 2, H_kv, block_size, D): K and V of n sealed units; block_k (n, H*D) their representative keys;
        init_k/v (H_kv, n_init, D); win_k/v (H_kv, n_local, D) the local window.  All host tensors of the
        activation dtype.  Afterwards length = n_init + n*block_size + n_local, batch size 1."""
        dtype, hkv, d = units.dtype, units.size(2), units.size(4)
        heads = block_k.size(1) // d
        if not self.initialized:
            dev = torch.device("cuda", torch.cuda.current_device())
            self._init(torch.empty((1, heads, 1, d), dtype=dtype, device=dev),
                       torch.empty((1, hkv, 1, d), dtype=dtype, device=dev))
        ts = [t.contiguous() for t in (units, block_k, init_k, init_v, win_k, win_v)]
        for t in ts:
            if t.is_cuda or t.dtype != dtype:
                raise ValueError("load_synthetic takes host tensors of one activation dtype")
        assert ts[0].shape[1:] == (2, self.unit_size_kv, self.block_size, self.dim_head)
        assert ts[4].shape == (self.unit_size_kv, self.n_local, self.dim_head)
        _lib.check(_lib.lib.infllm_ctx_load_synthetic(
            self._ctx[0], ts[0].size(0), ts[0].data_ptr(), ts[1].data_ptr(), ts[2].data_ptr(), ts[3].data_ptr(),
            ts[4].data_ptr(), ts[5].data_ptr(), _lib.stream_ptr(self.device)))
        self.length = self.info()["length"]

    # -- persistence (the reference keeps the memory only live, in past_key_values)
    def save(self, path):
        """Write the whole memory (sink, sealed units, representative keys, un-sealed tokens, LRU tables) to
        `path`.json plus one `path`.u<i> file per unit; load() on a manager built with the same arguments resumes
        the stream exactly where this one stands."""
        if not self.initialized:
            raise RuntimeError("nothing to save: the memory has seen no tokens")
        meta = dict(batch=self.batch_size, heads=self.num_heads, heads_kv=self.num_heads_kv, dim=self.dim_head,
                    dtype=str(self.dtype).split(".")[-1], length=self.length, units=self.num_units)
        stream = _lib.stream_ptr(self.device)
        for i, h in enumerate(self._ctx):
            _lib.check(_lib.lib.infllm_ctx_save(h, f"{path}.u{i}".encode(), stream))
        with open(f"{path}.json", "w") as f:
            json.dump(meta, f)

    def load(self, path, device=None):
        with open(f"{path}.json") as f:
            meta = json.load(f)
        dtype = getattr(torch, meta["dtype"])
        if not self.initialized:
            dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
            self._init(torch.empty((meta["batch"], meta["heads"], 1, meta["dim"]), dtype=dtype, device=dev),
                       torch.empty((meta["batch"], meta["heads_kv"], 1, meta["dim"]), dtype=dtype, device=dev))
        if (self.batch_size, self.num_heads, self.num_heads_kv, self.dim_head, self.dtype, self.num_units) != (
                meta["batch"], meta["heads"], meta["heads_kv"], meta["dim"], dtype, meta["units"]):
            raise ValueError("the saved memory has other shapes than this manager")
        stream = _lib.stream_ptr(self.device)
        for i, h in enumerate(self._ctx):
            _lib.check(_lib.lib.infllm_ctx_load(h, f"{path}.u{i}".encode(), stream))
        self.length = meta["length"]

    def reset(self):
        for h in self._ctx:
            _lib.check(_lib.lib.infllm_ctx_reset(h))
        self.length = 0
