"""infllm_shard_refill against a plain restatement of the reference's cache bookkeeping (context_manager.py:246-265,
495-515: evict the least recently stamped units that are not wanted, stamp the wanted ones with the load count,
load what is missing): slots, free stack, counters, LRU order, the copied units and both device tables."""
import ctypes

import numpy as np
import pytest
import torch

from infllm_b200 import _lib

pytestmark = pytest.mark.gpu


class PlainCache:
    """dict-ordered LRU of (id -> stamp), capacity slots, as the reference keeps it."""

    def __init__(self, cap):
        self.cap, self.lru, self.slot_of = cap, {}, {}
        self.free = list(range(cap - 1, -1, -1))
        self.count = self.hits = self.misses = 0

    def refill(self, owned):
        self.count += 1
        if not owned:
            return []
        need = sum(1 for b in owned if b not in self.slot_of)
        evict = []
        if need > len(self.free):
            for b, _ in sorted(((b, s) for b, s in self.lru.items() if b not in owned), key=lambda x: x[1]):
                evict.append(b)
                if len(evict) == need - len(self.free):
                    break
        for b in evict:
            self.free.append(self.slot_of.pop(b))
            del self.lru[b]
        loaded = []
        for b in owned:
            self.lru[b] = self.count
            if b in self.slot_of:
                self.hits += 1
                continue
            self.misses += 1
            self.slot_of[b] = self.free.pop()
            loaded.append(b)
        return loaded


def test_refill_matches_the_plain_cache():
    dev = torch.device("cuda:0")
    lo, n_owned, cap, topk, unit = 100, 40, 8, 6, 1024
    rng = np.random.default_rng(3)
    store = torch.arange(n_owned * unit // 2, dtype=torch.int16).view(n_owned, unit // 2).pin_memory()
    cache = torch.zeros((cap, unit // 2), dtype=torch.int16, device=dev)
    slot_table = torch.full((n_owned,), -1, dtype=torch.int32, device=dev)
    ptr_table = (store.data_ptr() + torch.arange(n_owned, dtype=torch.int64) * unit).to(dev)
    slot_arr = np.full((n_owned,), -1, dtype=np.int32)
    free_arr = np.arange(cap - 1, -1, -1, dtype=np.int32)
    lru = ctypes.c_void_p()
    _lib.check(_lib.lib.infllm_lru_create(cap, ctypes.byref(lru)))
    cs = _lib.ShardCache()
    cs.lru, cs.slot_of, cs.free_slots, cs.n_free = lru, slot_arr.ctypes.data, free_arr.ctypes.data, cap
    cs.id_lo, cs.n_owned, cs.unit_bytes = lo, n_owned, unit
    cs.d_cache, cs.h_units = cache.data_ptr(), store.data_ptr()
    cs.d_slot_table, cs.d_ptr_table = slot_table.data_ptr(), ptr_table.data_ptr()
    plain = PlainCache(cap)
    stream = _lib.stream_ptr()
    try:
        for step in range(60):
            # a retrieval: some of this shard's units, some of a neighbour's, a hole
            ids = rng.choice(np.arange(lo - 20, lo + n_owned + 20), size=topk, replace=False).astype(np.int32)
            if step % 7 == 0:
                ids[0] = -1
            arr = (ctypes.c_int32 * topk)(*ids.tolist())
            _lib.check(_lib.lib.infllm_shard_refill(ctypes.byref(cs), arr, topk, stream))
            plain.refill([int(b) for b in ids if lo <= b < lo + n_owned])
            torch.cuda.synchronize()
            got = {lo + int(i): int(slot_arr[i]) for i in np.nonzero(slot_arr >= 0)[0]}
            assert got == plain.slot_of, step
            assert cs.n_free == len(plain.free) and free_arr[:cs.n_free].tolist() == plain.free
            assert (cs.load_count, cs.hits, cs.misses) == (plain.count, plain.hits, plain.misses)
            n = ctypes.c_int()
            l_ids, l_st = (ctypes.c_int32 * cap)(), (ctypes.c_double * cap)()
            _lib.check(_lib.lib.infllm_lru_items(lru, l_ids, l_st, cap, ctypes.byref(n)))
            assert [(l_ids[i], l_st[i]) for i in range(n.value)] == [(b, float(s)) for b, s in plain.lru.items()]
            st, pt = slot_table.cpu().numpy(), ptr_table.cpu().numpy()
            assert st.tolist() == slot_arr.tolist()
            for i in range(n_owned):
                want = cache.data_ptr() + int(slot_arr[i]) * unit if slot_arr[i] >= 0 else store.data_ptr() + i * unit
                assert int(pt[i]) == want
            for b, slot in plain.slot_of.items():
                assert torch.equal(cache[slot].cpu(), store[b - lo])
    finally:
        _lib.lib.infllm_lru_destroy(lru)


def test_more_ids_than_the_call_takes_is_refused():
    cs = _lib.ShardCache()
    lru = ctypes.c_void_p()
    _lib.check(_lib.lib.infllm_lru_create(4, ctypes.byref(lru)))
    a, f = np.full((4,), -1, dtype=np.int32), np.arange(4, dtype=np.int32)
    cs.lru, cs.slot_of, cs.free_slots, cs.n_free, cs.n_owned = lru, a.ctypes.data, f.ctypes.data, 4, 4
    ids = (ctypes.c_int32 * 300)()
    try:
        assert _lib.lib.infllm_shard_refill(ctypes.byref(cs), ids, 300, None) == _lib.E_BADARG
    finally:
        _lib.lib.infllm_lru_destroy(lru)
