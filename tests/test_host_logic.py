"""CPU-only checks: the C-ABI library loads and exports what the header declares, argument
validation of the context memory, and the native LRU table against the oracle's."""
import ctypes
import os
import random
import re

import pytest
import torch

from oracle import infllm_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from infllm_b200 import _lib

    return _lib


def test_library_exports_every_declared_symbol():
    L = _lib()
    header = open(os.path.join(ROOT, "include", "infllm_b200.h")).read()
    declared = set(re.findall(r"\b(infllm_[a-z0-9_]+)\s*\(", header))
    declared -= {"infllm_ctx", "infllm_lru", "infllm_config", "infllm_ctx_info"}
    assert declared, "no declarations parsed"
    for name in sorted(declared):
        assert hasattr(L.lib, name), f"{name} is declared in the header but not exported"
        assert name in L.SIGNATURES, f"{name} has no ctypes signature"
    assert set(L.SIGNATURES) <= declared, f"bound but undeclared: {set(L.SIGNATURES) - declared}"
    assert b"sm_100a" in L.lib.infllm_version()


def _cfg(L, **kw):
    base = dict(n_heads=8, n_kv_heads=2, head_dim=128, n_init=128, n_local=512, block_size=128, max_cached_block=8,
                topk=4, exc_block_size=128, repr_topk=4, cache_strategy=L.CACHE_LRU, dtype=L.BF16, score_decay=0.0,
                rope_base=1e6, rope_scale=1.0, device=0, shard_rank=0, shard_world=1)
    base.update(kw)
    return L.Config(**base)


def test_ctx_create_validates_like_the_reference():
    L = _lib()
    h = ctypes.c_void_p()
    assert L.lib.infllm_ctx_create(ctypes.byref(_cfg(L)), ctypes.byref(h)) == L.OK
    assert L.lib.infllm_ctx_destroy(h) == L.OK
    # exc_block_size > n_local: the reference asserts in __init__
    assert L.lib.infllm_ctx_create(ctypes.byref(_cfg(L, exc_block_size=1024)), ctypes.byref(h)) == L.E_BADARG
    # max_cached_block < topk: the reference dies in CudaCache.alloc; here it is a capacity error up front
    rc = L.lib.infllm_ctx_create(ctypes.byref(_cfg(L, max_cached_block=8, topk=16)), ctypes.byref(h))
    assert rc == L.E_CAPACITY
    with pytest.raises(AssertionError):
        L.check(rc)
    assert b"max_cached_block" in L.lib.infllm_last_error()
    assert L.lib.infllm_ctx_create(ctypes.byref(_cfg(L, n_heads=6, n_kv_heads=4)), ctypes.byref(h)) == L.E_BADARG
    assert L.lib.infllm_ctx_create(ctypes.byref(_cfg(L, head_dim=96)), ctypes.byref(h)) == L.E_UNSUPPORTED
    assert L.lib.infllm_ctx_create(ctypes.byref(_cfg(L, dtype=7)), ctypes.byref(h)) == L.E_UNSUPPORTED


def test_decode_attention_rejects_zero_kv_heads():
    """Argument checks come before any division by the head counts and before any launch (no GPU needed)."""
    L = _lib()
    one = lambda t, x: (t * 1)(x)  # noqa: E731
    n = ctypes.c_int()
    for heads, kv in ((8, 0), (0, 2), (8, -1)):
        rc = L.lib.infllm_attn_decode(1 << 20, 1 << 20, heads, kv, 128, 1, one(ctypes.c_void_p, 1 << 20),
                                      one(ctypes.c_void_p, 1 << 20), one(ctypes.c_int64, 128 * 128), one(ctypes.c_int32, 128),
                                      one(ctypes.c_int32, 0), 1 << 20, 1 << 20, 4, ctypes.byref(n), -1, None, L.BF16, None)
        assert rc == L.E_BADARG, (heads, kv)


def _saved_header(L, **kw):
    """A header as infllm_ctx_save writes it for _cfg(L), with fields overridden."""
    import struct

    f = dict(magic=0x324d454d4c464e49, H=8, HKV=2, D=128, n_init=128, n_local=512, bs=128, dtype=L.BF16, length=128 + 128 + 512,
             frontier=256, n_units=1, init_len=128, init_full=1, load_count=3, n_lru=1, strategy=L.CACHE_LRU, max_cached=8,
             topk=4, exc=128, repr_topk=4, chunk=0, decay=0, pad0=0, pad1=0)
    f.update(kw)
    return struct.pack("<24q", *f.values()), f


def _saved_file(L, path, lru=((0, 3.0),), truncate=0, **kw):
    import struct

    hdr, f = _saved_header(L, **kw)
    live = f["length"] - f["frontier"]
    unit = 2 * f["HKV"] * f["bs"] * f["D"] * 2
    body = b"".join(struct.pack("<qd", i, s) for i, s in lru)
    body += bytes(2 * f["HKV"] * f["init_len"] * f["D"] * 2 + f["n_units"] * f["H"] * f["D"] * 2
                  + 2 * f["HKV"] * live * f["D"] * 2 + f["H"] * live * 4 + f["n_units"] * unit)
    data = hdr + body
    with open(path, "wb") as fh:
        fh.write(data[:len(data) - truncate] if truncate else data)


@pytest.mark.parametrize("why,kw", [
    ("not a saved context memory", dict(magic=1)),
    ("another configuration", dict(topk=5)),
    ("another configuration", dict(max_cached=16)),
    ("inconsistent lengths", dict(frontier=300)),
    ("inconsistent lengths", dict(length=100)),
    ("inconsistent lengths", dict(init_len=200)),
    ("cached units", dict(n_lru=9)),
    ("bytes its header implies", dict(truncate=100)),
    ("wrongly", dict(lru=((5, 3.0),))),
    ("wrongly", dict(n_lru=2, lru=((0, 3.0), (0, 4.0)))),
])
def test_ctx_load_refuses_corrupt_files_before_touching_anything(tmp_path, why, kw):
    """Every field of a saved memory is checked against the configuration and against the file's size before the
    context (or a GPU) is touched: these loads fail on a machine without a device."""
    L = _lib()
    h = ctypes.c_void_p()
    L.check(L.lib.infllm_ctx_create(ctypes.byref(_cfg(L)), ctypes.byref(h)))
    path = str(tmp_path / "mem.u0")
    _saved_file(L, path, **kw)
    assert L.lib.infllm_ctx_load(h, path.encode(), None) == L.E_BADARG
    assert why.encode() in L.lib.infllm_last_error(), L.lib.infllm_last_error()
    L.lib.infllm_ctx_destroy(h)


class _NativeLru:
    def __init__(self, L, cap):
        self.L, self.h = L, ctypes.c_void_p()
        L.check(L.lib.infllm_lru_create(cap, ctypes.byref(self.h)))

    def plan(self, wanted):
        arr = (ctypes.c_int32 * max(len(wanted), 1))(*wanted)
        ev, n = (ctypes.c_int32 * 4096)(), ctypes.c_int()
        self.L.check(self.L.lib.infllm_lru_plan(self.h, arr, len(wanted), ev, ctypes.byref(n)))
        return [int(ev[i]) for i in range(n.value)]

    def stamp(self, wanted, value):
        arr = (ctypes.c_int32 * max(len(wanted), 1))(*wanted)
        self.L.check(self.L.lib.infllm_lru_stamp(self.h, arr, len(wanted), float(value)))

    def items(self):
        ids, st, n = (ctypes.c_int32 * 4096)(), (ctypes.c_double * 4096)(), ctypes.c_int()
        self.L.check(self.L.lib.infllm_lru_items(self.h, ids, st, 4096, ctypes.byref(n)))
        return [(int(ids[i]), st[i]) for i in range(n.value)]

    def close(self):
        self.L.lib.infllm_lru_destroy(self.h)


def test_native_lru_tie_order_example():
    L = _lib()
    t = _NativeLru(L, 4)
    for bid, s in ((7, 3), (2, 3), (9, 1), (5, 3)):
        t.stamp([bid], s)
    assert t.plan([5, 11, 12, 13]) == [9, 7, 2]
    assert t.items() == [(5, 3.0)]
    t.close()


@pytest.mark.parametrize("seed", range(6))
def test_native_lru_matches_oracle_on_random_traffic(seed):
    L = _lib()
    rng = random.Random(seed)
    cap, k = rng.choice([(4, 4), (8, 3), (16, 5), (32, 16)])
    nat, ora = _NativeLru(L, cap), O.LruTable(cap)
    universe = rng.randint(k + 1, 4 * cap)
    clock = 0
    for step in range(300):
        wanted = rng.sample(range(universe), k)
        assert nat.plan(wanted) == ora.plan(wanted), f"step {step}"
        clock += 1
        stamp = clock if rng.random() < 0.8 else clock - rng.randint(0, 3)  # repeated stamps exercise the tie order
        nat.stamp(wanted, stamp)
        ora.stamp(wanted, stamp)
        assert nat.items() == [(b, float(s)) for b, s in ora.entries.items()]
    nat.close()


def test_python_layer_rejects_cpu_tensors_and_fp32():
    from infllm_b200.attention import ContextManager, RotaryEmbeddingESM

    pe = RotaryEmbeddingESM(128, 10000, 1.0)
    with pytest.raises(AssertionError):
        ContextManager(pe, 128, 512, 128, 8, 4, 1024)  # exc_block_size > n_local
    cm = ContextManager(pe, 128, 512, 128, 8, 4, 128)
    q = torch.zeros(1, 8, 4, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        cm.append(q, q[:, :2], q[:, :2], q, q[:, :2], q[:, :2])
    assert cm.size() == 0


def test_oracle_is_invariant_to_how_a_prompt_is_split_into_appends():
    """The native loop cuts long appends at exec-block boundaries; the algorithm must not care."""
    g = torch.Generator().manual_seed(3)
    H, HKV, D, L = 4, 2, 32, 640
    q, k, v = torch.randn(H, L, D, generator=g), torch.randn(HKV, L, D, generator=g), torch.randn(HKV, L, D, generator=g)
    mk = lambda: O.OracleContextMemory(16, 64, 16, 6, 3, 32, 2, 10000.0, 1.0)  # noqa: E731
    a, b = mk(), mk()
    oa = a.append(q, k, v)
    ob = torch.cat([b.append(q[:, s:s + 160], k[:, s:s + 160], v[:, s:s + 160]) for s in range(0, L, 160)], dim=1)
    assert [t.topk_raw for t in a.trace] == [t.topk_raw for t in b.trace]
    assert [t.cached_after for t in a.trace] == [t.cached_after for t in b.trace]
    torch.testing.assert_close(oa, ob, atol=1e-6, rtol=0)


def test_shard_refill_argument_checks_and_foreign_ids_need_no_device():
    """infllm_shard_refill: bad arguments are refused, and a retrieval that names only other ranks' units (or holes)
    counts the load and touches nothing else — no device call is made for it."""
    import numpy as np

    from infllm_b200 import _lib as L

    lru = ctypes.c_void_p()
    L.check(L.lib.infllm_lru_create(4, ctypes.byref(lru)))
    try:
        slots, free = np.full((8,), -1, dtype=np.int32), np.arange(3, -1, -1, dtype=np.int32)
        cs = L.ShardCache()
        cs.lru, cs.slot_of, cs.free_slots, cs.n_free = lru, slots.ctypes.data, free.ctypes.data, 4
        cs.id_lo, cs.n_owned, cs.unit_bytes = 100, 8, 1024
        ids = (ctypes.c_int32 * 4)(-1, 3, 99, 108)  # a hole, and ids below and above [100, 108)
        assert L.lib.infllm_shard_refill(ctypes.byref(cs), ids, 4, None) == L.OK
        assert (cs.load_count, cs.hits, cs.misses, cs.n_free) == (1, 0, 0, 4)
        assert (slots == -1).all()
        assert L.lib.infllm_shard_refill(None, ids, 4, None) == L.E_BADARG
        assert L.lib.infllm_shard_refill(ctypes.byref(cs), None, 4, None) == L.E_BADARG
        big = (ctypes.c_int32 * 300)()
        assert L.lib.infllm_shard_refill(ctypes.byref(cs), big, 300, None) == L.E_BADARG
        cs.lru = None
        assert L.lib.infllm_shard_refill(ctypes.byref(cs), ids, 4, None) == L.E_BADARG
    finally:
        L.lib.infllm_lru_destroy(lru)
