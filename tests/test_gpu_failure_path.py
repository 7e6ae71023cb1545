"""What happens when a peer never arrives at an exchange of the sharded decode.

Nothing here faults, traps or hangs a GPU: the wait kernel polls a flag word with a limit (two milliseconds in this
test); when the limit runs out it leaves 1 + the missing rank in an error word and returns, the kernels queued
behind it see the word and write nothing, and the context stays usable.  The missing peer is simply a flag that
nobody sets (a two-rank mailbox of which only this rank exists)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_wait_for_a_peer_that_never_posts_runs_out_and_voids_what_follows():
    from infllm_b200 import _lib as L

    topk, world = 4, 2
    handle_bytes = int(L.lib.infllm_mailbox_handle_bytes())
    mine = (ctypes.c_ubyte * handle_bytes)()
    mb = ctypes.c_void_p()
    flag_off, cand_off, cand_slot = 0, 512, 2 * topk * 4
    L.check(L.lib.infllm_mailbox_create(4096, 0, world, mine, ctypes.byref(mb)))  # rank 0 of 2; rank 1 does not exist
    try:
        local = int(L.lib.infllm_mailbox_local(mb))
        seq = 7
        # this rank's own flag shows the sequence number (as its own put would have left it); rank 1's never will
        own = (ctypes.c_int32 * 1)(seq)
        L.check(L.lib.infllm_unit_fetch(local + flag_off, own, 4, L.stream_ptr()))  # a 4-byte host-to-device copy
        torch.cuda.synchronize()
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        any_miss = torch.zeros(1, dtype=torch.int32, device=DEV)
        ids = torch.full((topk,), 123, dtype=torch.int32, device=DEV)
        out = torch.full((8, 128), 5.0, dtype=torch.bfloat16, device=DEV)
        lse = torch.full((8,), 5.0, dtype=torch.float32, device=DEV)
        parts = torch.zeros((world, 8 * 129 + 4), dtype=torch.float32, device=DEV)
        st = L.stream_ptr()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        L.check(L.lib.infllm_mailbox_wait(mb, flag_off, seq, 2000, err.data_ptr(), 0, 0, -1, any_miss.data_ptr(), None, st))
        t1.record()
        # queued behind the wait: the global top-k and the final merge, both told where the error word is
        L.check(L.lib.infllm_topk_pairs(local + cand_off, cand_slot // 4, world, topk, ids.data_ptr(), err.data_ptr(), st))
        L.check(L.lib.infllm_lse_merge_ex(parts.data_ptr(), parts.stride(0), parts.data_ptr() + 8 * 128 * 4, parts.stride(0),
                                          world, 8, 128, out.data_ptr(), 128, lse.data_ptr(), L.BF16, None, 0, None, 0,
                                          any_miss.data_ptr(), st))
        torch.cuda.synchronize()
        assert err.item() == 2, "1 + the rank whose flag never showed the sequence number"
        assert 1.0 <= t0.elapsed_time(t1) <= 50.0, "the wait gave up after about its limit of 2 ms"
        assert any_miss.item() == 1
        assert (ids == -1).all(), "no retrieval is published after a failed exchange"
        assert (out == 5.0).all() and (lse == 5.0).all(), "the merge behind a failed exchange writes nothing"
        # the context is intact: an ordinary call right after succeeds
        q = torch.randn(8, 128, device=DEV).to(torch.bfloat16)
        k = torch.randn(2, 300, 128, device=DEV).to(torch.bfloat16)
        v = torch.randn(2, 300, 128, device=DEV).to(torch.bfloat16)
        one = lambda t, x: (t * 1)(x)  # noqa: E731
        good = torch.empty(8, 128, dtype=torch.bfloat16, device=DEV)
        L.check(L.lib.infllm_attn_decode_noalloc(q.data_ptr(), q.data_ptr(), 8, 2, 128, 1, one(ctypes.c_void_p, k.data_ptr()),
                                                 one(ctypes.c_void_p, v.data_ptr()), one(ctypes.c_int64, 300 * 128),
                                                 one(ctypes.c_int32, 300), one(ctypes.c_int32, 0), good.data_ptr(), 128, None,
                                                 L.BF16, st))
        torch.cuda.synchronize()
        kk = k.float().repeat_interleave(4, dim=0)
        p = torch.softmax(torch.einsum("hd,hnd->hn", q.float(), kk) / 128 ** 0.5, dim=-1)
        want = torch.einsum("hn,hnd->hd", p, v.float().repeat_interleave(4, dim=0))
        assert (good.float() - want).abs().max().item() < 2e-2
    finally:
        L.lib.infllm_mailbox_destroy(mb)


def test_a_token_whose_peer_never_posts_gives_up_twice_and_leaves_the_memory_usable():
    """The product path itself (infllm_shard_token_run with its flag-in-data exchanges): rank 0 of a two-rank sharding
    whose rank 1 is a zeroed buffer of this process that nobody ever writes into.  Both polls of the token run out
    after their limit (2 ms each), the error word names rank 1, no retrieval is published and the output buffer is
    not written; the host raises at the next settle and an ordinary kernel call works afterwards."""
    from infllm_b200 import _lib as L
    from infllm_b200.attention import RotaryEmbeddingESM, ShardedDecodeMemory, UnitRangeShard, unit_range

    H, HKV, D, UNITS, topk = 8, 2, 128, 40, 4
    dev = torch.device(DEV)
    g = torch.Generator().manual_seed(5)
    bf = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16)  # noqa: E731
    units, block_k = bf(UNITS, 2, HKV, 128, D), bf(UNITS, H * D)
    lo, hi = unit_range(UNITS, 0, 2)
    sh = UnitRangeShard(0, 2, RotaryEmbeddingESM(D, 1e6, 1.0), 128, 512, 128, 6, topk, 4, H, HKV, D, torch.bfloat16, dev,
                        spare_units=1)
    sh.load_synthetic(UNITS, units[lo:hi], block_k[lo:hi], bf(HKV, 128, D), bf(HKV, 128, D), bf(HKV, 512, D), bf(HKV, 512, D))

    class Box:  # what PeerMailbox describes, without its collective constructor
        pass

    mb = Box()
    mb.rank, mb.world, mb.wait_us, mb.seq = 0, 2, 2000, 0
    mb.flag1, mb.flag2, mb.cand_off, mb.cand_bytes = 0, 256, 512, 2 * topk * 4
    mb.cand_slot = (mb.cand_bytes + 15) // 16 * 16
    mb.part_off = (mb.cand_off + 2 * mb.cand_slot + 255) // 256 * 256
    mb.part_bytes = (H * (D + 1) + 4) * 4
    mb.part_slot = (mb.part_bytes + 15) // 16 * 16
    mb.miss_off = H * (D + 1) * 4
    mb.ll_cand_off = (mb.part_off + 2 * mb.part_slot + 255) // 256 * 256
    mb.ll_cand_slot = 2 * topk * 8
    mb.ll_part_off = (mb.ll_cand_off + 2 * mb.ll_cand_slot + 255) // 256 * 256
    mb.ll_part_slot = mb.part_bytes // 4 * 8
    total = mb.ll_part_off + 2 * mb.ll_part_slot
    mine = (ctypes.c_ubyte * int(L.lib.infllm_mailbox_handle_bytes()))()
    mb.handle = ctypes.c_void_p()
    L.check(L.lib.infllm_mailbox_create(total, 0, 2, mine, ctypes.byref(mb.handle)))
    absent = torch.zeros(total, dtype=torch.uint8, device=dev)  # "rank 1": receives this rank's puts, never posts
    try:
        L.check(L.lib.infllm_mailbox_alias(mb.handle, 1, absent.data_ptr()))
        mb.local = int(L.lib.infllm_mailbox_local(mb.handle))
        mem = ShardedDecodeMemory([sh], distributed=True, mailbox=mb)
        mem.distributed = True
        q, k, v = bf(H, 1, D).to(dev), bf(HKV, 1, D).to(dev), bf(HKV, 1, D).to(dev)
        mb.seq = 1  # past the first-exchange barrier of a real process group: there is none here
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        out = mem.append(q, k, v)
        t1.record()
        torch.cuda.synchronize()
        assert 3.0 <= t0.elapsed_time(t1) <= 200.0, "two polls of about 2 ms each, then the token ended"
        status = sh.h_status.tolist()
        assert status[topk] == 2, "1 + the rank whose words never carried the sequence number"
        assert all(b == -1 for b in status[:topk]), "no retrieval is published after a failed exchange"
        assert int(absent.view(torch.int64)[mb.ll_cand_off // 8].item()) >> 32 == 2, "this rank's own put went out"
        with pytest.raises(L.InfLLMError):
            mem.last_ids  # noqa: B018  (the settle reads the status words)
        # the device is intact: an ordinary call right after succeeds
        del out
        x = torch.randn(8, 128, device=dev).to(torch.bfloat16)
        kk, vv = torch.randn(2, 300, 128, device=dev).to(torch.bfloat16), torch.randn(2, 300, 128, device=dev).to(torch.bfloat16)
        one = lambda t, y: (t * 1)(y)  # noqa: E731
        good = torch.empty(8, 128, dtype=torch.bfloat16, device=dev)
        L.check(L.lib.infllm_attn_decode_noalloc(x.data_ptr(), x.data_ptr(), 8, 2, 128, 1, one(ctypes.c_void_p, kk.data_ptr()),
                                                 one(ctypes.c_void_p, vv.data_ptr()), one(ctypes.c_int64, 300 * 128),
                                                 one(ctypes.c_int32, 300), one(ctypes.c_int32, 0), good.data_ptr(), 128, None,
                                                 L.BF16, L.stream_ptr()))
        torch.cuda.synchronize()
        assert torch.isfinite(good.float()).all()
    finally:
        L.lib.infllm_mailbox_destroy(mb.handle)
