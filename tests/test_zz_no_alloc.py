"""The allocation-free decode entry point against the ordinary one.

infllm_attn_decode_noalloc keeps its split-K partials in a scratch array built into the library, for
callers that cannot get device memory at call time (an engine that has claimed the whole GPU, a plugin
that must not allocate inside a step).  The scratch is shared by all calls and keeps the previous
call's contents, so the check runs twice in a row — the second time with fewer keys than the first,
where stale partials would show.  This file sorts last on purpose: with `-x` every other test has
already run when it starts, and it must also pass alone in a fresh process."""
import ctypes

import pytest
import torch

from helpers import MAX_ABS_TOL, MEAN_ABS_TOL
from oracle import infllm_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _decode_both(L, H, HKV, seg_lens, seed):
    D = 128
    g = torch.Generator().manual_seed(seed)
    q0 = torch.randn(H, D, generator=g).to(torch.bfloat16).to(DEV)
    q1 = torch.randn(H, D, generator=g).to(torch.bfloat16).to(DEV)
    ks = [torch.randn(HKV, n, D, generator=g).to(torch.bfloat16).to(DEV) for n in seg_lens]
    vs = [torch.randn(HKV, n, D, generator=g).to(torch.bfloat16).to(DEV) for n in seg_lens]
    n = len(seg_lens)
    arr = lambda t, xs: (t * n)(*xs)  # noqa: E731
    seg_k, seg_v = arr(ctypes.c_void_p, [k.data_ptr() for k in ks]), arr(ctypes.c_void_p, [v.data_ptr() for v in vs])
    seg_hs, seg_len = arr(ctypes.c_int64, [x * D for x in seg_lens]), arr(ctypes.c_int32, seg_lens)
    seg_q = arr(ctypes.c_int32, [0] + [1] * (n - 1))
    # existing path: caller-provided partial buffers, then the merge
    mp = int(L.lib.infllm_attn_decode_max_parts(n, sum(seg_lens)))
    part_o = torch.empty(mp, H, D, dtype=torch.float32, device=DEV)
    part_lse = torch.empty(mp, H, dtype=torch.float32, device=DEV)
    nparts = ctypes.c_int()
    L.check(L.lib.infllm_attn_decode(q0.data_ptr(), q1.data_ptr(), H, HKV, D, n, seg_k, seg_v, seg_hs, seg_len, seg_q,
                                     part_o.data_ptr(), part_lse.data_ptr(), mp, ctypes.byref(nparts), -1, None,
                                     L.BF16, L.stream_ptr()))
    want = torch.empty(H, D, dtype=torch.bfloat16, device=DEV)
    want_lse = torch.empty(H, dtype=torch.float32, device=DEV)
    L.check(L.lib.infllm_lse_merge(part_o.data_ptr(), part_lse.data_ptr(), nparts.value, H, D, want.data_ptr(), D,
                                   want_lse.data_ptr(), L.BF16, L.stream_ptr()))
    # the allocation-free entry point: inputs and outputs only
    got = torch.empty(H, D, dtype=torch.bfloat16, device=DEV)
    got_lse = torch.empty(H, dtype=torch.float32, device=DEV)
    call = lambda: L.check(L.lib.infllm_attn_decode_noalloc(  # noqa: E731
        q0.data_ptr(), q1.data_ptr(), H, HKV, D, n, seg_k, seg_v, seg_hs, seg_len, seg_q, got.data_ptr(), D,
        got_lse.data_ptr(), L.BF16, L.stream_ptr()))
    call()  # the first call on a device looks the scratch address up (and makes the module resident)
    torch.cuda.synchronize()
    before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    got.zero_()
    call()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before, "torch's allocator was used"
    assert torch.cuda.mem_get_info()[0] == free_before, "the device's free memory changed: something allocated"
    # the CPU oracle on the same inputs: first segment with the local query, the others with the global one
    stages = [O.Stage((q0 if i == 0 else q1).float().cpu()[:, None, :], k.float().cpu(), v.float().cpu())
              for i, (k, v) in enumerate(zip(ks, vs))]
    ora, _ = O.multi_stage_attention(stages)
    return got.float().cpu(), want.float().cpu(), got_lse.cpu(), want_lse.cpu(), ora[:, 0, :]


def test_noalloc_decode_matches_the_buffered_entry_point_twice_in_a_row():
    from infllm_b200 import _lib as L

    for seed, (H, HKV, seg_lens) in enumerate([(32, 8, [4096, 128, 128, 128, 128, 77, 300]), (8, 2, [200, 128, 5])]):
        got, want, got_lse, want_lse, ora = _decode_both(L, H, HKV, seg_lens, 100 + seed)
        for ref in (want, ora):  # the buffered entry point (same kernels) and the CPU oracle
            diff = (got - ref).abs()
            assert diff.max().item() <= MAX_ABS_TOL and diff.mean().item() <= MEAN_ABS_TOL
        torch.testing.assert_close(got_lse, want_lse, atol=1e-4, rtol=1e-5)


def test_noalloc_decode_rejects_sizes_beyond_its_scratch():
    from infllm_b200 import _lib as L

    D = 128
    q = torch.zeros(8, D, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(2, 128 * 161, D, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(8, D, dtype=torch.bfloat16, device=DEV)
    one = lambda t, x: (t * 1)(x)  # noqa: E731
    rc = L.lib.infllm_attn_decode_noalloc(q.data_ptr(), q.data_ptr(), 8, 2, D, 1, one(ctypes.c_void_p, k.data_ptr()),
                                          one(ctypes.c_void_p, k.data_ptr()), one(ctypes.c_int64, 128 * 161 * D),
                                          one(ctypes.c_int32, 128 * 161), one(ctypes.c_int32, 0), out.data_ptr(), D,
                                          None, L.BF16, L.stream_ptr())
    assert rc == L.E_CAPACITY
    assert b"160 chunks" in L.lib.infllm_last_error()
    qq = torch.zeros(65, D, dtype=torch.bfloat16, device=DEV)
    rc = L.lib.infllm_attn_decode_noalloc(qq.data_ptr(), qq.data_ptr(), 65, 65, D, 1, one(ctypes.c_void_p, k.data_ptr()),
                                          one(ctypes.c_void_p, k.data_ptr()), one(ctypes.c_int64, 128 * D),
                                          one(ctypes.c_int32, 128), one(ctypes.c_int32, 0), out.data_ptr(), D, None,
                                          L.BF16, L.stream_ptr())
    assert rc == L.E_CAPACITY
