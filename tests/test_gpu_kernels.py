"""GPU parity of the individual kernels, called through the C ABI, against the CPU oracle."""
import ctypes
import os

import numpy as np
import pytest
import torch

import cases as C
from helpers import GOLDEN, MAX_ABS_TOL, MEAN_ABS_TOL
from oracle import infllm_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _L():
    from infllm_b200 import _lib

    return _lib


def _check_out(got, want, what=""):
    diff = (got.float().cpu() - want.float()).abs()
    assert diff.max().item() <= MAX_ABS_TOL, f"{what} max-abs {diff.max().item():.4g}"
    assert diff.mean().item() <= MEAN_ABS_TOL, f"{what} mean-abs {diff.mean().item():.4g}"


# ----------------------------------------------------------------------------------------- RoPE
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rope_matches_oracle(dtype):
    from infllm_b200.attention import RotaryEmbeddingESM

    q, k = C.rope_inputs()
    q, k = q.to(dtype), k.to(dtype)
    pe = RotaryEmbeddingESM(128, 1000000.0, 1.0)
    rq, rk = pe(q[None].to(DEV), k[None].to(DEV))
    wq, wk = O.rope_local(q, k, 128, 1000000.0, 1.0)
    one = pe.apply_rotary_pos_emb_one_angle(q[None].to(DEV), 4096)
    wone = O.rope_one_angle(q, 4096, 128, 1000000.0, 1.0)
    eps = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    for got, want in ((rq[0], wq), (rk[0], wk), (one[0], wone)):
        g, w = got.float().cpu(), want.float()
        # device cos/sin may differ from the host's in the last place: at most one rounding step apart
        assert ((g - w).abs() <= eps * w.abs().clamp_min(1e-3) * 1.01).all()
        assert (g == w).float().mean() > 0.98


def test_rope_views_and_fresh_golden():
    """Strided (token-major) input views give the same result as contiguous ones."""
    from infllm_b200.attention import RotaryEmbeddingESM

    g = torch.Generator().manual_seed(5)
    x = torch.randn(1, 37, 4, 128, generator=g).to(torch.bfloat16).to(DEV)  # (B, L, H, D)
    pe = RotaryEmbeddingESM(128, 10000.0, 1.0)
    a = pe.apply_rotary_pos_emb_one_angle(x.permute(0, 2, 1, 3), 77)
    b = pe.apply_rotary_pos_emb_one_angle(x.permute(0, 2, 1, 3).contiguous(), 77)
    assert torch.equal(a, b)


# ------------------------------------------------------------------------ multi-stage attention
@pytest.mark.parametrize("ci", [i for i, s in enumerate(C.MULTI_STAGE_SPECS) if s[2] in (64, 128)])
def test_multi_stage_attention_matches_oracle_and_golden(ci):
    from infllm_b200.attention import CudaMultiStageDotProductionAttention

    H, HKV, D, Lq, stages = C.MULTI_STAGE_SPECS[ci]
    tensors = C.multi_stage_inputs(ci)
    want, want_scores = O.multi_stage_attention(
        [O.Stage(q, k, v, sw, comp, gs) for (q, k, v), (_, sw, comp, gs) in zip(tensors, stages)])
    z = np.load(os.path.join(GOLDEN, "multi_stage.npz"))
    np.testing.assert_allclose(want.numpy(), z[f"c{ci}_ret"], atol=1e-5)  # the oracle itself is pinned
    att = CudaMultiStageDotProductionAttention((1, H, Lq, D), torch.bfloat16, DEV)
    for si, ((q, k, v), (_, sw, comp, gs)) in enumerate(zip(tensors, stages)):
        att.append(q[None].to(torch.bfloat16).to(DEV), k[None].to(torch.bfloat16).to(DEV),
                   v[None].to(torch.bfloat16).to(DEV), sliding_window=sw, complement_sliding_window=comp,
                   end=(si == len(stages) - 1), get_score=gs)
    ret, scores = att.get_result()
    _check_out(ret[0], want, f"case {ci}")
    for si, (s, ws) in enumerate(zip(att.score_list_fp32, want_scores)):
        assert (s is None) == (ws is None)
        if ws is not None:
            # a score is a sum of up to Lq probabilities: relative tolerance on top of the absolute one
            torch.testing.assert_close(s[0].cpu(), ws, atol=2e-3, rtol=2e-2)


@pytest.mark.parametrize("lq,lk,window", [(1, 1, 4), (64, 64, 64), (65, 200, 100), (200, 777, 128), (128, 4224, 4096)])
def test_attention_ragged_shapes_with_strided_views(lq, lk, window):
    """Token-major (B, L, H, D) projections viewed head-major, GQA, causal window; sizes around the tile edges."""
    from infllm_b200.attention import CudaMultiStageDotProductionAttention

    g = torch.Generator().manual_seed(lq * 1000 + lk)
    H, HKV, D = 4, 2, 128
    q = torch.randn(1, lq, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, lk, HKV, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, lk, HKV, D, generator=g).to(torch.bfloat16)
    att = CudaMultiStageDotProductionAttention((1, H, lq, D), torch.bfloat16, DEV)
    att.append(q.to(DEV).permute(0, 2, 1, 3), k.to(DEV).permute(0, 2, 1, 3), v.to(DEV).permute(0, 2, 1, 3),
               sliding_window=window, end=True, get_score=True)
    ret, _ = att.get_result()
    want, ws = O.multi_stage_attention([O.Stage(q[0].permute(1, 0, 2).float(), k[0].permute(1, 0, 2).float(),
                                                v[0].permute(1, 0, 2).float(), window, False, True)])
    _check_out(ret[0], want)
    torch.testing.assert_close(att.score_list_fp32[0][0].cpu(), ws[0], atol=2e-3, rtol=2e-2)
    # size-independent property: every query's probabilities sum to one, so the scores sum to the
    # number of queries that see at least one key
    visible = O.stage_mask(lq, lk, window, False).any(dim=1).sum().item()
    torch.testing.assert_close(att.score_list_fp32[0][0].sum(-1).cpu(), torch.full((H,), float(visible)), rtol=2e-3, atol=1e-2)


def test_attention_row_without_visible_keys_gives_zero():
    from infllm_b200.attention import CudaMultiStageDotProductionAttention

    H, D, lq, lk = 2, 128, 5, 9
    q = torch.ones(1, H, lq, D, dtype=torch.bfloat16, device=DEV)
    k = torch.ones(1, H, lk, D, dtype=torch.bfloat16, device=DEV)
    att = CudaMultiStageDotProductionAttention((1, H, lq, D), torch.bfloat16, DEV)
    # complement window that hides every key from the first rows
    att.append(q, k, k, sliding_window=(0, 3), complement_sliding_window=True, end=True, get_score=True)
    ret, sc = att.get_result()
    assert torch.isfinite(ret.float()).all()
    assert (ret[0, :, :3] == 0).all() and (ret[0, :, 3:] == 1).all()


# -------------------------------------------------------------------------- retrieval kernels
@pytest.mark.parametrize("n,k,width", [(5, 5, 1024), (40, 4, 4096), (991, 16, 4096), (8192, 32, 4096), (3000, 64, 512),
                                       (5000, 100, 512), (20000, 16, 256), (12345, 48, 512), (16384, 64, 256)])
def test_block_topk_matches_torch(n, k, width):
    L = _L()
    g = torch.Generator().manual_seed(n + k)
    bk = torch.randn(n, width, generator=g).to(torch.bfloat16)
    qbar = torch.randn(width, generator=g)
    want_scores = bk.float() @ qbar
    d_bk, d_q = bk.to(DEV), qbar.to(DEV)
    d_scores = torch.empty(n, dtype=torch.float32, device=DEV)
    d_ids = torch.empty(k, dtype=torch.int32, device=DEV)
    d_top = torch.empty(k, dtype=torch.float32, device=DEV)
    L.check(L.lib.infllm_block_topk(d_bk.data_ptr(), n, width, d_q.data_ptr(), d_scores.data_ptr(), k, 7,
                                    d_ids.data_ptr(), d_top.data_ptr(), L.BF16, L.stream_ptr()))
    torch.testing.assert_close(d_scores.cpu(), want_scores, rtol=1e-4, atol=1e-3)
    ids = (d_ids.cpu() - 7).tolist()
    # exact top-k of the scores the device computed, descending, ties to the lower id
    dev_scores = d_scores.cpu()
    order = sorted(range(n), key=lambda i: (-dev_scores[i].item(), i))[:k]
    assert ids == order
    assert torch.equal(d_top.cpu(), dev_scores[ids])
    from helpers import near_tie_ok

    assert near_tie_ok(want_scores.topk(k).indices.tolist(), ids, want_scores)


def test_block_topk_ties_go_to_lower_ids():
    L = _L()
    n, k, width = 300, 10, 256
    bk = torch.zeros(n, width, dtype=torch.bfloat16)
    bk[:, 0] = 1.0  # all scores equal
    bk[250, 0] = 2.0
    d_bk, d_q = bk.to(DEV), torch.ones(width, device=DEV)
    d_scores = torch.empty(n, dtype=torch.float32, device=DEV)
    d_ids = torch.empty(k, dtype=torch.int32, device=DEV)
    L.check(L.lib.infllm_block_topk(d_bk.data_ptr(), n, width, d_q.data_ptr(), d_scores.data_ptr(), k, 0,
                                    d_ids.data_ptr(), None, L.BF16, L.stream_ptr()))
    assert d_ids.cpu().tolist() == [250] + list(range(9))


@pytest.mark.parametrize("H,HKV,bs,r,n_new", [(8, 2, 128, 4, 3), (4, 4, 128, 1, 1), (32, 8, 128, 8, 4), (4, 1, 64, 2, 2)])
def test_repr_select_matches_reference_formula(H, HKV, bs, r, n_new):
    L = _L()
    D, cap, tok0 = 128, 1000, 137
    g = torch.Generator().manual_seed(H * 100 + r)
    k = torch.randn(HKV, cap, D, generator=g).to(torch.bfloat16)
    score = torch.rand(H, cap, generator=g)
    out = torch.empty(n_new, H * D, dtype=torch.bfloat16, device=DEV)
    d_k, d_s = k.to(DEV), score.to(DEV)
    L.check(L.lib.infllm_repr_select(d_k.data_ptr(), cap * D, D, d_s.data_ptr(), cap, tok0, n_new, bs, r, H, HKV, D,
                                     out.data_ptr(), L.BF16, L.stream_ptr()))
    kk = k.repeat_interleave(H // HKV, dim=0).float()
    for b in range(n_new):
        st = tok0 + b * bs
        idx = score[:, st:st + bs].topk(r, dim=-1).indices  # context_manager.py:274
        rep = torch.gather(kk[:, st:st + bs], 1, idx[:, :, None].expand(H, r, D)).mean(dim=1)
        want = rep.reshape(-1).to(torch.bfloat16)
        assert torch.equal(out[b].cpu(), want), f"block {b}"


# ------------------------------------------------------------------------------ decode attention
@pytest.mark.parametrize("H,HKV,seg_lens", [(8, 2, [300, 128, 128, 77]), (32, 8, [4096, 128, 128, 128, 128, 128, 5]),
                                            (4, 4, [1]), (8, 1, [129, 127])])
def test_decode_split_k_and_merge_match_oracle(H, HKV, seg_lens):
    L = _L()
    D = 128
    g = torch.Generator().manual_seed(sum(seg_lens) + H)
    q0 = torch.randn(H, 1, D, generator=g).to(torch.bfloat16)
    q1 = torch.randn(H, 1, D, generator=g).to(torch.bfloat16)
    ks = [torch.randn(HKV, n, D, generator=g).to(torch.bfloat16) for n in seg_lens]
    vs = [torch.randn(HKV, n, D, generator=g).to(torch.bfloat16) for n in seg_lens]
    qsel = [0] + [1] * (len(seg_lens) - 1)
    stages = [O.Stage((q1 if s else q0).float(), k.float(), v.float(), None, False, i == 0)
              for i, (s, k, v) in enumerate(zip(qsel, ks, vs))]
    want, wsc = O.multi_stage_attention(stages)
    dk, dv = [k.to(DEV) for k in ks], [v.to(DEV) for v in vs]
    n = len(seg_lens)
    mp = int(L.lib.infllm_attn_decode_max_parts(n, sum(seg_lens)))
    part_o = torch.empty(mp, H, D, dtype=torch.float32, device=DEV)
    part_lse = torch.empty(mp, H, dtype=torch.float32, device=DEV)
    logits = torch.empty(H, seg_lens[0], dtype=torch.float32, device=DEV)
    nparts = ctypes.c_int()
    arr = lambda t, xs: (t * n)(*xs)  # noqa: E731
    dq0, dq1 = q0.to(DEV), q1.to(DEV)
    L.check(L.lib.infllm_attn_decode(
        dq0.data_ptr(), dq1.data_ptr(), H, HKV, D, n, arr(ctypes.c_void_p, [k.data_ptr() for k in dk]),
        arr(ctypes.c_void_p, [v.data_ptr() for v in dv]), arr(ctypes.c_int64, [x * D for x in seg_lens]),
        arr(ctypes.c_int32, seg_lens), arr(ctypes.c_int32, qsel), part_o.data_ptr(), part_lse.data_ptr(), mp,
        ctypes.byref(nparts), 0, logits.data_ptr(), L.BF16, L.stream_ptr()))
    assert 1 <= nparts.value <= mp  # one partial per run of 16-key groups: two CTAs per SM, fewer for short lists
    out = torch.empty(H, D, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(H, dtype=torch.float32, device=DEV)
    L.check(L.lib.infllm_lse_merge(part_o.data_ptr(), part_lse.data_ptr(), nparts.value, H, D, out.data_ptr(), D,
                                   lse.data_ptr(), L.BF16, L.stream_ptr()))
    _check_out(out, want[:, 0])
    # exported logits + final lse reproduce the local-stage probabilities (the per-key score of a one-token block)
    p = torch.exp2(logits - lse[:, None]).cpu()
    torch.testing.assert_close(p, wsc[0], atol=1e-3, rtol=2e-2)
    # merging is associative: merge two halves, then merge the results
    if nparts.value >= 2:
        h1 = nparts.value // 2
        po = torch.empty(2, H, D, dtype=torch.float32, device=DEV)
        pl = torch.empty(2, H, dtype=torch.float32, device=DEV)
        tmp = torch.empty(H, D, dtype=torch.bfloat16, device=DEV)
        for i, (a, b) in enumerate(((0, h1), (h1, nparts.value))):
            L.check(L.lib.infllm_lse_merge(part_o[a:b].data_ptr(), part_lse[a:b].data_ptr(), b - a, H, D,
                                           tmp.data_ptr(), D, pl[i].data_ptr(), L.BF16, L.stream_ptr()))
            po[i] = tmp.float()
        out2 = torch.empty(H, D, dtype=torch.bfloat16, device=DEV)
        L.check(L.lib.infllm_lse_merge(po.data_ptr(), pl.data_ptr(), 2, H, D, out2.data_ptr(), D, None, L.BF16,
                                       L.stream_ptr()))
        _check_out(out2, want[:, 0])


def test_tensor_core_kernels_reported_no_timeout():
    """Collected after the kernel tests of this file: no bounded wait may have run out."""
    assert _L().device_error() == (0, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["infinite-lm", "stream-llm"])
def test_sink_window_attention_types_match_oracle(kind):
    """The reference's "infinite-lm" and "stream-llm" attention types on the CUDA kernels (window stage + sink stage
    with a complement mask that hides pairs), call by call against the CPU oracle."""
    import cases as C

    from infllm_b200.attention import ATTN_FORWRAD, RotaryEmbeddingESM
    from oracle.sink_window_oracle import SinkWindowMemory

    c = C.SINK_WINDOW
    pq, pk, pv, po = C.sink_window_projections()
    forward = ATTN_FORWRAD[kind](c["n_local"], c["n_init"], fattn=True)
    pe = RotaryEmbeddingESM(c["D"], c["base"], 1.0)
    mem = SinkWindowMemory(c["n_local"], c["n_init"], c["D"], c["base"], kind)
    past = None
    for i, x in enumerate(C.sink_window_inputs()):
        L = x.size(0)
        dx = x.to(DEV).to(torch.bfloat16)[None]
        o, past = forward(None, dx, dx, pe, True, past, pq, pk, pv, po, c["D"], c["H"], c["HKV"])
        q = pq(x).view(L, c["H"], c["D"]).permute(1, 0, 2)
        k = pk(x).view(L, c["HKV"], c["D"]).permute(1, 0, 2)
        v = pv(x).view(L, c["HKV"], c["D"]).permute(1, 0, 2)
        want = mem.append(q, k, v).permute(1, 0, 2).reshape(L, -1)
        diff = (o[0].float().cpu() - want).abs()
        assert diff.max().item() <= MAX_ABS_TOL and diff.mean().item() <= MEAN_ABS_TOL, f"{kind} call {i}"
    assert past[2] == mem.length == sum(c["lens"])
