"""The oracle against the vectors recorded from the reference itself (tests/golden/make_golden.py)."""
import json
import os

import numpy as np
import pytest
import torch

import cases as C
from helpers import GOLDEN, golden_cached, load_golden
from oracle import infllm_oracle as O


@pytest.mark.parametrize("name", sorted(C.CASES))
def test_context_memory_matches_reference(name):
    meta, z = load_golden(name)
    case = C.CASES[name]
    assert meta["case"] == json.loads(json.dumps(case)), "fixture was recorded for other parameters"
    inputs = C.make_inputs(case)
    assert C.inputs_digest(inputs) == meta["digest"], "input generator drifted; re-record the fixtures"
    mem = O.OracleContextMemory(case["n_init"], case["n_local"], case["bs"], case["max_cached"], case["topk"],
                                case["exc"], case["repr_topk"], case["base"], 1.0, case["strategy"], case["decay"],
                                chunk_topk_calc=case.get("chunk_topk"))
    outs = [mem.append(q, k, v).permute(1, 0, 2) for q, k, v in inputs]
    o = torch.cat(outs, dim=0)
    # retrieval order and LRU table of every exec block: exact
    assert len(mem.trace) == z["topk"].shape[0]
    for i, tr in enumerate(mem.trace):
        want = [int(x) for x in z["topk"][i] if x >= 0]
        assert tr.topk_raw == want, f"exec block {i}"
        got_c, want_c = tr.cached_after, golden_cached(z, i)
        assert [b for b, _ in got_c] == [b for b, _ in want_c], f"LRU order, exec block {i}"
        np.testing.assert_allclose([s for _, s in got_c], [s for _, s in want_c], rtol=1e-5, atol=1e-6)
    assert mem.num_blocks == meta["n_blocks"] and mem.init_len == meta["init_len"]
    assert mem.length == meta["length"] and mem.length - mem.frontier == meta["remainder_len"]
    # outputs: every row through the float64 projection, sampled rows in full
    np.testing.assert_allclose(C.project_rows(o).numpy(), z["o_proj"], rtol=0, atol=2e-4)
    rows = torch.from_numpy(z["o16_rows"])
    np.testing.assert_allclose(o[rows].numpy(), z["o16"].astype(np.float32), rtol=2e-3, atol=2e-3)
    if mem.num_blocks:
        np.testing.assert_allclose(C.project_rows(torch.stack(mem.block_k)).numpy(), z["block_k_proj"], atol=2e-4)


def test_multi_stage_attention_matches_reference():
    z = np.load(os.path.join(GOLDEN, "multi_stage.npz"))
    for ci, (H, HKV, D, Lq, stages) in enumerate(C.MULTI_STAGE_SPECS):
        tensors = C.multi_stage_inputs(ci)
        st = [O.Stage(q, k, v, sw, comp, gs) for (q, k, v), (_, sw, comp, gs) in zip(tensors, stages)]
        ret, scores = O.multi_stage_attention(st)
        np.testing.assert_allclose(ret.numpy(), z[f"c{ci}_ret"], atol=1e-5)
        for si, s in enumerate(scores):
            if s is None:
                assert f"c{ci}_score{si}" not in z
            else:
                np.testing.assert_allclose(s.numpy(), z[f"c{ci}_score{si}"], atol=1e-5)


def test_rope_matches_reference():
    z = np.load(os.path.join(GOLDEN, "multi_stage.npz"))
    q, k = C.rope_inputs()
    rq, rk = O.rope_local(q, k, 128, 1000000.0, 1.0)
    np.testing.assert_array_equal(rq.numpy(), z["rope_rq"])
    np.testing.assert_array_equal(rk.numpy(), z["rope_rk"])
    np.testing.assert_array_equal(O.rope_one_angle(q, 4096, 128, 1000000.0, 1.0).numpy(), z["rope_one"])


def test_lru_tie_order():
    """Ties at eviction fall back to dict insertion order (stable sort over items)."""
    t = O.LruTable(4)
    t.entries = {7: 3, 2: 3, 9: 1, 5: 3}
    assert t.plan([5, 11, 12, 13]) == [9, 7, 2]
    assert list(t.entries) == [5]


def test_perhead_matches_reference():
    """perhead=True: one oracle per query head (a unit of its own with the KV head of its group) against the
    reference's recording."""
    case = C.PERHEAD
    z = np.load(os.path.join(GOLDEN, "perhead.npz"))
    inputs = C.make_inputs(case)
    assert C.inputs_digest(inputs) == str(z["digest"])
    g = case["H"] // case["HKV"]
    mems = [O.OracleContextMemory(case["n_init"], case["n_local"], case["bs"], case["max_cached"], case["topk"],
                                  case["exc"], case["repr_topk"], case["base"], 1.0) for _ in range(case["H"])]
    outs = []
    for q, k, v in inputs:
        per_head = [mems[h].append(q[h:h + 1], k[h // g:h // g + 1], v[h // g:h // g + 1]) for h in range(case["H"])]
        outs.append(torch.cat(per_head, dim=0).permute(1, 0, 2))
    o = torch.cat(outs, dim=0)
    for h, mem in enumerate(mems):
        assert len(mem.trace) == z["topk"].shape[0]
        for i, tr in enumerate(mem.trace):
            assert tr.topk_raw == [int(x) for x in z["topk"][i, h] if x >= 0], f"head {h}, exec block {i}"
        assert mem.num_blocks == int(z["n_blocks"])
    np.testing.assert_allclose(C.project_rows(o).numpy(), z["o_proj"], rtol=0, atol=2e-4)
