"""The CPU oracle of the sink + window attention types against recordings of the reference itself."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))

import cases as C  # noqa: E402
from oracle.sink_window_oracle import SinkWindowMemory  # noqa: E402


@pytest.mark.parametrize("kind,key", [("infinite-lm", "infinite"), ("stream-llm", "stream")])
def test_oracle_matches_the_reference_recording(kind, key):
    c = C.SINK_WINDOW
    z = np.load(os.path.join(ROOT, "tests", "golden", "sink_window.npz"))
    pq, pk, pv, _ = C.sink_window_projections()
    mem = SinkWindowMemory(c["n_local"], c["n_init"], c["D"], c["base"], kind)
    for i, x in enumerate(C.sink_window_inputs()):
        L = x.size(0)
        q = pq(x).view(L, c["H"], c["D"]).permute(1, 0, 2)
        k = pk(x).view(L, c["HKV"], c["D"]).permute(1, 0, 2)
        v = pv(x).view(L, c["HKV"], c["D"]).permute(1, 0, 2)
        got = mem.append(q, k, v).permute(1, 0, 2).reshape(L, -1)
        want = torch.from_numpy(z[f"{key}_{i}"])
        assert (got - want).abs().max().item() < 2e-5, f"call {i}"
    assert mem.length == int(z[f"{key}_len"]) == sum(c["lens"])
