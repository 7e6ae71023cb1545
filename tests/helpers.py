"""Shared test utilities: golden-fixture loading and the comparison rules used everywhere."""
import json
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# tolerance of the bf16 CUDA path against the fp32 oracle (the figures the build target states)
MAX_ABS_TOL = 2e-2
MEAN_ABS_TOL = 1e-3


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, f"cm_{name}.npz"))
    meta = json.loads(str(z["meta"]))
    return meta, z


def golden_cached(z, step):
    a, b = int(z["cached_off"][step]), int(z["cached_off"][step + 1])
    return list(zip(z["cached_ids"][a:b].tolist(), z["cached_val"][a:b].tolist()))


def near_tie_ok(ref_ids, got_ids, scores, rel=1e-3):
    """The retrieval rule: id sets equal, or every id on which they differ has a reference score
    within `rel` (relative) of the k-th best score, i.e. the difference is a near-tie at the cut."""
    ref_set, got_set = set(ref_ids), set(got_ids)
    if ref_set == got_set:
        return True
    if scores is None:
        return False
    s = torch.as_tensor(scores, dtype=torch.float64)
    kth = torch.sort(s, descending=True).values[len(ref_ids) - 1].item()
    scale = max(abs(kth), 1e-30)
    return all(abs(s[i].item() - kth) <= rel * scale for i in ref_set ^ got_set)


# lines for the end-of-run summary (tests/conftest.py prints them): observed counts behind the tests' caps
REPORT = []


def report(line):
    REPORT.append(line)
