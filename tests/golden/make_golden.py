"""Record golden vectors from the reference itself.

Run on a machine that has a checkout of the reference (thunlp/InfLLM):

    python tests/golden/make_golden.py --ref /path/to/InfLLM

It imports the reference's context_manager / rope / torch multi-stage attention through
ref_shim (device literals rewritten to cpu, nothing else), runs the cases of cases.py in
fp32 and writes one small .npz per case next to this file.  Stored per case: the top-k ids
of every exec block in the order calc_block_topk returned them, the LRU table after every
exec block, the output (fp16 + a float64 random projection of every row), and a float64
projection of the representative-key rows.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases as C  # noqa: E402
import ref_shim  # noqa: E402


def record_context_manager(cm, rope, name, case):
    inputs = C.make_inputs(case)
    r = rope.RotaryEmbeddingESM(case["D"], case["base"], 1.0)
    mgr = cm.ContextManager(r, case["n_init"], case["n_local"], case["bs"], case["max_cached"], case["topk"],
                            case["exc"], case["decay"], False, case["repr_topk"], case["strategy"],
                            case.get("chunk_topk"), False, False, False, False)
    topks, cached = [], []
    orig_topk = cm.ContextManager.calc_block_topk
    orig_append = cm.ContextManager._append

    def spy_topk(self, gq):
        ret = orig_topk(self, gq)
        topks.append(list(ret[0]))  # copy before get_global_hidden_and_mask sorts it in place
        return ret

    def spy_append(self, *a, **k):
        ret = orig_append(self, *a, **k)
        cached.append(list(self.cached_blocks[0].items()))
        return ret

    cm.ContextManager.calc_block_topk = spy_topk
    cm.ContextManager._append = spy_append
    outs = []
    try:
        with torch.inference_mode():
            for q, k, v in inputs:
                o = mgr.append(q[None], k[None], v[None], q[None], k[None], v[None])
                outs.append(o[0].permute(1, 0, 2).contiguous())  # (L, H, D)
    finally:
        cm.ContextManager.calc_block_topk = orig_topk
        cm.ContextManager._append = orig_append
    o = torch.cat(outs, dim=0)
    n_steps = len(topks)
    tk = np.full((n_steps, case["topk"]), -1, dtype=np.int32)
    for i, t in enumerate(topks):
        tk[i, : len(t)] = t
    c_off = np.zeros(n_steps + 1, dtype=np.int64)
    c_ids, c_val = [], []
    for i, items in enumerate(cached):
        c_off[i + 1] = c_off[i] + len(items)
        c_ids += [b for b, _ in items]
        c_val += [float(s) for _, s in items]
    bk = mgr.block_k[0].get_data() if mgr.num_global_block else torch.zeros((0, case["H"] * case["D"]))
    rows = C.sample_rows(o.shape[0], 32 if name in C.LARGE else 96)
    # the per-row fingerprints of the large cases are kept in fp32: half the bytes, still 1e-7 relative
    fp = np.float32 if name in C.LARGE else np.float64
    meta = dict(case=case, name=name, torch=torch.__version__, digest=C.inputs_digest(inputs),
                n_blocks=int(mgr.num_global_block), init_len=int(mgr.init_k.size(-2)),
                remainder_len=int(mgr.global_remainder[0].size(-2)), length=int(mgr.length))
    np.savez_compressed(
        os.path.join(HERE, f"cm_{name}.npz"), meta=json.dumps(meta), topk=tk, cached_off=c_off,
        cached_ids=np.asarray(c_ids, dtype=np.int32), cached_val=np.asarray(c_val, dtype=np.float64),
        o16_rows=rows.numpy(), o16=o[rows].to(torch.float16).numpy(), o_proj=C.project_rows(o).numpy().astype(fp),
        block_k_proj=C.project_rows(bk).numpy().astype(fp))
    print(f"{name}: {n_steps} exec blocks, {mgr.num_global_block} sealed, out {tuple(o.shape)}")


def record_multi_stage(Attn, rope):
    """Direct cases of the multi-stage attention class and of the RoPE module."""
    out = {}
    for ci, (H, HKV, D, Lq, stages) in enumerate(C.MULTI_STAGE_SPECS):
        att = Attn((1, H, Lq, D), torch.float32, "cpu")
        tensors = C.multi_stage_inputs(ci)
        for si, (Lk, sw, comp, gs) in enumerate(stages):
            q, k, v = tensors[si]
            att.append(q[None], k[None], v[None], sliding_window=sw, complement_sliding_window=comp,
                       end=(si == len(stages) - 1), get_score=gs)
        ret, scores = att.get_result()
        out[f"c{ci}_ret"] = ret[0].numpy()
        for si, s in enumerate(scores):
            if s is not None:
                out[f"c{ci}_score{si}"] = s[0].numpy()
    # RoPE: window-relative and one-angle forms
    r = rope.RotaryEmbeddingESM(128, 1000000.0, 1.0)
    q, k = C.rope_inputs()
    q, k = q[None], k[None]
    rq, rk = r(q, k)
    out["rope_rq"], out["rope_rk"] = rq[0].numpy(), rk[0].numpy()
    out["rope_one"] = r.apply_rotary_pos_emb_one_angle(q, 4096)[0].numpy()
    np.savez_compressed(os.path.join(HERE, "multi_stage.npz"), **out)
    print("multi_stage: recorded", len(C.MULTI_STAGE_SPECS), "cases + rope")


def record_perhead(cm, rope):
    """cases.PERHEAD through the reference with perhead=True: outputs and the retrieval of every head (unit)."""
    case = C.PERHEAD
    inputs = C.make_inputs(case)
    r = rope.RotaryEmbeddingESM(case["D"], case["base"], 1.0)
    mgr = cm.ContextManager(r, case["n_init"], case["n_local"], case["bs"], case["max_cached"], case["topk"],
                            case["exc"], case["decay"], False, case["repr_topk"], case["strategy"], None,
                            False, False, False, True)
    topks = []
    orig_topk = cm.ContextManager.calc_block_topk

    def spy_topk(self, gq):
        ret = orig_topk(self, gq)
        topks.append([list(u) for u in ret])  # one list per unit (= head)
        return ret

    cm.ContextManager.calc_block_topk = spy_topk
    outs = []
    try:
        with torch.inference_mode():
            for q, k, v in inputs:
                o = mgr.append(q[None], k[None], v[None], q[None], k[None], v[None])
                outs.append(o[0].permute(1, 0, 2).contiguous())  # (L, H, D)
    finally:
        cm.ContextManager.calc_block_topk = orig_topk
    o = torch.cat(outs, dim=0)
    tk = np.full((len(topks), case["H"], case["topk"]), -1, dtype=np.int32)
    for i, per_unit in enumerate(topks):
        for u, t in enumerate(per_unit):
            tk[i, u, : len(t)] = t
    rows = C.sample_rows(o.shape[0])
    np.savez_compressed(os.path.join(HERE, "perhead.npz"), digest=C.inputs_digest(inputs), topk=tk, o16_rows=rows.numpy(),
                        o16=o[rows].to(torch.float16).numpy(), o_proj=C.project_rows(o).numpy(),
                        n_blocks=int(mgr.num_global_block))
    print("perhead:", len(topks), "exec blocks,", mgr.num_global_block, "sealed per head, out", tuple(o.shape))


def record_sink_window(rope):
    """The reference's two sink + window attention types (infinite_lm.py, stream_llm.py) over the calls of
    cases.SINK_WINDOW: the output of every call."""
    import importlib

    c = C.SINK_WINDOW
    pq, pk, pv, po = C.sink_window_projections()
    out = {}
    for key, mod, fn in (("infinite", "inf_llm.attention.infinite_lm", "infinite_lm_forward"),
                         ("stream", "inf_llm.attention.stream_llm", "stream_llm_forward")):
        forward = getattr(importlib.import_module(mod), fn)(c["n_local"], c["n_init"], fattn=False)
        r = rope.RotaryEmbeddingESM(c["D"], c["base"], 1.0)
        past = None
        with torch.inference_mode():
            for i, x in enumerate(C.sink_window_inputs()):
                o, past = forward(None, x[None], x[None], r, True, past, pq, pk, pv, po, c["D"], c["H"], c["HKV"])
                out[f"{key}_{i}"] = o[0].numpy()
        out[f"{key}_len"] = np.asarray(past[2])
    np.savez_compressed(os.path.join(HERE, "sink_window.npz"), **out)
    print("sink_window: recorded", len(c["lens"]), "calls of both attention types")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("INFLLM_REFERENCE"), required="INFLLM_REFERENCE" not in os.environ,
                    help="checkout of the reference (or set INFLLM_REFERENCE)")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    cm, rope, Attn = ref_shim.install(args.ref)
    torch.manual_seed(0)
    for name, case in C.CASES.items():
        if args.only and name != args.only:
            continue
        record_context_manager(cm, rope, name, case)
    if not args.only:
        record_multi_stage(Attn, rope)
        record_sink_window(rope)
        record_perhead(cm, rope)


if __name__ == "__main__":
    main()
