#!/usr/bin/env python
"""Benchmark of the context-memory attention layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T]

Workload (N=1): one Mistral-7B-shaped attention layer in bf16 — hidden 4096, 32 query / 8 KV heads,
head_dim 128, RoPE base 1e6 — over a 131072-token prompt of seeded N(0,1) hidden states fed through
the attention-forward API in 8192-token calls and executed in 512-token exec blocks; n_init 128,
n_local 4096, memory units of 128 tokens, topk 16, repr_topk 4, max_cached_block 32, LRU.  64 units are
"planted": their hidden states lean (cos 0.6) towards a direction that a later 512-token query span
leans towards in projection space, so retrieval has real winners.  One step = one whole prompt.

Prints ONE JSON line.  `value` is tokens/s with the hidden states resident in HBM, `e2e` the same
through the same call with hidden states in pinned host memory (H2D and D2H copies timed),
`roofline` the exec-block attention kernel against the measured tensor peak, `cpu_baseline` the CPU
oracle (a restatement of the reference's torch path) on the host cores for a bounded steady-state
sample.  `--impl reference` times only that CPU path.  With N > 1 (torchrun) every rank runs its own
prompt through its own layer replica: the path has no cross-sequence exchange, so scaling is weak and
there is no collective on the data path.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(hidden=4096, H=32, HKV=8, D=128, base=1e6, n_init=128, n_local=4096, bs=128, topk=16, repr_topk=4,
           max_cached=32, exc=512, chunk=8192, tokens=131072, planted=64)


# ------------------------------------------------------------------------------------ workload
def make_weights(device, dtype):
    ws = []
    for seed, shape in zip((1, 2, 3, 4), ((CFG["H"] * CFG["D"], CFG["hidden"]), (CFG["HKV"] * CFG["D"], CFG["hidden"]),
                                          (CFG["HKV"] * CFG["D"], CFG["hidden"]), (CFG["hidden"], CFG["H"] * CFG["D"]))):
        g = torch.Generator().manual_seed(seed)
        ws.append((torch.randn(shape, generator=g) * 0.02).to(device=device, dtype=dtype))
    return ws


def make_hidden(tokens, seed, weights, device):
    """(1, tokens, hidden) bf16 on `device`: N(0,1) with planted key units and matching query spans."""
    wq, wk, _, _ = weights
    g = torch.Generator(device=device).manual_seed(seed)
    h = torch.empty((1, tokens, CFG["hidden"]), dtype=torch.bfloat16, device=device)
    step = 16384
    for s in range(0, tokens, step):
        n = min(step, tokens - s)
        h[0, s:s + n] = torch.randn((n, CFG["hidden"]), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    n_units = (tokens - CFG["n_init"] - CFG["n_local"]) // CFG["bs"]
    n_plant = min(CFG["planted"], max(n_units // 4, 0))
    if n_plant:
        gc = torch.Generator().manual_seed(5)
        units = torch.randperm(n_units, generator=gc)[:n_plant].tolist()
        u = torch.randn((n_plant, CFG["hidden"]), generator=gc).to(device)
        u = u / u.norm(dim=1, keepdim=True)
        # query-side direction whose projection points where the planted keys' projection points
        grp = CFG["H"] // CFG["HKV"]
        target = (wk.float() @ u.T).view(CFG["HKV"], 1, CFG["D"], n_plant).expand(-1, grp, -1, -1).reshape(-1, n_plant)
        w = torch.linalg.lstsq(wq.float(), target).solution.T  # (n_plant, hidden)
        w = w / w.norm(dim=1, keepdim=True)
        scale = math.sqrt(CFG["hidden"])
        n_eb = tokens // CFG["exc"]
        for i, b in enumerate(units):
            st = CFG["n_init"] + b * CFG["bs"]
            blk = h[0, st:st + CFG["bs"]].float()
            h[0, st:st + CFG["bs"]] = (0.8 * blk + 0.6 * scale * u[i]).to(torch.bfloat16)
            first_eb = (st + CFG["bs"] + CFG["n_local"]) // CFG["exc"] + 2  # first exec block that can retrieve it
            if first_eb >= n_eb:
                continue
            eb = first_eb + int(torch.randint(0, n_eb - first_eb, (1,), generator=gc))
            span = h[0, eb * CFG["exc"]:(eb + 1) * CFG["exc"]].float()
            h[0, eb * CFG["exc"]:(eb + 1) * CFG["exc"]] = (0.8 * span + 0.6 * scale * w[i]).to(torch.bfloat16)
    return h


class Layer:
    """The attention layer as a caller of the attention-forward API sees it.  With world > 1 this rank holds the
    projections of its slice of the heads (rows of wq/wk/wv, columns of wo) and sums the output projection's
    partial results over the ranks: tensor-parallel attention by KV-head groups."""

    def __init__(self, device, forward, rope, dtype=torch.bfloat16, rank=0, world=1):
        self.wq, self.wk, self.wv, self.wo = make_weights(device, dtype)
        self.heads, self.kv_heads = CFG["H"] // world, CFG["HKV"] // world
        if world > 1:
            import torch.distributed as dist

            nq, nk = self.heads * CFG["D"], self.kv_heads * CFG["D"]
            self.wq = self.wq[rank * nq:(rank + 1) * nq].contiguous()
            self.wk = self.wk[rank * nk:(rank + 1) * nk].contiguous()
            self.wv = self.wv[rank * nk:(rank + 1) * nk].contiguous()
            self.wo = self.wo[:, rank * nq:(rank + 1) * nq].contiguous()
        self.forward, self.rope, self.pkv = forward, rope, None
        lin = torch.nn.functional.linear
        self.pq, self.pk = (lambda x: lin(x, self.wq)), (lambda x: lin(x, self.wk))
        self.pv = lambda x: lin(x, self.wv)
        if world > 1:
            def out_proj(x):
                o = lin(x, self.wo)
                dist.all_reduce(o)
                return o
            self.po = out_proj
        else:
            self.po = lambda x: lin(x, self.wo)

    def __call__(self, x):
        o, self.pkv = self.forward(None, x, x, self.rope, True, self.pkv, self.pq, self.pk, self.pv, self.po,
                                   CFG["D"], self.heads, self.kv_heads)
        return o

    def reset(self):
        if self.pkv is not None:
            self.pkv.reset()


def prefill_device(layer, hidden):
    layer.reset()
    out = None
    for s in range(0, hidden.size(1), CFG["chunk"]):
        out = layer(hidden[:, s:s + CFG["chunk"]])
    return out


class HostPipe:
    """Two device input buffers and two copy streams: chunk i+1 travels to the device and the output of chunk i-1
    back to the host while chunk i runs through the layer."""

    def __init__(self, dev, dtype):
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.d_in = [torch.empty((1, CFG["chunk"], CFG["hidden"]), dtype=dtype, device=dev) for _ in range(2)]
        self.ev_in = [torch.cuda.Event(), torch.cuda.Event()]
        self.ev_free = [torch.cuda.Event(), torch.cuda.Event()]


def prefill_host(layer, h_hidden, h_out, pipe):
    """Same prompt with the hidden states in pinned host memory: every chunk is copied in, its output copied out.
    The caller's side of the attention-forward API is unchanged (one call per chunk on the current stream); the
    copies run on streams of their own, ordered by events."""
    layer.reset()
    main = torch.cuda.current_stream()
    total, chunk = h_hidden.size(1), CFG["chunk"]
    starts = list(range(0, total, chunk))
    pipe.s_in.wait_stream(main)
    pipe.s_out.wait_stream(main)

    def copy_in(i):
        b, s0 = i & 1, starts[i]
        n = min(chunk, total - s0)
        with torch.cuda.stream(pipe.s_in):
            if i >= 2:
                pipe.s_in.wait_event(pipe.ev_free[b])  # the layer has consumed chunk i-2
            pipe.d_in[b][:, :n].copy_(h_hidden[:, s0:s0 + n], non_blocking=True)
            pipe.ev_in[b].record(pipe.s_in)

    copy_in(0)
    for i, s0 in enumerate(starts):
        if i + 1 < len(starts):
            copy_in(i + 1)
        b, n = i & 1, min(chunk, total - s0)
        main.wait_event(pipe.ev_in[b])
        o = layer(pipe.d_in[b][:, :n])
        pipe.ev_free[b].record(main)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(pipe.s_out):
            pipe.s_out.wait_event(done)
            h_out[:, s0:s0 + n].copy_(o, non_blocking=True)
        o.record_stream(pipe.s_out)
    main.wait_stream(pipe.s_out)  # the step ends when its last output is on the host


# --------------------------------------------------------------------------------- CPU oracle arm
def cpu_steady_state_sample(tokens_at=65536, sample_tokens=2048, repeats=1, threads=None):
    """Times the CPU oracle (the reference's torch path restated) on `sample_tokens` tokens of the same
    layer in steady state: context memory pre-filled to `tokens_at` tokens (seeded random keys, values,
    representative keys and scores), projections included.  Returns (tokens/s, seconds, cores)."""
    from oracle.infllm_oracle import OracleContextMemory

    if threads:
        torch.set_num_threads(threads)
    cores = torch.get_num_threads()
    wq, wk, wv, wo = make_weights("cpu", torch.float32)
    g = torch.Generator().manual_seed(99)
    best = None
    for _ in range(repeats):
        mem = OracleContextMemory(CFG["n_init"], CFG["n_local"], CFG["bs"], CFG["max_cached"], CFG["topk"], CFG["exc"],
                                  CFG["repr_topk"], CFG["base"], 1.0)
        nb = (tokens_at - CFG["n_local"] - CFG["n_init"]) // CFG["bs"]
        mem.length = tokens_at
        mem.init_len, mem.init_full = CFG["n_init"], True
        mem.frontier = CFG["n_init"] + nb * CFG["bs"]
        mem.k_log = torch.randn((CFG["HKV"], tokens_at, CFG["D"]), generator=g)
        mem.v_log = torch.randn((CFG["HKV"], tokens_at, CFG["D"]), generator=g)
        mem.acc = torch.rand((CFG["H"], tokens_at), generator=g)
        mem.block_k = list(torch.randn((nb, CFG["H"] * CFG["D"]), generator=g))
        x = torch.randn((sample_tokens, CFG["hidden"]), generator=g)
        t0 = time.perf_counter()
        with torch.inference_mode():
            q = (x @ wq.T).view(sample_tokens, CFG["H"], CFG["D"]).permute(1, 0, 2)
            k = (x @ wk.T).view(sample_tokens, CFG["HKV"], CFG["D"]).permute(1, 0, 2)
            v = (x @ wv.T).view(sample_tokens, CFG["HKV"], CFG["D"]).permute(1, 0, 2)
            o = mem.append(q, k, v)
            _ = o.permute(1, 0, 2).reshape(sample_tokens, -1) @ wo.T
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return sample_tokens / best, best, cores


def cpu_decode_sample(units=2048, steps=32):
    """Times the CPU oracle on `steps` decode tokens over a memory of `units` sealed units (seeded random keys,
    values and representative keys; full window and sink).  Returns (us per token, seconds, cores)."""
    from oracle.infllm_oracle import OracleContextMemory

    cores = torch.get_num_threads()
    H, HKV, D = CFG["H"], CFG["HKV"], CFG["D"]
    g = torch.Generator().manual_seed(98)
    mem = OracleContextMemory(DEC["n_init"], DEC["n_local"], DEC["bs"], DEC["max_cached"], DEC["topk"], DEC["exc"],
                              DEC["repr_topk"], CFG["base"], 1.0)
    tokens_at = DEC["n_init"] + units * DEC["bs"] + DEC["n_local"]
    mem.length = tokens_at
    mem.init_len, mem.init_full = DEC["n_init"], True
    mem.frontier = DEC["n_init"] + units * DEC["bs"]
    mem.k_log = torch.randn((HKV, tokens_at, D), generator=g)
    mem.v_log = torch.randn((HKV, tokens_at, D), generator=g)
    mem.acc = torch.zeros((H, tokens_at))
    mem.block_k = list(torch.randn((units, H * D), generator=g))
    toks = [(torch.randn((H, 1, D), generator=g), torch.randn((HKV, 1, D), generator=g), torch.randn((HKV, 1, D), generator=g))
            for _ in range(steps + 2)]
    with torch.inference_mode():
        for q, k, v in toks[:2]:
            mem.append(q, k, v)
        t0 = time.perf_counter()
        for q, k, v in toks[2:]:
            mem.append(q, k, v)
        dt = time.perf_counter() - t0
    return 1e6 * dt / steps, dt, cores


SAMPLE_DESC = ("{n} tokens ({eb} exec blocks of 512) of the same layer in steady state at 65536 tokens of context "
               "(479 sealed units, full window), projections included, fp32 torch on the host")
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
REF_SETUP, REF_SAMPLE = 12288, 2048


class ReferenceLayer:
    """The reference's own ContextManager (unmodified copy under baseline/_ref, device literals rewritten to cpu at
    import by tests/golden/ref_shim.py) behind the same projections as the GPU arm, fp32 on the host cores.  The
    memory is brought to steady state once (REF_SETUP tokens: full window, 62 sealed units, retrieval of 16 active);
    every sample() then appends the next REF_SAMPLE tokens (4 exec blocks of 512) and returns the seconds it took."""

    def __init__(self):
        sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
        import ref_shim

        cm, rope, _ = ref_shim.install(REF_DIR)
        self.w = make_weights("cpu", torch.float32)
        self.g = torch.Generator().manual_seed(99)
        self.mgr = cm.ContextManager(rope.RotaryEmbeddingESM(CFG["D"], CFG["base"], 1.0), CFG["n_init"], CFG["n_local"],
                                     CFG["bs"], CFG["max_cached"], CFG["topk"], CFG["exc"], None, False, CFG["repr_topk"],
                                     "lru", None, False, False, False, False)
        with torch.inference_mode():
            for _ in range(0, REF_SETUP, 4096):
                self._feed(4096)

    def _feed(self, n):
        wq, wk, wv, wo = self.w
        x = torch.randn((n, CFG["hidden"]), generator=self.g)
        q = (x @ wq.T).view(n, CFG["H"], CFG["D"]).permute(1, 0, 2)[None]
        k = (x @ wk.T).view(n, CFG["HKV"], CFG["D"]).permute(1, 0, 2)[None]
        v = (x @ wv.T).view(n, CFG["HKV"], CFG["D"]).permute(1, 0, 2)[None]
        o = self.mgr.append(q, k, v, q, k, v)
        return o[0].permute(1, 0, 2).reshape(n, -1) @ wo.T

    def sample(self):
        t0 = time.perf_counter()
        with torch.inference_mode():
            self._feed(REF_SAMPLE)
        return time.perf_counter() - t0


def triton_exec_block_timing(dev):
    """The reference's GPU kernel for the same exec block (its Triton _attn_fwd two-stage append with fattn=True,
    triton_impl.py:430-478 and :520-556): 512 queries x 32 heads over a 4608-key window stage and a 2688-key global
    stage, bf16, with the score pass of the local stage.  Returns microseconds per exec block, or the error."""
    try:
        sys.path.insert(0, REF_DIR)
        from inf_llm.attention.dot_production_attention.triton_impl import TritonMultiStageDotProductionAttention as Att

        H, HKV, D, lq = CFG["H"], CFG["HKV"], CFG["D"], CFG["exc"]
        g = torch.Generator(device=dev).manual_seed(3)
        mk = lambda h, n: torch.randn((1, h, n, D), generator=g, device=dev).to(torch.bfloat16)  # noqa: E731
        q, kl, vl = mk(H, lq), mk(HKV, CFG["n_local"] + lq), mk(HKV, CFG["n_local"] + lq)
        glk = CFG["topk"] * CFG["bs"] + CFG["n_init"] + lq
        kg, vg = mk(HKV, glk), mk(HKV, glk)

        def block():
            att = Att(q.shape, q.dtype, q.device)
            att.append(q, kl, vl, get_score=True, sliding_window=CFG["n_local"])
            att.append(q, kg, vg, end=True, get_score=False, sliding_window=(glk + lq, CFG["n_local"]),
                       complement_sliding_window=True)
            return att.get_result()

        for _ in range(3):
            block()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            block()
        b.record()
        torch.cuda.synchronize()
        us = 1e3 * a.elapsed_time(b) / 10
        flops = 4.0 * D * H * (sum(min(CFG["n_local"], CFG["n_local"] + i + 1) for i in range(lq)) + lq * glk)
        return dict(us_per_exec_block=us, tflops=flops / us / 1e6, includes="attention of both stages + the local score pass",
                    triton=__import__("triton").__version__)
    except Exception as e:  # the reference pins an older Triton
        return dict(error=f"{type(e).__name__}: {str(e)[:300]}")
    finally:
        # the package was imported as it is on disk: forget it, the CPU arm imports it again through its shim
        for name in [m for m in sys.modules if m == "inf_llm" or m.startswith("inf_llm.")]:
            del sys.modules[name]
        if REF_DIR in sys.path:
            sys.path.remove(REF_DIR)


def run_reference(args, rank):
    """The reference arm: rank 0 alone, on every host core it can use."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)  # a launcher may have set OMP_NUM_THREADS=1
    cores = torch.get_num_threads()
    have_ref = os.path.isdir(os.path.join(REF_DIR, "inf_llm"))
    n = REF_SAMPLE
    # the reference's GPU kernel first: the CPU shim below replaces torch.cuda's stream and event classes for good
    gpu_kernel = triton_exec_block_timing(torch.device("cuda", 0)) if (have_ref and torch.cuda.is_available() and
                                                                      not args.no_ref_gpu) else None
    if have_ref:
        layer = ReferenceLayer()
        sample, kind = layer.sample, "reference"
        desc = (f"{n} tokens (4 exec blocks of 512) appended to the reference's own ContextManager (inf_llm/attention/"
                f"context_manager.py, torch path, fattn=False) in steady state after {REF_SETUP} tokens (full 4096-token "
                "window, retrieval of 16 units active; context grows by 2048 tokens per step), projections included, "
                "fp32 on the host cores")
    else:
        sample = lambda: cpu_steady_state_sample(sample_tokens=n, threads=cores)[1]  # noqa: E731
        kind, desc = "port", SAMPLE_DESC.format(n=n, eb=n // 512)
    for _ in range(args.warmup):
        sample()
    secs = [sample() for _ in range(args.steps)]
    dt = sum(secs)
    val = n * args.steps / dt
    line = dict(metric="exec-block prefill tokens/s/GPU @128K ctx", value=val, unit="tokens/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=1e3 * dt / args.steps, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=dict(workload="mistral-7b attention layer, 131072-token prefill, exec 512, n_local 4096, "
                                     "topk 16, repr_topk 4, max_cached 32 (CPU arm: steady-state sample)"),
                cpu_baseline=dict(value=val, unit="tokens/s", cores=cores, kind=kind, sample=desc),
                e2e=dict(value=val, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    if gpu_kernel is not None:
        line["reference_gpu_kernel"] = gpu_kernel
    print(json.dumps(line))


# ------------------------------------------------------------------------------------- GPU arm
def sample_clocks_start(gpu_index):
    """One sampler for the whole job: local rank 0 polls the GPUs of all local ranks (eight pollers, one per rank, took
    host time and driver locks from the ranks they were watching)."""
    f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
    if gpu_index != 0:
        return None, f
    n_local = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")))
    gpu_index = ",".join(str(i) for i in range(max(n_local, 1)))
    q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        p = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={q}", "--format=csv,noheader,nounits",
                              "-lms", "200"], stdout=f, stderr=subprocess.DEVNULL)
    except OSError:
        return None, f
    return p, f


def sample_clocks_stop(p, f):
    if p is not None:
        p.terminate()
        try:
            p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            p.kill()
    f.flush()
    f.seek(0)
    sm, mx, reasons = [], 0, set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for ln in f.read().splitlines():
        parts = [x.strip() for x in ln.split(",")]
        if len(parts) < 7:
            continue
        try:
            sm.append(float(parts[0]))
            mx = max(mx, float(parts[1]))
        except ValueError:
            continue
        for nme, val in zip(names, parts[3:7]):
            if val.lower().startswith("active"):
                reasons.add(nme)
    f.close()
    os.unlink(f.name)
    sm.sort()
    med = sm[len(sm) // 2] if sm else None
    return dict(sm_mhz=med, sm_max_mhz=mx or None, reasons=sorted(reasons), samples=len(sm))


def profile_traffic(name):
    """DRAM bytes per launch (read + write) from the ncu summary kept under profiles/<name>.md, or None."""
    import re

    try:
        text = open(os.path.join(ROOT, "profiles", name + ".md")).read()
    except OSError:
        return None
    unit = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    total = 0.0
    for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        m = re.search(re.escape(key) + r" \[(\w+)\] = ([0-9.]+)", text)
        if not m or m.group(1) not in unit:
            return None
        total += float(m.group(2)) * unit[m.group(1)]
    return total


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops_sustained") or d.get("bf16_tflops"), d.get("hbm_gbs"), "measured"
    return 1400.0, 6650.0, "fallback"


def run_ours(args, rank, world, local_rank, device_store_mb=0, light=False):
    """The prefill workload.  device_store_mb = 0 (the headline): sealed units live in the pinned host store only and
    every cache refill is a cudaMemcpyAsync over PCIe on a side stream, as in the reference.  > 0: the variant that
    also keeps a device copy of the store (refills are device-to-device copies).  `light` skips the end-to-end pass,
    the overlap trace and the CPU sample."""
    import torch.distributed as dist

    from infllm_b200 import _lib
    from infllm_b200.attention import ATTN_FORWRAD, ContextManager, RotaryEmbeddingESM, device_store_reserve

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    tokens = args.tokens or CFG["tokens"]
    groups = world if (args.head_groups and world > 1) else 1  # one layer over all GPUs instead of a replica per GPU
    comm = None
    if groups > 1:
        from infllm_b200.attention import HeadGroupComm

        if CFG["HKV"] % groups:
            raise SystemExit(f"--head-groups: {CFG['HKV']} KV heads do not split over {groups} GPUs")
        comm = HeadGroupComm()
    fwd = ATTN_FORWRAD["inf-llm"](n_local=CFG["n_local"], n_init=CFG["n_init"], topk=CFG["topk"], block_size=CFG["bs"],
                                  max_cached_block=CFG["max_cached"], exc_block_size=CFG["exc"], fattn=True,
                                  repr_topk=CFG["repr_topk"], head_group_comm=comm, device_store_mb=device_store_mb)
    if device_store_mb:
        device_store_reserve(device_store_mb, dev)
    full = make_weights(dev, torch.bfloat16)  # the planted directions are built from the whole projections
    layer = Layer(dev, fwd, RotaryEmbeddingESM(CFG["D"], CFG["base"], 1.0), rank=rank if groups > 1 else 0, world=groups)
    hidden = make_hidden(tokens, seed=0 if groups > 1 else rank, weights=full, device=dev)
    del full
    h_hidden = torch.empty(hidden.shape, dtype=hidden.dtype, pin_memory=True)
    h_hidden.copy_(hidden)
    h_out = torch.empty((1, tokens, CFG["hidden"]), dtype=hidden.dtype, pin_memory=True)
    pipe = HostPipe(dev, hidden.dtype)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    parity = head_groups_selfcheck(rank, world, dev, comm) if groups > 1 else None
    with torch.inference_mode():
        for _ in range(max(args.warmup, 1)):  # the first pass also creates the context memory
            prefill_device(layer, hidden)
        layer.pkv.profile(True)
        layer.pkv.get_profile()
        layer.pkv.host_timers()
        clk_p, clk_f = sample_clocks_start(local_rank)
        l0 = _lib.lib.infllm_launch_count()
        ms = timed(lambda: prefill_device(layer, hidden), args.steps)
        launches = _lib.lib.infllm_launch_count() - l0
        prof = layer.pkv.get_profile()
        info = layer.pkv.info()
        host_us = layer.pkv.host_timers()
        layer.pkv.profile(False)
        clocks = sample_clocks_stop(clk_p, clk_f)
        overlap = None
        if not light:
            # one more prompt with the event trace on (untimed): where the refill copies ran relative to the attention
            layer.pkv.trace(True)
            prefill_device(layer, hidden)
            overlap = ContextManager.refill_overlap(layer.pkv.get_trace())
            layer.pkv.trace(False)
        ms_e2e = None
        if not light:
            for _ in range(min(args.warmup, 1)):
                prefill_host(layer, h_hidden, h_out, pipe)
            ms_e2e = timed(lambda: (prefill_host(layer, h_hidden, h_out, pipe), h_out[0, -1, 0].item()), args.steps)

    value = (world // groups) * tokens * args.steps / (ms / 1e3)
    if light:
        return dict(value=value, unit="tokens/s", ms_per_step=ms / args.steps, steps=args.steps,
                    store=dict(device_store_mb=device_store_mb, h2d_bytes=info["h2d_bytes"], d2h_bytes=info["d2h_bytes"],
                               hits=info["cache_hits"], misses=info["cache_misses"]),
                    kernels={k: dict(ms=v[0], launches=v[2]) for k, v in prof.items()},
                    note="the same prompt and layer with a device copy of the store: refills are device-to-device copies")
    e2e = (world // groups) * tokens * args.steps / (ms_e2e / 1e3)
    tf_peak, _, which = measured_peaks()
    attn_ms, attn_flops, attn_n = prof["attn"]
    achieved = attn_flops / (attn_ms / 1e3) / 1e12 if attn_ms > 0 else None
    line = dict(
        metric="exec-block prefill tokens/s/GPU @128K ctx", value=value, unit="tokens/s", n_gpus=world,
        steps=args.steps, warmup=args.warmup, ms_per_step=ms / args.steps, higher_is_better=True,
        scaling="strong" if groups > 1 else "weak", vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload=f"mistral-7b attention layer (hidden 4096, 32q/8kv, d128, rope 1e6), {tokens}-token prefill "
                             "in 8192-token calls, exec 512, n_init 128, n_local 4096, unit 128, topk 16, repr_topk 4, "
                             f"max_cached {CFG['max_cached']}, lru; 64 planted units", l2="inputs (1 GiB of hidden states per step) exceed L2",
                    replicas=world // groups,
                    store="pinned host store; every cache refill is a 512 KiB cudaMemcpyAsync over PCIe on a side stream",
                    parallelism=(f"kv-head groups x{groups}: one layer over all GPUs, retrieval scores and output "
                                 "projection all-reduced (NCCL)") if groups > 1 else f"dp{world}: one layer replica per GPU"),
        e2e=dict(value=e2e, unit="tokens/s", h2d_bytes_per_step=int(hidden.numel() * 2),
                 d2h_bytes_per_step=int(h_out.numel() * 2), ms_per_step=ms_e2e / args.steps),
        gpu_launches=int(launches),
        roofline=dict(bound="tensor", kernel="exec-block attention (local + global stage)", achieved=achieved,
                      peak=tf_peak, unit="TFLOP/s", frac=(achieved / tf_peak if achieved else None),
                      # DRAM bytes per launch of a steady-state exec block from an ncu capture of this kernel on a
                      # 32768-token prompt (its summary is kept with the other profiles); a launch at 131072 tokens
                      # reads the same operands.  None when the heads are sharded (other shapes per launch).
                      traffic=(profile_traffic("attn_tc3_kernel_exec_block") if groups == 1 else None),
                      traffic_source="ncu summary profiles/attn_tc3_kernel_exec_block.md (32768-token case)",
                      peak_source=f"bf16_tflops_sustained of {which}", launches=int(attn_n),
                      us_per_launch=1e3 * attn_ms / max(attn_n, 1),
                      flops_per_launch=attn_flops / max(attn_n, 1)),
        kernels={k: dict(ms=v[0], launches=v[2]) for k, v in prof.items()},
        store=dict(h2d_bytes=info["h2d_bytes"], h2d_late_bytes=info["h2d_late_bytes"], d2h_bytes=info["d2h_bytes"],
                   hits=info["cache_hits"], misses=info["cache_misses"], evictions=info["evictions"],
                   h2d_overlap_frac=(overlap or {}).get("overlap_frac"), h2d_hidden_frac=(overlap or {}).get("hidden_frac"),
                   refill_copy_ms_per_step=(overlap or {}).get("copy_ms"),
                   note="counters since the context was created (warm-up and timed prompts); overlap_frac = share of the "
                        "refill-copy time during which an exec-block attention kernel was running, hidden_frac = share "
                        "that no exec block waited for (event trace of one untimed prompt)"),
        host_ms_per_step={k: v / 1e3 / args.steps for k, v in host_us.items()},
        clocks=clocks)
    if parity is not None:
        line["parity"] = parity
    if rank == 0 and world == 1 and not args.no_cpu:
        torch.set_num_threads(os.cpu_count() or 1)
        ref = None
        if os.path.isdir(os.path.join(REF_DIR, "inf_llm")):
            # the reference itself, in a process of its own (its CPU shim replaces torch.cuda's stream classes)
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "2", "--warmup", "1",
                                "--no-ref-gpu"], capture_output=True, text=True,
                               env=dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS=str(os.cpu_count() or 1)))
            for ln in r.stdout.splitlines():
                if ln.startswith("{"):
                    ref = json.loads(ln)["cpu_baseline"]
        if ref is not None:
            line["cpu_baseline"] = ref
        else:
            v, secs, cores = cpu_steady_state_sample(sample_tokens=2048)
            line["cpu_baseline"] = dict(value=v, unit="tokens/s", cores=cores, kind="port", seconds=secs,
                                        sample=SAMPLE_DESC.format(n=2048, eb=4))
    return line


# ------------------------------------------------------------------------------ decode workload
DEC = dict(units=8192, topk=32, max_cached=32, n_local=4096, n_init=128, bs=128, repr_topk=4, exc=512, planted_frac=0.01,
           layers=2)


def make_decode_memory(dev, rope, seed):
    """Host tensors of a 1M-token memory for one Mistral-shaped layer: sealed units ~N(0,1), representative keys
    ~N(0,1) except 1% planted units whose representative keys lean towards the direction the query stream
    leans towards (after the one-angle rotation that retrieval applies), sink and window ~N(0,1).  The planted
    units lean by graded amounts, so the per-token noise of the queries reorders only the ones near the top-k
    boundary: most retrieved units stay cached from one token to the next, a few miss."""
    H, HKV, D, n = CFG["H"], CFG["HKV"], CFG["D"], DEC["units"]
    g = torch.Generator(device=dev).manual_seed(seed)
    units = torch.empty((n, 2, HKV, DEC["bs"], D), dtype=torch.bfloat16)
    for s in range(0, n, 512):
        m = min(512, n - s)
        units[s:s + m] = torch.randn((m, 2, HKV, DEC["bs"], D), generator=g, device=dev).to(torch.bfloat16).cpu()
    block_k = torch.randn((n, H * D), generator=g, device=dev)
    direction = torch.randn((H, 1, D), generator=g, device=dev)
    direction = direction / direction.norm(dim=-1, keepdim=True)
    rotated = rope.apply_rotary_pos_emb_one_angle(direction.to(torch.bfloat16)[None], DEC["n_local"])[0].float().reshape(-1)
    n_plant = max(1, int(n * DEC["planted_frac"]))
    gc = torch.Generator().manual_seed(seed + 1)
    planted = torch.randperm(n, generator=gc)[:n_plant].to(dev)
    lean = torch.linspace(9.0, 3.0, n_plant, device=dev)[:, None]  # all clearly above the random scores
    block_k[planted] = 0.7 * block_k[planted] + lean * rotated
    small = lambda *shape: torch.randn(shape, generator=g, device=dev).to(torch.bfloat16).cpu()  # noqa: E731
    return (units, block_k.to(torch.bfloat16).cpu(), small(HKV, DEC["n_init"], D), small(HKV, DEC["n_init"], D),
            small(HKV, DEC["n_local"], D), small(HKV, DEC["n_local"], D)), direction


def run_decode(args, rank, world, local_rank, device_store_mb=0):
    """The decode workload on one GPU per rank.  device_store_mb = 0 (the headline): the 8192 units of a layer live in
    the pinned host store and every cache refill crosses PCIe.  > 0: the variant with a device copy of the store."""
    import torch.distributed as dist

    from infllm_b200 import _lib
    from infllm_b200.attention import ContextManager, RotaryEmbeddingESM, device_store_reserve

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    H, HKV, D = CFG["H"], CFG["HKV"], CFG["D"]
    rope = RotaryEmbeddingESM(D, CFG["base"], 1.0)
    # several layers' memories take turns, as in a model: one layer's 64 MiB of representative keys and its
    # 34 MB of window and unit K/V would otherwise stay in the 126 MB L2 from one token to the next
    n_layers = DEC["layers"]
    cms, dirs = [], []
    for li in range(n_layers):
        mem, direction = make_decode_memory(dev, rope, seed=17 * rank + li)
        if device_store_mb and li == 0:
            device_store_reserve(device_store_mb * n_layers, dev)
        cm = ContextManager(rope, DEC["n_init"], DEC["n_local"], DEC["bs"], DEC["max_cached"], DEC["topk"], DEC["exc"],
                            None, True, DEC["repr_topk"], device_store_mb=device_store_mb)
        cm.load_synthetic(*mem)
        del mem
        cms.append(cm)
        dirs.append(direction)
    total = (args.warmup + 3 * args.steps + 2) * n_layers
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    lean = torch.stack([dirs[i % n_layers] for i in range(total)])[:, None]  # (total, 1, H, 1, D)
    qs = (torch.randn((total, 1, H, 1, D), generator=g, device=dev) + 3.0 * lean).to(torch.bfloat16)
    ks = torch.randn((total, 1, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)
    vs = torch.randn((total, 1, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)
    h_q, h_k, h_v = (t.cpu().pin_memory() for t in (qs, ks, vs))
    h_o = torch.empty((1, H, 1, D), dtype=torch.bfloat16).pin_memory()
    pos = [0]

    toks = [(qs[i], ks[i], vs[i]) for i in range(total)]  # views made once: the timed loop is the library's

    def step_device():  # one token through every layer
        for cm in cms:
            q, k, v = toks[pos[0]]
            pos[0] += 1
            cm.append(q, k, v, q, k, v)

    def step_host():
        for cm in cms:
            i = pos[0]
            pos[0] += 1
            q, k, v = (t[i].to(dev, non_blocking=True) for t in (h_q, h_k, h_v))
            h_o.copy_(cm.append(q, k, v, q, k, v), non_blocking=True)
            torch.cuda.current_stream().synchronize()  # the caller consumes a layer's output before the next layer

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    def merged(dicts):
        out = {}
        for d in dicts:
            for k, v in d.items():
                out[k] = tuple(x + y for x, y in zip(out[k], v)) if k in out else tuple(v)
        return out

    with torch.inference_mode():
        # (the sampler starts with the warm-up: the timed region of a decode run is shorter than a polling period)
        clk_p, clk_f = sample_clocks_start(local_rank)
        for _ in range(args.warmup):
            step_device()
        info0 = [cm.info() for cm in cms]
        l0 = _lib.lib.infllm_launch_count()
        ms = timed(step_device, args.steps)
        launches = _lib.lib.infllm_launch_count() - l0
        info1 = [cm.info() for cm in cms]
        # the kernels' own durations: the same K steps once more with CUDA events around the scoring and the
        # attention of every token.  Kept out of `value`'s region: four event records per 50 us token cost 14 us of it
        for cm in cms:
            cm.profile(True)
            cm.get_profile()
        ms_events = timed(step_device, args.steps)
        prof = merged([cm.get_profile() for cm in cms])
        for cm in cms:
            cm.profile(False)
        clocks = sample_clocks_stop(clk_p, clk_f)
        step_host()
        ms_e2e = timed(step_host, args.steps)
    _, hbm_peak, which = measured_peaks()
    per_layer = args.steps * n_layers
    us = 1e3 * ms / per_layer
    topk_ms, topk_bytes, topk_n = prof["topk"]
    dec_ms, dec_bytes, dec_n = prof["decode"]
    achieved = topk_bytes / (topk_ms / 1e3) / 1e9 if topk_ms > 0 else None
    hits = sum(y["cache_hits"] - x["cache_hits"] for x, y in zip(info0, info1))
    misses = sum(y["cache_misses"] - x["cache_misses"] for x, y in zip(info0, info1))
    cold = DEC["units"] * n_layers >= 16384
    line = dict(
        metric="decode-attn us/token @1M ctx", value=us, unit="us/token", n_gpus=world, steps=args.steps,
        warmup=args.warmup, ms_per_step=ms / args.steps, higher_is_better=False, scaling="weak", vs_baseline=None,
        dtype="bf16", data="synthetic",
        config=dict(workload=f"mistral-7b-shaped layer, decode over {DEC['units']} memory units of 128 tokens "
                             f"({DEC['n_init'] + DEC['units'] * DEC['bs'] + DEC['n_local']} tokens), topk 32, repr_topk 4, "
                             "max_cached 32, n_local 4096, n_init 128; 1% planted units with graded lean; "
                             f"a step is one token through {n_layers} layers with separate memories, value is per layer",
                    l2=(f"{n_layers} layers take turns: {n_layers} x (64 MiB representative keys + 34 MB K/V) exceed the "
                        "126 MB L2") if cold else "working set below L2 at this reduced size",
                    replicas=world),
        e2e=dict(value=1e3 * ms_e2e / per_layer, unit="us/token", h2d_bytes_per_step=int((H + 2 * HKV) * D * 2 * n_layers),
                 d2h_bytes_per_step=int(H * D * 2 * n_layers)),
        gpu_launches=int(launches),
        roofline=dict(bound="hbm", kernel="block_score_topk_kernel (unit scoring + top-k)", achieved=achieved,
                      peak=hbm_peak, unit="GB/s", frac=(achieved / hbm_peak if achieved else None), traffic=None,
                      peak_source=f"hbm_gbs of {which}", launches=int(topk_n),
                      us_per_launch=1e3 * topk_ms / max(topk_n, 1), bytes_per_launch=topk_bytes / max(topk_n, 1),
                      timed_in="a second pass of the same K steps with CUDA events around the kernel on its stream",
                      us_per_token_with_events=1e3 * ms_events / per_layer),
        kernels={k: dict(ms=v[0], launches=v[2], work=v[1]) for k, v in prof.items()},
        decode_attention=dict(kernels="attn_decode_kernel + lse_merge_kernel",
                              achieved_gbs=(dec_bytes / (dec_ms / 1e3) / 1e9 if dec_ms > 0 else None),
                              us_per_launch=1e3 * dec_ms / max(dec_n, 1), bytes_per_launch=dec_bytes / max(dec_n, 1)),
        store=dict(hits=hits, misses=misses, miss_rate=misses / max(hits + misses, 1),
                   h2d_bytes_per_token_layer=sum(y["h2d_bytes"] - x["h2d_bytes"] for x, y in zip(info0, info1)) / max(per_layer, 1),
                   units_read_in_place_per_token_layer=sum(y["inplace_units"] - x["inplace_units"]
                                                           for x, y in zip(info0, info1)) / max(per_layer, 1),
                   refill_source=("device copy of the store" if device_store_mb else "pinned host store over PCIe")),
        clocks=clocks)
    if rank == 0 and world == 1 and not args.no_cpu:
        v, secs, cores = cpu_decode_sample()
        line["cpu_baseline"] = dict(value=v, unit="us/token", cores=cores, kind="port", seconds=secs,
                                    sample="32 decode tokens of one layer over a memory of 2048 units (266368 tokens) "
                                           "instead of 8192, fp32 torch on the host; the unit scoring is a quarter of "
                                           "the full size's, the attention the same")
    return line


THRASH = dict(H=32, HKV=32, D=128, base=1e6, n_init=128, n_local=4096, bs=128, topk=16, repr_topk=8, max_cached=16, exc=256,
              chunk=8192, tokens=524288, groups=8)


def thrash_chunk(dev, start, n, dirs_k, dirs_q, unit_gain, gen):
    """q, k, v (heads, n, D) bf16 of tokens [start, start + n) of the cache-thrash prompt: N(0,1), the keys of memory
    unit b leaning (cos 0.6, times a per-unit gain) towards the direction of group b % G, the queries of exec block t
    leaning towards the direction that retrieval's one-angle rotation turns into group t % G's."""
    T = THRASH
    H, D, G = T["H"], T["D"], T["groups"]
    q = torch.randn((H, n, D), generator=gen, device=dev)
    k = torch.randn((H, n, D), generator=gen, device=dev)
    v = torch.randn((H, n, D), generator=gen, device=dev)
    tok = torch.arange(start, start + n, device=dev)
    amp, keep = 0.6 * math.sqrt(D), 0.8
    unit = ((tok - T["n_init"]).clamp(min=0) // T["bs"]).clamp(max=unit_gain.numel() - 1)
    in_unit = (tok >= T["n_init"]).float()
    k = keep * k + (amp * in_unit * unit_gain[unit])[None, :, None] * dirs_k[unit % G].permute(1, 0, 2)
    eb = tok // T["exc"]
    q = keep * q + amp * dirs_q[eb % G].permute(1, 0, 2)
    return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)


def run_thrash(args, rank, world, local_rank):
    """Cache-thrash stress: a Qwen-1.5-7B-shaped layer (32 query / 32 KV heads), 524288 tokens = 4096 memory units of
    2 MiB, topk 16, repr_topk 8, exec blocks of 256, and a cache of exactly one retrieval (max_cached_block 16: the
    configuration's literal 8 cannot hold a retrieval and is refused, as the reference asserts).  Consecutive exec
    blocks retrieve disjoint groups of units, so every exec block evicts the whole cache and refills it from the
    pinned host store: 32 MiB over PCIe per 256 tokens."""
    from infllm_b200 import _lib
    from infllm_b200.attention import ContextManager, RotaryEmbeddingESM

    T = THRASH
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    tokens = args.tokens or T["tokens"]
    H, D, G = T["H"], T["D"], T["groups"]
    rope = RotaryEmbeddingESM(D, T["base"], 1.0)
    refused = None
    try:
        probe = ContextManager(rope, T["n_init"], T["n_local"], T["bs"], 8, T["topk"], T["exc"], None, True, T["repr_topk"])
        z = torch.zeros((1, H, T["exc"], D), dtype=torch.bfloat16, device=dev)
        probe.append(z, z, z, z, z, z)
    except _lib.InfLLMCapacityError as e:
        refused = str(e)
    gen = torch.Generator(device=dev).manual_seed(1000 + rank)
    dirs = torch.randn((G, H, D), generator=gen, device=dev)
    dirs_k = dirs / dirs.norm(dim=-1, keepdim=True)
    # the direction that the one-angle rotation to position n_local - 1 (rope.py:89-104) turns into dirs_k
    inv = 1.0 / (T["base"] ** (torch.arange(0, D, 2, device=dev, dtype=torch.float64) / D))
    ang = (T["n_local"] - 1) * inv
    x1, x2 = dirs_k[..., :D // 2].double(), dirs_k[..., D // 2:].double()
    dirs_q = torch.cat((x1 * ang.cos() + x2 * ang.sin(), x2 * ang.cos() - x1 * ang.sin()), dim=-1).float()
    n_units = (tokens - T["n_init"]) // T["bs"] + 1
    unit_gain = 1.0 + 0.3 * torch.rand((n_units,), generator=gen, device=dev)
    chunks = [thrash_chunk(dev, s0, min(T["chunk"], tokens - s0), dirs_k, dirs_q, unit_gain, gen)
              for s0 in range(0, tokens, T["chunk"])]
    cm = ContextManager(rope, T["n_init"], T["n_local"], T["bs"], T["max_cached"], T["topk"], T["exc"], None, True,
                        T["repr_topk"])

    def prompt():
        cm.reset()
        o = None
        for q, k, v in chunks:
            o = cm.append(q[None], k[None], v[None], q[None], k[None], v[None])
        return o

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    steps, warm = max(1, min(args.steps, 2)), 3
    with torch.inference_mode():
        for _ in range(warm):
            prompt()
        barrier()
        clk_p, clk_f = sample_clocks_start(local_rank)
        l0 = _lib.lib.infllm_launch_count()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            prompt()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        launches = _lib.lib.infllm_launch_count() - l0
        info = cm.info()
        clocks = sample_clocks_stop(clk_p, clk_f)
        cm.trace(True)
        prompt()
        trace = cm.get_trace()
        overlap = ContextManager.refill_overlap(trace)
        cm.trace(False)
        # how many of the exec blocks past the first 2 * G * topk units evicted the whole cache
        last = cm.last_topk()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.item()
    n_eb = tokens // T["exc"]
    groups_last = sorted({b % G for b in last[-1]}) if last else []
    return dict(
        metric="cache-thrash prefill tokens/s/GPU (max_cached == topk)", value=world * tokens * steps / (ms / 1e3),
        unit="tokens/s", n_gpus=world, steps=steps, warmup=warm, ms_per_step=ms / steps, higher_is_better=True,
        scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload=f"qwen-1.5-7b-shaped attention layer (32q/32kv, d128, rope 1e6), {tokens}-token prefill in "
                             f"8192-token calls, exec 256, n_local 4096, unit 128 (2 MiB), topk 16, repr_topk 8, "
                             f"max_cached 16; {G} unit groups, exec block t retrieves group t % {G}",
                    literal_max_cached_8=("refused: " + refused) if refused else "NOT refused",
                    l2="16 units x 2 MiB refilled per exec block exceed nothing by themselves; the 4 GiB of q/k/v per "
                       "131072 tokens do", replicas=world),
        gpu_launches=int(launches),
        store=dict(misses_per_exec_block=info["cache_misses"] / max(n_eb, 1), evictions_per_exec_block=info["evictions"] / max(n_eb, 1),
                   h2d_bytes_per_exec_block=info["h2d_bytes"] / max(n_eb, 1), h2d_late_bytes=info["h2d_late_bytes"],
                   h2d_gbs=info["h2d_bytes"] / (ms / steps / 1e3) / 1e9,
                   h2d_overlap_frac=overlap["overlap_frac"], h2d_hidden_frac=overlap["hidden_frac"],
                   refill_copy_ms_per_step=overlap["copy_ms"], groups_in_last_retrieval=groups_last),
        clocks=clocks)


def sharded_decode_selfcheck(rank, world, dev, mailbox_on=True, tokens=48):
    """Untimed: a small memory (64 units per rank, bench head shape) decoded for `tokens` tokens through the unit-range
    shards of all ranks, and on rank 0 also through one unsharded context: same retrievals (a flip or two on a near-tie
    allowed) and outputs within 2e-2 wherever the retrievals agree.  Returns {ok, tokens, flips, max_abs} on every rank."""
    import torch.distributed as dist

    from infllm_b200.attention import (ContextManager, PeerMailbox, RotaryEmbeddingESM, ShardedDecodeMemory, UnitRangeShard,
                                       unit_range)

    H, HKV, D, bs, topk = CFG["H"], CFG["HKV"], CFG["D"], DEC["bs"], DEC["topk"]
    n, n_local, n_init = 64 * world, 1024, DEC["n_init"]
    rope = RotaryEmbeddingESM(D, CFG["base"], 1.0)
    g = torch.Generator().manual_seed(4321)  # the same on every rank
    bf = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16)  # noqa: E731
    units, block_k = bf(n, 2, HKV, bs, D), torch.randn(n, H * D, generator=g)
    direction = torch.randn(H, 1, D, generator=g)
    direction = direction / direction.norm(dim=-1, keepdim=True)
    rot = rope.apply_rotary_pos_emb_one_angle(direction.to(torch.bfloat16)[None].to(dev), n_local)[0].float().cpu().reshape(-1)
    planted = torch.randperm(n, generator=g)[:topk + 8]
    block_k[planted] = 0.7 * block_k[planted] + torch.linspace(9.0, 3.0, topk + 8)[:, None] * rot
    block_k = block_k.to(torch.bfloat16)
    init_k, init_v, win_k, win_v = bf(HKV, n_init, D), bf(HKV, n_init, D), bf(HKV, n_local, D), bf(HKV, n_local, D)
    toks = [((torch.randn(H, 1, D, generator=g) + 3.0 * direction).to(torch.bfloat16), bf(HKV, 1, D), bf(HKV, 1, D))
            for _ in range(tokens)]
    lo, hi = unit_range(n, rank, world)
    sh = UnitRangeShard(rank, world, rope, n_init, n_local, bs, DEC["max_cached"], topk, DEC["repr_topk"], H, HKV, D,
                        torch.bfloat16, dev)
    sh.load_synthetic(n, units[lo:hi], block_k[lo:hi], init_k, init_v, win_k, win_v)
    mb = PeerMailbox(topk, H, D, device=dev) if (world > 1 and mailbox_on) else None
    mem = ShardedDecodeMemory([sh], distributed=world > 1, mailbox=mb)
    outs, ids = [], []
    for q, k, v in toks:
        outs.append(mem.append(q.to(dev), k.to(dev), v.to(dev)).float())
        ids.append(list(mem.last_ids))
    torch.cuda.synchronize()
    res = torch.zeros(3, dtype=torch.float64, device=dev)  # ok, flips, max_abs
    if rank == 0:
        cm = ContextManager(rope, n_init, n_local, bs, DEC["max_cached"], topk, DEC["exc"], None, True, DEC["repr_topk"])
        cm.load_synthetic(units, block_k, init_k, init_v, win_k, win_v)
        flips, worst = 0, 0.0
        for i, (q, k, v) in enumerate(toks):
            dq, dk, dv = (t[None].to(dev) for t in (q, k, v))
            want = cm.append(dq, dk, dv, dq, dk, dv)[0].float()
            if sorted(cm.last_topk()[0]) != sorted(ids[i]):
                flips += 1
                continue
            worst = max(worst, (outs[i] - want).abs().max().item())
        res[0], res[1], res[2] = float(flips <= 2 and worst <= 2e-2), flips, worst
    if world > 1:
        dist.broadcast(res, 0)
        dist.barrier()
    if mb is not None:
        mb.close()
    return dict(ok=bool(res[0].item()), tokens=tokens, retrieval_flips=int(res[1].item()), max_abs=res[2].item(),
                against="one unsharded context on rank 0 over the same 64-units-per-rank memory")


def head_groups_selfcheck(rank, world, dev, comm, tokens=16384):
    """Untimed: a `tokens`-token prompt through one layer sharded by KV-head groups over all ranks, and on rank 0 also
    through the whole layer.  Per exec block: the retrieved unit sets, and the outputs (within 2 % of their range) for
    as long as the two runs have retrieved the same units.  The two runs do not use the same attention kernel (few
    heads per GPU take the two-heads-per-CTA kernel), so their accumulated local scores differ in the last bits and a
    representative key can be built from another of several tied tokens; from then on the retrievals may differ
    legitimately.  ok = every exec block before the first difference agrees in its outputs (that prefix holds at least
    the exec blocks that retrieve every unit there is) and the retrieved sets overlap by 80 % or more over the prompt."""
    import torch.distributed as dist

    from infllm_b200.attention import ATTN_FORWRAD, RotaryEmbeddingESM

    mk = lambda c: ATTN_FORWRAD["inf-llm"](  # noqa: E731
        n_local=CFG["n_local"], n_init=CFG["n_init"], topk=CFG["topk"], block_size=CFG["bs"], max_cached_block=CFG["max_cached"],
        exc_block_size=CFG["exc"], fattn=True, repr_topk=CFG["repr_topk"], head_group_comm=c)
    full = make_weights(dev, torch.bfloat16)
    hidden = make_hidden(tokens, seed=77, weights=full, device=dev)
    rope = RotaryEmbeddingESM(CFG["D"], CFG["base"], 1.0)

    def run(layer):
        outs, ids = [], []
        for s0 in range(0, tokens, CFG["chunk"]):
            outs.append(layer(hidden[:, s0:s0 + CFG["chunk"]]))
            ids += layer.pkv.last_topk()
        return torch.cat(outs, dim=1), ids

    res = torch.zeros(5, dtype=torch.float64, device=dev)
    with torch.inference_mode():
        got, ids = run(Layer(dev, mk(comm), rope, rank=rank, world=world))
        if rank == 0:
            want, want_ids = run(Layer(dev, mk(None), rope))
            n_eb = len(want_ids)
            same = [sorted(a) == sorted(b) for a, b in zip(ids, want_ids)]
            prefix = same.index(False) if False in same else n_eb
            scored = [i for i in range(n_eb) if len(want_ids[i]) == CFG["topk"]]
            overlap = (sum(len(set(ids[i]) & set(want_ids[i])) for i in scored) / max(1, CFG["topk"] * len(scored)))
            scale = want.float().abs().max().item()
            upto = prefix * CFG["exc"]
            worst = (got[:, :upto].float() - want[:, :upto].float()).abs().max().item() / scale if upto else 0.0
            first_scored = scored[0] if scored else n_eb
            ok = worst <= 0.02 and prefix >= first_scored and overlap >= 0.8
            res[0], res[1], res[2], res[3], res[4] = float(ok), prefix, n_eb, overlap, worst
    dist.broadcast(res, 0)
    dist.barrier()
    return dict(ok=bool(res[0].item()), tokens=tokens, exec_blocks=int(res[2].item()),
                exec_blocks_before_first_retrieval_difference=int(res[1].item()), retrieved_set_overlap=res[3].item(),
                max_abs_over_range_before_it=res[4].item(), against="the whole layer on rank 0")


def run_decode_sharded(args, rank, world, local_rank):
    """The 1M-token decode with the memory sharded by unit range over the ranks (strong scaling: one sequence)."""
    import torch.distributed as dist

    from infllm_b200 import _lib
    from infllm_b200.attention import PeerMailbox, RotaryEmbeddingESM, ShardedDecodeMemory, UnitRangeShard, unit_range

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    H, HKV, D, n, bs = CFG["H"], CFG["HKV"], CFG["D"], DEC["units"], DEC["bs"]
    rope = RotaryEmbeddingESM(D, CFG["base"], 1.0)
    # per-rank working set of one layer shrinks with the world size: more layers take turns to stay above L2
    n_layers = DEC["layers"] * world
    lo, hi = unit_range(n, rank, world)
    mems, dirs = [], []
    # one mailbox for all layers: both exchanges of a token run inside kernels over peer memory (--nccl-exchange
    # keeps them as NCCL all-gathers with a host round trip between them)
    mailbox = PeerMailbox(DEC["topk"], H, D, device=dev) if (world > 1 and not args.nccl_exchange) else None
    for li in range(n_layers):
        gs = torch.Generator(device=dev).manual_seed(7000 + li)  # the same on every rank
        direction = torch.randn((H, 1, D), generator=gs, device=dev)
        direction = direction / direction.norm(dim=-1, keepdim=True)
        rotated = rope.apply_rotary_pos_emb_one_angle(direction.to(torch.bfloat16)[None], DEC["n_local"])[0].float().reshape(-1)
        small = lambda *shape: torch.randn(shape, generator=gs, device=dev).to(torch.bfloat16).cpu()  # noqa: E731
        init_k, init_v = small(HKV, DEC["n_init"], D), small(HKV, DEC["n_init"], D)
        win_k, win_v = small(HKV, DEC["n_local"], D), small(HKV, DEC["n_local"], D)
        n_plant = max(1, int(n * DEC["planted_frac"]))
        planted = torch.randperm(n, generator=torch.Generator().manual_seed(7100 + li))[:n_plant]
        lean = torch.linspace(9.0, 3.0, n_plant)
        gr = torch.Generator(device=dev).manual_seed(9000 + 131 * li + rank)  # this rank's own units
        units = torch.empty((hi - lo, 2, HKV, bs, D), dtype=torch.bfloat16)
        for s0 in range(0, hi - lo, 512):
            m = min(512, hi - lo - s0)
            units[s0:s0 + m] = torch.randn((m, 2, HKV, bs, D), generator=gr, device=dev).to(torch.bfloat16).cpu()
        block_k = torch.randn((hi - lo, H * D), generator=gr, device=dev)
        for b, a in zip(planted.tolist(), lean.tolist()):
            if lo <= b < hi:
                block_k[b - lo] = 0.7 * block_k[b - lo] + a * rotated
        sh = UnitRangeShard(rank, world, rope, DEC["n_init"], DEC["n_local"], bs, DEC["max_cached"], DEC["topk"],
                            DEC["repr_topk"], H, HKV, D, torch.bfloat16, dev)
        sh.load_synthetic(n, units, block_k.to(torch.bfloat16).cpu(), init_k, init_v, win_k, win_v)
        del units, block_k
        mems.append(ShardedDecodeMemory([sh], distributed=world > 1, mailbox=mailbox))
        dirs.append(direction)
    total = (args.warmup + 2 * args.steps + 2 + 32) * n_layers
    g = torch.Generator(device=dev).manual_seed(100)  # the same token stream on every rank
    lean_q = torch.stack([dirs[i % n_layers] for i in range(total)])
    qs = (torch.randn((total, H, 1, D), generator=g, device=dev) + 3.0 * lean_q).to(torch.bfloat16)
    ks = torch.randn((total, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)
    vs = torch.randn((total, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)
    h_q, h_k, h_v = (t.cpu().pin_memory() for t in (qs, ks, vs))
    h_o = torch.empty((H, 1, D), dtype=torch.bfloat16).pin_memory()
    pos = [0]

    toks = [(qs[i], ks[i], vs[i]) for i in range(total)]  # views made once: the timed loop is the library's

    def step_device():
        for m in mems:
            q, k, v = toks[pos[0]]
            pos[0] += 1
            m.append(q, k, v)

    def step_host():
        for m in mems:
            i = pos[0]
            pos[0] += 1
            q, k, v = (t[i].to(dev, non_blocking=True) for t in (h_q, h_k, h_v))
            h_o.copy_(m.append(q, k, v), non_blocking=True)
            torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    with torch.inference_mode():
        parity = sharded_decode_selfcheck(rank, world, dev, mailbox_on=not args.nccl_exchange) if world > 1 else None
        clk_p, clk_f = sample_clocks_start(local_rank)  # with the warm-up: the timed region is shorter than a polling period
        for _ in range(args.warmup):
            step_device()
        shards = [m.shards[0] for m in mems]
        for sh in shards:
            sh.profile = True
            sh.hits = sh.misses = 0
        l0 = _lib.lib.infllm_launch_count()
        ms = timed(step_device, args.steps)
        launches = _lib.lib.infllm_launch_count() - l0
        prof = [sh.get_profile() for sh in shards]
        for sh in shards:
            sh.profile = False
        if sum(p["topk"][1] for p in prof) == 0:
            # the one-call token path records no events: time this rank's scoring + top-k launches on their own,
            # rotating over the layers so that the representative keys come from HBM
            import ctypes

            evs = []
            for i in range(8 * len(shards)):
                sh = shards[i % len(shards)]
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                _lib.check(_lib.lib.infllm_block_topk(sh._p["block_k"], sh.n_owned, H * D, sh._p["qbar"], sh._p["scores_buf"],
                                                      min(sh.topk, sh.n_owned), sh.lo, sh._p["cand"] + 4 * sh.topk,
                                                      sh._p["cand"], sh.code, _lib.stream_ptr()))
                b.record()
                evs.append((a, b))
            torch.cuda.synchronize()
            prof = [dict(topk=(sum(a.elapsed_time(b) for a, b in evs[len(shards):]), len(evs) - len(shards)), decode=(0.0, 0))]
        clocks = sample_clocks_stop(clk_p, clk_f)
        hits, misses = sum(sh.hits for sh in shards), sum(sh.misses for sh in shards)
        # where a token's time goes on this rank's GPU: a short pass with a one-thread timestamp kernel between the
        # token's launches (each adds about a microsecond to the phase before it; untimed)
        phases = None
        if all(sh._token_args is not None for sh in shards):
            n_st = 32
            for sh in shards:
                sh.stamps, sh.stamp_row = torch.zeros((n_st, 8), dtype=torch.int64, device=dev), 0
            for _ in range(n_st):
                step_device()
            torch.cuda.synchronize()
            st = torch.stack([sh.stamps for sh in shards]).double()[:, 4:]          # (layers, tokens, 8 stamps)
            for sh in shards:
                sh.stamps = None
            d = (st[..., 1:] - st[..., :-1]).mean(dim=(0, 1)) / 1e3                 # us
            names = ("ingest", "scoring_topk", "exchange1_rank", "attention", "local_merge", "put_partials",
                     "wait_final_merge")
            phases = {n: round(float(x), 2) for n, x in zip(names, d)}
            phases["token_on_device"] = round(float((st[..., 7] - st[..., 0]).mean() / 1e3), 2)
            phases["note"] = "mean over the layers' last tokens of a 32-token pass; rank %d" % rank
        step_host()
        ms_e2e = timed(step_host, args.steps)
    _, hbm_peak, which = measured_peaks()
    per_layer = args.steps * n_layers
    topk_ms = sum(p["topk"][0] for p in prof)
    topk_n = sum(p["topk"][1] for p in prof)
    dec_ms = sum(p["decode"][0] for p in prof)
    dec_n = sum(p["decode"][1] for p in prof)
    topk_bytes = float(hi - lo) * H * D * 2
    achieved = topk_bytes * topk_n / (topk_ms / 1e3) / 1e9 if topk_ms > 0 else None
    counts = torch.tensor([hits, misses], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(counts)
    line = dict(
        metric="decode-attn us/token @1M ctx", value=1e3 * ms / per_layer, unit="us/token", n_gpus=world,
        steps=args.steps, warmup=args.warmup, ms_per_step=ms / args.steps, higher_is_better=False, scaling="strong",
        vs_baseline=None, dtype="bf16", data="synthetic",
        config=dict(workload=f"mistral-7b-shaped layer, decode over {n} memory units of 128 tokens "
                             f"({DEC['n_init'] + n * bs + DEC['n_local']} tokens) sharded by unit range over {world} GPUs, "
                             "topk 32, repr_topk 4, max_cached 32 per GPU, n_local 4096, n_init 128; 1% planted units "
                             f"with graded lean; a step is one token through {n_layers} layers, value is per layer",
                    l2=f"{n_layers} layers take turns so that each rank's working set exceeds the 126 MB L2",
                    parallelism=(f"unit-range x{world}: (score, id) candidates and (o, lse) partials exchanged per token "
                                 + ("by kernels that write the peers' mailboxes (CUDA IPC), retrieval ranked on the "
                                    "device" if mailbox is not None else "by NCCL all-gathers")
                                 + "; all-reduce of 128 score columns per sealed unit (NCCL)"),
                    tokens_redone=sum(m.redone for m in mems)),
        parity=parity,
        e2e=dict(value=1e3 * ms_e2e / per_layer, unit="us/token", h2d_bytes_per_step=int((H + 2 * HKV) * D * 2 * n_layers),
                 d2h_bytes_per_step=int(H * D * 2 * n_layers)),
        gpu_launches=int(launches),
        roofline=dict(bound="hbm", kernel="block_score_topk_kernel + topk_fast_kernel (this rank's units)",
                      achieved=achieved, peak=hbm_peak, unit="GB/s", frac=(achieved / hbm_peak if achieved else None),
                      traffic=None, peak_source=f"hbm_gbs of {which}", launches=int(topk_n),
                      us_per_launch=1e3 * topk_ms / max(topk_n, 1), bytes_per_launch=topk_bytes),
        decode_attention=dict(kernels="attn_decode_kernel + lse_merge_kernel (rank 0)",
                              us_per_launch=1e3 * dec_ms / max(dec_n, 1)),
        store=dict(hits=int(counts[0].item()), misses=int(counts[1].item()),
                   miss_rate=counts[1].item() / max(counts.sum().item(), 1)),
        phases_us=phases,
        clocks=clocks)
    return line


def run_model(args, rank, world, local_rank):
    """A Llama-3-8B-shaped random-init decoder (32 layers, 32/8 heads of 128, FFN 14336) over the attention-forward
    API: chunked prefill of a synthetic prompt, then greedy tokens.  With N > 1 the model is split by KV-head groups
    (strong scaling).  Not part of the default run: the headline metric is the layer's."""
    from infllm_b200.attention import HeadGroupComm
    from infllm_b200.utils import HeadGroupDecoder

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = HeadGroupComm() if world > 1 else None
    attn = dict(n_local=CFG["n_local"], n_init=CFG["n_init"], topk=CFG["topk"], block_size=CFG["bs"],
                max_cached_block=CFG["max_cached"], exc_block_size=CFG["exc"], fattn=True, repr_topk=CFG["repr_topk"])
    dec = HeadGroupDecoder(32, 4096, CFG["H"], CFG["HKV"], CFG["D"], 14336, 128256, attn, rank=rank, world=world,
                           comm=comm, seed=0, device=dev, rope_base=500000.0)
    g = torch.Generator().manual_seed(0)
    tokens = args.tokens or CFG["tokens"]
    h_ids = torch.randint(0, 128256, (1, tokens), generator=g).pin_memory()
    n_new = 64

    def prompt():
        dec.reset()
        logits = None
        for st in range(0, tokens, CFG["chunk"]):
            logits = dec.step(h_ids[:, st:st + CFG["chunk"]].to(dev, non_blocking=True))
        return logits

    for _ in range(1 if tokens >= 131072 else max(1, min(args.warmup, 2))):
        prompt()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    ms_prefill = ms_decode = 0.0
    out_ids, prints = [], []
    for _ in range(args.steps):
        ev[0].record()
        logits = prompt()
        ev[1].record()
        for i in range(n_new):
            nxt = logits.argmax(dim=-1)
            out_ids.append(int(nxt))
            if i < 4 and len(prints) < 4:  # to compare runs on other GPU counts with: the chosen token and its margin
                top = logits.float().flatten().topk(2).values
                prints.append(dict(token=int(nxt), logit=round(top[0].item(), 4), margin=round((top[0] - top[1]).item(), 4),
                                   logit_range=round((logits.float().max() - logits.float().min()).item(), 3)))
            logits = dec.step(nxt[:, None])
        ev[2].record()
        torch.cuda.synchronize()
        ms_prefill += ev[0].elapsed_time(ev[1])
        ms_decode += ev[1].elapsed_time(ev[2])
    t = torch.tensor([ms_prefill, ms_decode], device=dev)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_prefill, ms_decode = (t / args.steps).tolist()
    del dec
    if comm is not None:
        comm.close()
    return dict(metric="whole-model chunked prefill tokens/s (Llama-3-8B shape, random weights)",
                value=tokens / (ms_prefill / 1e3), unit="tokens/s", n_gpus=world, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms_prefill, higher_is_better=True,
                scaling="strong" if world > 1 else "weak", vs_baseline=None, dtype="bf16", data="synthetic",
                config=dict(workload=f"32-layer decoder, {tokens}-token prompt in chunks of {CFG['chunk']}, "
                                     f"exec blocks of {CFG['exc']}, then {n_new} greedy tokens; host token ids",
                            parallelism=f"kv-head-groups{world}" if world > 1 else "single"),
                decode_ms_per_token=ms_decode / n_new, greedy_tokens=out_ids[:n_new], first_steps=prints,
                pinned_store_gib=32 * (tokens - CFG["n_init"] - CFG["n_local"]) // CFG["bs"] * 524288 / world / 2 ** 30)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="default 3 (prefill prompts) or 256 (decode tokens)")
    ap.add_argument("--warmup", type=int, default=None,
                    help="default 3 (prefill) or 136 (decode: past the first sealing, whose one-time growth of the "
                         "representative-key array would otherwise sit in the timed region)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=None,
                    help="prompt length: default 131072 (prefill, model) or 524288 (thrash)")
    ap.add_argument("--workload", default="both", choices=["both", "prefill", "decode", "model", "thrash"],
                    help="prefill: 131072-token prompt, the first half of the metric and the line's value; decode: the "
                         "1M-token decode, the second half; both (default): the prefill line with the decode line "
                         "under its key 'decode'")
    ap.add_argument("--decode-steps", type=int, default=128, help="decode tokens timed when --workload both")
    ap.add_argument("--head-groups", action="store_true",
                    help="prefill with N > 1: one layer sharded by KV-head groups over the GPUs instead of N replicas")
    ap.add_argument("--nccl-exchange", action="store_true",
                    help="sharded decode: exchange candidates and partials with NCCL all-gathers instead of peer-memory kernels")
    ap.add_argument("--sharded", action="store_true",
                    help="decode through the unit-range sharded implementation even on one GPU (it is what N > 1 runs)")
    ap.add_argument("--units", type=int, default=DEC["units"], help="memory units of the decode workload")
    ap.add_argument("--layers", type=int, default=DEC["layers"], help="layer memories that take turns in the decode workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-ref-gpu", action="store_true", help="reference arm: skip the timing of the reference's Triton kernel")
    ap.add_argument("--device-store-mb", type=int, default=0,
                    help="decode workload alone: MiB per layer of device copy of the store (0 = pinned host store only)")
    ap.add_argument("--max-cached", type=int, default=CFG["max_cached"], help="max_cached_block (32 in the named config)")
    args = ap.parse_args()
    CFG["max_cached"] = args.max_cached
    DEC["units"] = args.units
    DEC["layers"] = max(1, args.layers)
    if args.steps is None:
        args.steps = 256 if args.workload == "decode" else (1 if args.workload == "model" else 3)
    if args.warmup is None:
        args.warmup = 136 if args.workload == "decode" else 3
    args.warmup = max(args.warmup, 3)  # fewer warm-up steps would time cold caches and first-use allocations
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU arm)")
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.device_store_mb and not (world > 1 or args.sharded):
        import functools

        decode = functools.partial(run_decode, device_store_mb=args.device_store_mb)
    else:
        decode = run_decode_sharded if (world > 1 or args.sharded) else run_decode
    if args.workload == "decode":
        line = decode(args, rank, world, local_rank)
    elif args.workload == "model":
        line = run_model(args, rank, world, local_rank)
    elif args.workload == "thrash":
        line = run_thrash(args, rank, world, local_rank)
    else:
        line = run_ours(args, rank, world, local_rank)
        import copy
        import gc

        if not args.head_groups:
            gc.collect()
            torch.cuda.empty_cache()
            vargs = copy.copy(args)
            vargs.steps = min(args.steps, 2)
            line["device_store"] = run_ours(vargs, rank, world, local_rank, device_store_mb=1024, light=True)
        if args.workload == "both":

            gc.collect()
            torch.cuda.empty_cache()
            dargs = copy.copy(args)
            dargs.steps, dargs.warmup = args.decode_steps, 136
            line["decode"] = decode(dargs, rank, world, local_rank)
            if world == 1 and not args.sharded and not args.device_store_mb:
                # the same decode with a device copy of the store (refills do not cross PCIe), beside the headline
                gc.collect()
                torch.cuda.empty_cache()
                dv = run_decode(dargs, rank, world, local_rank, device_store_mb=4096)
                line["decode"]["device_store"] = {k: dv[k] for k in ("value", "unit", "ms_per_step", "roofline",
                                                                     "decode_attention", "store")}
                gc.collect()
                torch.cuda.empty_cache()
                line["thrash"] = run_thrash(args, rank, world, local_rank)
            if world > 1 and not args.head_groups and CFG["HKV"] % world == 0:
                # the same prompt through ONE layer sharded by KV-head groups over the GPUs (strong scaling)
                gc.collect()
                torch.cuda.empty_cache()
                hargs = copy.copy(args)
                hargs.head_groups, hargs.no_cpu, hargs.steps = True, True, min(args.steps, 2)
                hg = run_ours(hargs, rank, world, local_rank)
                line["head_groups"] = {k: hg[k] for k in ("value", "unit", "ms_per_step", "scaling", "e2e", "roofline", "config",
                                                           "host_ms_per_step", "parity") if k in hg}
    # the record of a run may keep only the end of this line: the figures that matter most, once more, last
    dec = line.get("decode", line if line.get("unit") == "us/token" else {})
    hg = line.get("head_groups", {})
    line["summary"] = dict(
        prefill_tokens_s=line.get("value") if line.get("unit") == "tokens/s" else None,
        prefill_e2e_tokens_s=(line.get("e2e") or {}).get("value") if line.get("unit") == "tokens/s" else None,
        prefill_roofline_frac=(line.get("roofline") or {}).get("frac") if line.get("unit") == "tokens/s" else None,
        decode_us=dec.get("value"), decode_roofline_frac=(dec.get("roofline") or {}).get("frac"),
        decode_parity_ok=(dec.get("parity") or {}).get("ok"),
        head_groups_ms=hg.get("ms_per_step"), head_groups_parity_ok=(hg.get("parity") or {}).get("ok"),
        thrash_tokens_s=(line.get("thrash") or {}).get("value"), n_gpus=world)
    if rank == 0:
        print(json.dumps(line))
    bad = [k for k in ("decode_parity_ok", "head_groups_parity_ok") if line["summary"].get(k) is False]
    if bad:
        raise SystemExit(f"self-check failed: {bad}")
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
