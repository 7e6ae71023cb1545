"""Host-side protocol of the unit-range sharded decode, without a GPU: the driver (candidate gather, global
top-k, partial gather, merge, score all-reduce at a sealing) runs over stand-in shards that do the per-rank math
in plain torch on the CPU — once with every rank in this process, once as two gloo processes — and must give
what one unsharded rank gives."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from infllm_b200.attention.sharded_decode import ShardedDecodeMemory, global_topk, unit_range  # noqa: E402

H, HKV, D, BS, N_INIT, N_LOCAL, TOPK, REPR, UNITS, STEPS = 4, 2, 16, 8, 4, 16, 3, 2, 13, 40
LOG2E = 1.4426950408889634


class CpuShard:
    """The interface of UnitRangeShard (begin / attend / finish / seal) in fp32 torch, no RoPE, no cache."""

    def __init__(self, rank, world, seed=0):
        self.rank, self.world, self.topk, self.H, self.D, self.dtype = rank, world, TOPK, H, D, torch.float32
        g = torch.Generator().manual_seed(seed)
        units = torch.randn(UNITS, 2, HKV, BS, D, generator=g)
        block_k = torch.randn(UNITS, H * D, generator=g)
        self.init = torch.randn(2, HKV, N_INIT, D, generator=g)
        win = torch.randn(2, HKV, N_LOCAL, D, generator=g)
        lo, hi = unit_range(UNITS, rank, world)
        self.lo, self.units, self.block_k = lo, list(units[lo:hi]), list(block_k[lo:hi])
        self.n_total = UNITS
        self.k, self.v = win[0].clone(), win[1].clone()  # tokens [frontier, length)
        self.score = torch.zeros(H, N_LOCAL)
        self.frontier = N_INIT + UNITS * BS
        self.length = self.frontier + N_LOCAL

    def _heads(self, x):  # (HKV, n, D) -> (H, n, D)
        return x.repeat_interleave(H // HKV, dim=0)

    def begin(self, q, k, v):
        self.k, self.v = torch.cat((self.k, k), dim=1), torch.cat((self.v, v), dim=1)
        self.score = torch.cat((self.score, torch.zeros(H, 1)), dim=1)
        self.q = q[:, 0]
        cand = torch.full((2, TOPK), -1, dtype=torch.int32)
        cand[0] = torch.full((TOPK,), float("-inf")).view(torch.int32)
        if self.block_k:
            s = torch.stack(self.block_k) @ self.q.reshape(-1)
            kk = min(TOPK, len(self.block_k))
            best = torch.tensor(global_topk(s, torch.arange(len(self.block_k), dtype=torch.int32), kk))
            cand[0, :kk] = s[best].view(torch.int32)
            cand[1, :kk] = (best + self.lo).to(torch.int32)
        return cand

    def attend(self, ids):
        ks, vs = [], []
        for b in ids:
            if self.lo <= b < self.lo + len(self.units):
                ks.append(self.units[b - self.lo][0])
                vs.append(self.units[b - self.lo][1])
        n = self.k.size(1)
        wlo = n - N_LOCAL  # slot of the first window token
        a, b_ = wlo + (N_LOCAL * self.rank) // self.world, wlo + (N_LOCAL * (self.rank + 1)) // self.world
        self.share = (a, b_)
        first = sum(x.size(1) for x in ks)  # where the window share starts among this rank's keys
        ks.append(self.k[:, a:b_])
        vs.append(self.v[:, a:b_])
        if self.rank == 0:
            ks.append(self.init[0])
            vs.append(self.init[1])
        if self.rank == self.world - 1 and wlo > 0:
            ks.append(self.k[:, :wlo])
            vs.append(self.v[:, :wlo])
        kk, vv = self._heads(torch.cat(ks, dim=1)), self._heads(torch.cat(vs, dim=1))
        logit = torch.einsum("hd,hnd->hn", self.q, kk) * (LOG2E / D ** 0.5)
        self.win_logit = logit[:, first:first + (b_ - a)]
        lse = torch.logsumexp(logit * 0.6931471805599453, dim=1) * LOG2E
        o = torch.einsum("hn,hnd->hd", torch.exp2(logit - lse[:, None]), vv)
        return torch.cat((o.reshape(-1), lse))

    def merge(self, parts):
        part_o, part_lse = parts[:, :H * D].reshape(-1, H, D), parts[:, H * D:]
        mx = part_lse.max(dim=0).values
        w = torch.exp2(part_lse - mx)
        out = (w[:, :, None] * part_o).sum(dim=0) / w.sum(dim=0)[:, None]
        lse = mx + torch.log2(w.sum(dim=0))
        a, b = self.share
        self.score[:, a:b] += torch.exp2(self.win_logit - lse[:, None])
        return out

    def finish(self):
        self.length += 1
        if self.length - self.frontier - BS >= N_LOCAL:
            return self.score[:, :BS].contiguous()
        return None

    def seal(self, scores):
        if self.rank == self.world - 1:
            idx = scores.topk(REPR, dim=1).indices  # (H, REPR)
            kh = self._heads(self.k[:, :BS])
            self.block_k.append(torch.gather(kh, 1, idx[:, :, None].expand(-1, -1, D)).mean(dim=1).reshape(-1))
            self.units.append(torch.stack((self.k[:, :BS], self.v[:, :BS])))
        self.k, self.v, self.score = self.k[:, BS:], self.v[:, BS:], self.score[:, BS:]
        self.frontier += BS
        self.n_total += 1


def token(step):
    g = torch.Generator().manual_seed(1000 + step)
    return torch.randn(H, 1, D, generator=g), torch.randn(HKV, 1, D, generator=g), torch.randn(HKV, 1, D, generator=g)


def run(memory):
    outs, ids = [], []
    for step in range(STEPS):
        outs.append(memory.append(*token(step)))
        ids.append(list(memory.last_ids))
    return torch.stack(outs), ids


def test_global_topk_orders_by_score_then_id():
    s = torch.tensor([1.0, 5.0, 5.0, -2.0, 7.0, float("-inf")])
    i = torch.tensor([9, 4, 2, 1, 8, -1], dtype=torch.int32)
    assert global_topk(s, i, 3) == [8, 2, 4]
    assert global_topk(s, i, 10) == [8, 2, 4, 9, 1]  # padding never comes back


def test_unit_ranges_cover_every_unit_once():
    for n, g in ((8192, 8), (13, 2), (5, 8), (0, 4)):
        spans = [unit_range(n, r, g) for r in range(g)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))


@pytest.mark.parametrize("world", [2, 3])
def test_emulated_ranks_match_one_rank(world):
    want, want_ids = run(ShardedDecodeMemory([CpuShard(0, 1)]))
    got, got_ids = run(ShardedDecodeMemory([CpuShard(r, world) for r in range(world)]))
    assert got_ids == want_ids
    assert (got - want).abs().max().item() < 1e-4
    assert STEPS // BS >= 4  # several units sealed on the way


def _worker(rank, world, port, path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        got, ids = run(ShardedDecodeMemory([CpuShard(rank, world)], distributed=True))
        torch.save((got, ids), f"{path}.{rank}")
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_match_one_rank(tmp_path):
    want, want_ids = run(ShardedDecodeMemory([CpuShard(0, 1)]))
    path = str(tmp_path / "out")
    mp.spawn(_worker, args=(2, 29500 + os.getpid() % 1000, path), nprocs=2, join=True)
    for rank in range(2):
        got, ids = torch.load(f"{path}.{rank}")
        assert ids == want_ids
        assert (got - want).abs().max().item() < 1e-4


def _worker_that_leaves(rank, world, port, path):
    """Rank 1 takes part in three tokens and then leaves between steps; rank 0 goes on to a fourth token."""
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    mem = ShardedDecodeMemory([CpuShard(rank, world)], distributed=True)
    g = torch.Generator().manual_seed(1)
    toks = [(torch.randn(H, 1, D, generator=g), torch.randn(HKV, 1, D, generator=g), torch.randn(HKV, 1, D, generator=g))
            for _ in range(4)]
    outs = [mem.append(*t) for t in toks[:3]]
    if rank == 1:
        torch.save("left", f"{path}.1")
        os._exit(0)  # no goodbye: the peer finds out at its next collective
    try:
        mem.append(*toks[3])
        verdict = "no error"
    except Exception as e:  # the gather of the candidates cannot complete: a timeout or a closed connection
        verdict = f"error: {type(e).__name__}"
    torch.save((verdict, torch.stack(outs)), f"{path}.0")
    os._exit(0)


def test_a_rank_that_leaves_ends_the_next_exchange_with_an_error(tmp_path):
    """Failure detection on the host: when a rank is gone, the other rank's next collective ends with an error
    within the process group's (short) timeout instead of hanging, and what was computed before stays valid."""
    path = str(tmp_path / "out")
    mp.spawn(_worker_that_leaves, args=(2, 30500 + os.getpid() % 1000, path), nprocs=2, join=True)
    verdict, outs = torch.load(f"{path}.0")
    assert verdict.startswith("error"), verdict
    want = ShardedDecodeMemory([CpuShard(0, 1)])
    g = torch.Generator().manual_seed(1)
    for i in range(3):
        t = (torch.randn(H, 1, D, generator=g), torch.randn(HKV, 1, D, generator=g), torch.randn(HKV, 1, D, generator=g))
        assert (want.append(*t) - outs[i]).abs().max().item() < 1e-4
