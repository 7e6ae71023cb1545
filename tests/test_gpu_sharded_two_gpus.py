"""Unit-range sharded decode on two GPUs with the exchanges inside kernels over peer memory (PeerMailbox): the
outputs and retrievals must equal the unsharded context's on the same synthetic memory, through refills and a
sealing.  Needs two GPUs; skipped otherwise."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

pytestmark = pytest.mark.gpu

H, HKV, D, UNITS, STEPS = 8, 2, 128, 40, 150
CFG = dict(n_init=128, n_local=512, bs=128, max_cached=6, topk=4, exc=128, repr_topk=4, base=1e6)


PLANTED = (3, 17, 25, 33, 36)  # units whose representative keys lean towards the queries' common direction


def _direction():
    d = torch.randn(H, 1, D, generator=torch.Generator().manual_seed(4))
    return d / d.norm(dim=-1, keepdim=True)


def _memory():
    """Most tokens retrieve four of the five planted units (two per rank), so after the first refills the caches
    hold what is retrieved and only now and then a token finds a unit missing."""
    from infllm_b200.attention import RotaryEmbeddingESM

    g = torch.Generator().manual_seed(5)
    bf = lambda *shape: torch.randn(*shape, generator=g).to(torch.bfloat16)  # noqa: E731
    units, block_k = bf(UNITS, 2, HKV, 128, D), torch.randn(UNITS, H * D, generator=g)
    pe = RotaryEmbeddingESM(D, CFG["base"], 1.0)
    rot = pe.apply_rotary_pos_emb_one_angle(_direction().to(torch.bfloat16)[None].cuda(), CFG["n_local"])[0]
    rot = rot.float().cpu().reshape(-1)
    for i, b in enumerate(PLANTED):
        block_k[b] = 0.5 * block_k[b] + (8.0 - i) * rot
    return units, block_k.to(torch.bfloat16), bf(HKV, 128, D), bf(HKV, 128, D), bf(HKV, 512, D), bf(HKV, 512, D)


def _tokens():
    g = torch.Generator().manual_seed(6)
    d = _direction()
    return [((torch.randn(H, 1, D, generator=g) + 3.0 * d).to(torch.bfloat16),
             torch.randn(HKV, 1, D, generator=g).to(torch.bfloat16), torch.randn(HKV, 1, D, generator=g).to(torch.bfloat16))
            for _ in range(STEPS)]


def _run(rank, world, port, path, use_mailbox):
    import torch.distributed as dist

    from infllm_b200.attention import PeerMailbox, RotaryEmbeddingESM, ShardedDecodeMemory, UnitRangeShard, unit_range

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        units, block_k, init_k, init_v, win_k, win_v = _memory()
        lo, hi = unit_range(UNITS, rank, world)
        sh = UnitRangeShard(rank, world, RotaryEmbeddingESM(D, CFG["base"], 1.0), CFG["n_init"], CFG["n_local"], CFG["bs"],
                            CFG["max_cached"], CFG["topk"], CFG["repr_topk"], H, HKV, D, torch.bfloat16, dev, spare_units=1)
        sh.load_synthetic(UNITS, units[lo:hi], block_k[lo:hi], init_k, init_v, win_k, win_v)
        mb = PeerMailbox(CFG["topk"], H, D) if use_mailbox else None
        mem = ShardedDecodeMemory([sh], distributed=True, mailbox=mb)
        outs, ids = [], []
        for q, k, v in _tokens():
            outs.append(mem.append(q.to(dev), k.to(dev), v.to(dev)).float().cpu())
            ids.append(list(mem.last_ids))
        torch.save((torch.stack(outs), ids, mem.redone, sh.n_total), f"{path}.{rank}")
        torch.cuda.synchronize()
        if mb is not None:
            dist.barrier()
            mb.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("use_mailbox", [True, False])
def test_two_ranks_match_the_unsharded_context(tmp_path, use_mailbox):
    from infllm_b200.attention import ContextManager, RotaryEmbeddingESM

    path = str(tmp_path / "out")
    mp.spawn(_run, args=(2, 29700 + os.getpid() % 200 + int(use_mailbox), path, use_mailbox), nprocs=2, join=True)
    parts = [torch.load(f"{path}.{r}") for r in range(2)]
    assert parts[0][1] == parts[1][1], "the ranks ranked different retrievals"
    assert (parts[0][0] - parts[1][0]).abs().max().item() == 0.0, "the ranks merged different outputs"
    assert parts[0][3] == UNITS + 1  # one unit sealed on the way
    assert parts[0][2] == parts[1][2] == 0  # no token is run twice: a unit that is not cached is read where it lives
    dev = torch.device("cuda", 0)
    cm = ContextManager(RotaryEmbeddingESM(D, CFG["base"], 1.0), CFG["n_init"], CFG["n_local"], CFG["bs"],
                        CFG["max_cached"], CFG["topk"], CFG["exc"], None, False, CFG["repr_topk"])
    cm.load_synthetic(*_memory())
    flips = 0
    for i, (q, k, v) in enumerate(_tokens()):
        dq, dk, dv = (t[None].to(dev) for t in (q, k, v))
        want = cm.append(dq, dk, dv, dq, dk, dv)[0].float().cpu()
        same = cm.last_topk()[0] == parts[0][1][i]
        flips += not same
        if same:
            assert (parts[0][0][i] - want).abs().max().item() <= 2e-2, f"token {i}"
    assert flips <= 5
