"""KV-head-group sharding of the context memory across GPUs (no counterpart in the reference, which keeps all
heads of a layer on one GPU).

Each rank projects and keeps only its slice of the query and KV heads (tensor-parallel attention).  Everything in
the context memory is per head — window, sink, sealing, representative keys, attention — except the retrieval
score of a memory unit, which the reference forms from the mean query of ALL heads
(inf_llm/attention/context_manager.py:373-378).  With a `HeadGroupComm` every context sums its partial scores
over the ranks (an NCCL all-reduce of one float per unit) before ranking them, so all ranks retrieve the same units
and keep the same LRU order; a rank stores only its heads' slice of every unit.
"""
import ctypes

import torch

from .. import _lib


class HeadGroupComm:
    """The communicator shared by the contexts of this process.  Collective: every rank of `group` constructs it."""

    def __init__(self, group=None, device=None):
        import torch.distributed as dist

        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        n = int(_lib.lib.infllm_comm_id_bytes())
        ident = (ctypes.c_ubyte * n)()
        if self.rank == 0:
            _lib.check(_lib.lib.infllm_comm_unique_id(ident))
        t = torch.tensor(list(ident), dtype=torch.uint8, device=device)
        dist.broadcast(t, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        ident = (ctypes.c_ubyte * n)(*t.cpu().tolist())
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(device):
            _lib.check(_lib.lib.infllm_comm_create(ident, self.rank, self.world, ctypes.byref(self.handle)))

    def close(self):
        if getattr(self, "handle", None):
            _lib.lib.infllm_comm_destroy(self.handle)
            self.handle = None

    def __del__(self):
        self.close()
