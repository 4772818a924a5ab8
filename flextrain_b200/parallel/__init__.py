"""Parallel layouts on one NVSwitch box: data parallel (sharded), tensor parallel, expert parallel."""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch


def build_parallel(*, world_size: int, rank: int, shard: str, tp: int, ep: int, device, process_group=None,
                   backend: Optional[str] = None):
    """Returns ``(dp, tp_group, ep_group)`` handles for the engine (any of them may be ``None``).

    ``backend``: ``"p2p"`` (peer-memory kernels; default on CUDA) or ``"collective"`` (library collectives:
    the baseline path, and the only one on CPU / gloo).  ``FTB_DP_BACKEND`` overrides.
    """
    dev = torch.device(device)
    backend = backend or os.environ.get("FTB_DP_BACKEND") or ("p2p" if dev.type == "cuda" else "collective")
    dp_size = world_size // max(tp, 1)
    tp_group = ep_group = dp = None
    mp = tp if tp > 1 else ep                       # size of the model-parallel (tensor or expert) group
    mp_pg, replica_pg = process_group, None
    if 1 < mp < world_size:
        # hybrid grid: consecutive ranks form a model-parallel group, ranks with the same position in their groups
        # are replicas of one another.  Library collectives only: the peer-memory kernels address the whole job.
        if backend == "p2p":
            raise NotImplementedError(
                f"a {world_size // mp} x {mp} grid needs the library-collective back end (FTB_DP_BACKEND=collective); "
                "the peer-memory kernels cover model-parallel groups that span the job")
        if world_size % mp:
            raise ValueError(f"world size {world_size} is not a multiple of the model-parallel size {mp}")
        import torch.distributed as dist
        for g in range(world_size // mp):           # every rank creates every group, in the same order
            ranks = list(range(g * mp, (g + 1) * mp))
            pg = dist.new_group(ranks)
            if rank in ranks:
                mp_pg = pg
        for r in range(mp):
            ranks = list(range(r, world_size, mp))
            pg = dist.new_group(ranks)
            if rank in ranks:
                replica_pg = pg
    if tp > 1:
        from .tp import TensorParallel
        tp_group = TensorParallel(rank % tp, tp, dev, mp_pg, backend=backend)
    if ep > 1:
        from .ep import ExpertParallel
        ep_group = ExpertParallel(rank % ep, ep, dev, mp_pg, backend=backend)
    if dp_size > 1 or tp > 1:
        # under tensor parallelism the ranks still hold replicated tensors (embedding, head, norm weights) whose
        # gradients come from different token shards: the data-parallel machinery reduces and updates exactly those
        from .dp import CollectiveDataParallel, P2PDataParallel
        if backend == "p2p":
            dp = P2PDataParallel(rank, world_size, dev, process_group)
        else:
            dp = CollectiveDataParallel(rank, world_size, dev, process_group)
            dp.replica_pg, dp.replica_src = replica_pg, rank % mp if replica_pg is not None else 0
    for h in (tp_group, ep_group):
        if h is not None:
            h.group_pg = mp_pg                      # what exports gather tensor- / expert-parallel parts over
    return dp, tp_group, ep_group
