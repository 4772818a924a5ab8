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
    if tp > 1:
        from .tp import TensorParallel
        tp_group = TensorParallel(rank % tp, tp, dev, process_group, backend=backend)
    if ep > 1:
        from .ep import ExpertParallel
        ep_group = ExpertParallel(rank % ep, ep, dev, process_group, backend=backend)
    if dp_size > 1 or tp > 1:
        # under tensor parallelism the ranks still hold replicated tensors (embedding, head, norm weights) whose
        # gradients come from different token shards: the data-parallel machinery reduces and updates exactly those
        from .dp import CollectiveDataParallel, P2PDataParallel
        if backend == "p2p":
            dp = P2PDataParallel(rank, world_size, dev, process_group)
        else:
            dp = CollectiveDataParallel(rank, world_size, dev, process_group)
    return dp, tp_group, ep_group
