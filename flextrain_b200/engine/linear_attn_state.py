"""Per-round plan of which packed sequences carry linear-attention state across chunks
(flextrain/engine/linear_attn_state.py:27-144).

For every ``(chunk, packed sequence)`` it records whether the sequence started in an earlier chunk (its recurrent
and convolution states must be threaded in) and whether it continues in a later chunk (its final states must be
kept).  The engine consults it when it hands ``lin_state_in`` / ``lin_conv_in`` to Gated-DeltaNet layers."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

from ..core.layer import ChunkMeta


@dataclass(frozen=True)
class MultiChunkSeqInfo:
    has_prior_chunks: bool
    has_more_chunks: bool
    prior_chunk: int = -1          # chunk index holding the previous piece of this sequence


def build_state_plan(metas: List[ChunkMeta]) -> Dict[Tuple[int, int], MultiChunkSeqInfo]:
    """``{(chunk_index, position_in_chunk): MultiChunkSeqInfo}`` for one round."""
    last_seen: Dict[int, int] = {}
    plan: Dict[Tuple[int, int], MultiChunkSeqInfo] = {}
    for c, m in enumerate(metas):
        for j, sid in enumerate(m.seq_ids):
            prior = m.prior_lens[j] > 0
            plan[(c, j)] = MultiChunkSeqInfo(prior, bool(m.has_more_chunks[j]), last_seen.get(sid, -1) if prior else -1)
            last_seen[sid] = c
    return plan


def needs_state_threading(metas: List[ChunkMeta]) -> bool:
    return any(m.has_prior or any(m.has_more_chunks) for m in metas)
