"""Round splitting, chunk packing and chunk materialisation (flextrain/engine/schedule.py:88-513).

* ``split_sequences``: greedy rounds — a sequence joins the current round unless the round would
  exceed ``target_round_tokens`` or the estimated chunk count would exceed ``max_training_chunks``;
  a sequence longer than ``max_total_round_tokens`` is an error.
* ``pack_sequences``: sequences no longer than a chunk are first-fit packed into a running chunk;
  a longer sequence flushes the running chunk and takes ``ceil(len / chunk)`` dedicated consecutive
  chunks, each carrying ``prior_len`` and ``has_more_chunks``.
* A new *sequence group* starts at every chunk whose first sequence begins at offset 0; backward
  walks groups in reverse, chunks in reverse inside a group.
* ``prepare_training_chunks``: one pinned staging buffer and one H2D copy per chunk.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence as Seq, Tuple

import torch

from ..core.layer import ChunkMeta
from ..io.sequence import Sequence


class ChunkPolicy(enum.Enum):
    CAUSAL = "causal"
    NON_CAUSAL = "non_causal"


@dataclass
class ChunkPlan:
    """Host-side description of one chunk: ``pieces[i] = (seq_index, start, length)``."""
    pieces: List[Tuple[int, int, int]]
    seq_group: int = 0

    @property
    def num_tokens(self) -> int:
        return sum(p[2] for p in self.pieces)


def split_sequences(seqs: Seq[Sequence], *, target_round_tokens: int, max_chunk_size: int,
                    max_training_chunks: int, max_total_round_tokens: Optional[int] = None,
                    policy: ChunkPolicy = ChunkPolicy.CAUSAL) -> List[List[Sequence]]:
    max_total = max_total_round_tokens or max(target_round_tokens, max_chunk_size * max_training_chunks)
    rounds: List[List[Sequence]] = []
    cur: List[Sequence] = []
    cur_tokens = 0
    for s in seqs:
        n = len(s)
        if n > max_total:
            raise ValueError(f"sequence of {n} tokens exceeds max_total_round_tokens={max_total}")
        if n > max_chunk_size and policy is ChunkPolicy.NON_CAUSAL:
            raise ValueError("a non-causal model cannot split a sequence across chunks")
        est_chunks = len(pack_sequences(cur + [s], max_chunk_size)) if cur else math.ceil(n / max_chunk_size)
        if cur and (cur_tokens + n > target_round_tokens or est_chunks > max_training_chunks):
            rounds.append(cur)
            cur, cur_tokens = [], 0
        cur.append(s)
        cur_tokens += n
    if cur:
        rounds.append(cur)
    return rounds


def pack_sequences(seqs: Seq[Sequence], max_chunk_size: int) -> List[ChunkPlan]:
    chunks: List[ChunkPlan] = []
    running: List[Tuple[int, int, int]] = []
    running_tokens = 0

    def flush():
        nonlocal running, running_tokens
        if running:
            chunks.append(ChunkPlan(running))
            running, running_tokens = [], 0

    for i, s in enumerate(seqs):
        n = len(s)
        if n <= max_chunk_size:
            if running_tokens + n > max_chunk_size:
                flush()
            running.append((i, 0, n))
            running_tokens += n
        else:
            flush()
            for start in range(0, n, max_chunk_size):
                chunks.append(ChunkPlan([(i, start, min(max_chunk_size, n - start))]))
    flush()
    g = -1
    for c in chunks:
        if c.pieces[0][1] == 0:
            g += 1
        c.seq_group = max(g, 0)
    return chunks


def prepare_training_chunks(seqs: Seq[Sequence], max_chunk_size: int, device, *, staging=None,
                            mrope: bool = False, pad_multiple: int = 1) -> List[ChunkMeta]:
    """Pack ``seqs`` into chunks and upload ids / targets / masks (one H2D copy per chunk).

    ``pad_multiple > 1`` (tensor parallelism shards a chunk's tokens in 128-row tiles per rank) rounds a chunk's token
    count up by extending its LAST piece with unscored filler tokens.  That piece must end its sequence: the filler
    then sits after every real token of a causal model, so no real token sees it, it carries no loss and it feeds no
    later chunk.  A chunk that ends inside a sequence has exactly ``max_chunk_size`` tokens, which therefore has to be
    a multiple of ``pad_multiple`` itself.  ``meta.extra["pad_tokens"]`` records the filler count."""
    plans = pack_sequences(seqs, max_chunk_size)
    metas: List[ChunkMeta] = []
    dev = torch.device(device)
    for cid, plan in enumerate(plans):
        Tr = plan.num_tokens
        pad = (-Tr) % pad_multiple if pad_multiple > 1 else 0
        if pad:
            li, ls, ln = plan.pieces[-1]
            if ls + ln < len(seqs[li]):
                raise ValueError(f"a chunk of {Tr} tokens ends inside a sequence and cannot be padded to a multiple of "
                                 f"{pad_multiple}: make max_chunk_size ({max_chunk_size}) a multiple of it")
        T = Tr + pad
        any_mask = any(seqs[i].loss_mask is not None for i, _, _ in plan.pieces) or pad > 0
        any_adv = any(seqs[i].advantages is not None for i, _, _ in plan.pieces)
        rows = 2 + (1 if any_mask else 0)
        host = torch.empty(rows, T, dtype=torch.int64, pin_memory=(dev.type == "cuda"))
        off = 0
        seq_ids, lens, priors, more = [], [], [], []
        for i, start, n in plan.pieces:
            s = seqs[i]
            host[0, off:off + n] = s.tokens[start:start + n]
            host[1, off:off + n] = s.targets[start:start + n]
            if any_mask:
                host[2, off:off + n] = (s.loss_mask[start:start + n] > 0).to(torch.int64) if s.loss_mask is not None else 1
            off += n
            seq_ids.append(s.seq_id); lens.append(n); priors.append(start); more.append(start + n < len(s))
        if pad:
            host[0, Tr:] = host[0, Tr - 1]                     # any valid token id
            host[1, Tr:] = -100
            host[2, Tr:] = 0
            lens[-1] += pad
        devbuf = host.to(dev, non_blocking=True)
        mask = devbuf[2].to(torch.float32) if any_mask else None
        meta = ChunkMeta.build(cid, seq_ids, lens, priors, more, dev, tokens=devbuf[0], targets=devbuf[1],
                               loss_mask=mask, seq_group=plan.seq_group)
        meta.extra["pieces"] = plan.pieces
        meta.extra["pad_tokens"] = pad
        tail = lambda t, fill: torch.cat([t, torch.full((pad,), fill, dtype=t.dtype)]) if pad else t
        if any_adv:
            adv = torch.cat([(seqs[i].advantages[st:st + n] if seqs[i].advantages is not None else torch.ones(n))
                             for i, st, n in plan.pieces])
            meta.extra["advantages"] = tail(adv, 0.0).to(dev, non_blocking=True)
            if any(seqs[i].ref_logprobs is not None for i, _, _ in plan.pieces):
                ref = torch.cat([(seqs[i].ref_logprobs[st:st + n] if seqs[i].ref_logprobs is not None else torch.zeros(n))
                                 for i, st, n in plan.pieces])
                meta.extra["ref_logprobs"] = tail(ref, 0.0).to(dev, non_blocking=True)
        if mrope:
            pos = [compute_mrope_position_ids(seqs[i], start, n) for i, start, n in plan.pieces]
            if pad:                                            # filler continues after the sequence's last position
                nxt = int(pos[-1].max()) + 1 if pos[-1].numel() else 0
                pos.append((nxt + torch.arange(pad, dtype=torch.int32)).unsqueeze(1).expand(pad, 3))
            meta.positions = torch.cat(pos, 0).to(dev)
        metas.append(meta)
    return metas


def compute_mrope_position_ids(seq: Sequence, start: int, n: int) -> torch.Tensor:
    """3-axis (t, h, w) positions for a slice of a sequence (flextrain/engine/schedule.py:516-666).

    Text tokens advance all three axes together. An image span declared in
    ``seq.modality_inputs["image_spans"] = [(first_token, grid_t, grid_h, grid_w), ...]`` takes
    ``t`` constant per frame and ``h, w`` from the (merged) patch grid; text after the image resumes
    from ``max(position) + 1``.
    """
    L = len(seq)
    pos = torch.zeros(L, 3, dtype=torch.int32)
    spans = sorted((seq.modality_inputs or {}).get("image_spans", []))
    cur, nxt, si = 0, 0, 0
    while cur < L:
        if si < len(spans) and spans[si][0] == cur:
            _, gt, gh, gw = spans[si]
            cnt = gt * gh * gw
            idx = torch.arange(cnt)
            pos[cur:cur + cnt, 0] = nxt + idx // (gh * gw)
            pos[cur:cur + cnt, 1] = nxt + (idx // gw) % gh
            pos[cur:cur + cnt, 2] = nxt + idx % gw
            nxt = nxt + max(gt, gh, gw)
            cur += cnt
            si += 1
        else:
            end = spans[si][0] if si < len(spans) else L
            cnt = end - cur
            pos[cur:end] = (nxt + torch.arange(cnt, dtype=torch.int32)).unsqueeze(1)
            nxt += cnt
            cur = end
    return pos[start:start + n]
