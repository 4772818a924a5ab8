"""Concat splice: placeholder token rows of the embedded text are replaced by encoder rows
(flextrain/nn/splices/concat.py:1-40).  Backward zeroes the gradient of the placeholder rows before the embedding
scatter (those rows did not come from the embedding table) and hands them to the encoder when it trains.

The row maps are built once per round on the host (:func:`build_splice_maps`): a sequence may span several chunks, so
a chunk's placeholders continue where the previous chunk's stopped in that sequence's encoder rows."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence as Seq, Tuple

import torch


def build_splice_maps(seqs, pieces_per_chunk: Seq[Seq[Tuple[int, int, int]]], placeholder_ids: Seq[int],
                      row_offset_of_seq: Dict[int, int]) -> List[Optional[Tuple[torch.Tensor, torch.Tensor]]]:
    """For every chunk: ``(chunk_rows, encoder_rows)`` int64 host tensors, or ``None`` when it holds no placeholder.

    ``pieces_per_chunk[c]`` lists ``(sequence index, first token, token count)`` in chunk order;
    ``row_offset_of_seq[i]`` is where sequence ``i``'s rows start in the round's concatenated encoder output."""
    ph = torch.tensor(list(placeholder_ids), dtype=torch.int64)
    before: Dict[int, torch.Tensor] = {}                      # per sequence: placeholders strictly before each token
    out: List[Optional[Tuple[torch.Tensor, torch.Tensor]]] = []
    for pieces in pieces_per_chunk:
        rows, src, off = [], [], 0
        for i, start, n in pieces:
            if i in row_offset_of_seq:
                if i not in before:
                    is_ph = torch.isin(seqs[i].tokens, ph)
                    before[i] = (torch.cumsum(is_ph, 0) - is_ph.to(torch.int64), is_ph)
                cnt, is_ph = before[i]
                local = is_ph[start:start + n].nonzero(as_tuple=True)[0]
                if local.numel():
                    rows.append(local + off)
                    src.append(cnt[start:start + n][local] + row_offset_of_seq[i])
            off += n
        out.append((torch.cat(rows), torch.cat(src)) if rows else None)
    return out


def splice_forward(x: torch.Tensor, placeholder_rows: torch.Tensor, encoder_rows: torch.Tensor) -> torch.Tensor:
    """``x (T, d)`` text embeddings; rows ``placeholder_rows`` (int64) are overwritten by ``encoder_rows`` in order."""
    if placeholder_rows.numel() != encoder_rows.shape[0]:
        raise ValueError(f"{placeholder_rows.numel()} placeholder tokens but {encoder_rows.shape[0]} encoder rows")
    return x.index_copy(0, placeholder_rows, encoder_rows.to(x.dtype))


def splice_backward(dx: torch.Tensor, placeholder_rows: torch.Tensor, want_encoder_grad: bool = False):
    """Zeroes the placeholder rows of ``dx`` IN PLACE; returns ``(dx, d_encoder_rows or None)``."""
    d_enc = dx.index_select(0, placeholder_rows) if want_encoder_grad else None
    dx.index_fill_(0, placeholder_rows, 0)
    return dx, d_enc
