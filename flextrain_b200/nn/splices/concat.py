"""Concat splice: replace placeholder token rows of the embedded text with encoder rows
(flextrain/nn/splices/concat.py:1-40).  Backward zeroes the gradient of placeholder rows before the embedding
scatter (they did not come from the embedding table) and hands those rows to the encoder when it trains."""
from __future__ import annotations

import torch


def splice_forward(x: torch.Tensor, placeholder_rows: torch.Tensor, encoder_rows: torch.Tensor) -> torch.Tensor:
    """``x (T, d)`` text embeddings; rows ``placeholder_rows`` (int64) are overwritten by ``encoder_rows`` in order."""
    if placeholder_rows.numel() != encoder_rows.shape[0]:
        raise ValueError(f"{placeholder_rows.numel()} placeholder tokens but {encoder_rows.shape[0]} encoder rows")
    x = x.clone()
    x[placeholder_rows] = encoder_rows.to(x.dtype)
    return x


def splice_backward(dx: torch.Tensor, placeholder_rows: torch.Tensor):
    """Returns ``(dx_text, d_encoder_rows)``: placeholder rows are zero in ``dx_text``."""
    d_enc = dx[placeholder_rows].clone()
    dx = dx.clone()
    dx[placeholder_rows] = 0
    return dx, d_enc
