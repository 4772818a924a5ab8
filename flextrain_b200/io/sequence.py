"""One training sequence (flextrain/io/sequence.py:21-107)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch


@dataclass
class Sequence:
    tokens: torch.Tensor                         # (L,) int64, CPU (pinned when a GPU is present)
    targets: Optional[torch.Tensor] = None       # default: roll(tokens, -1) (last position wraps)
    loss_mask: Optional[torch.Tensor] = None
    advantages: Optional[torch.Tensor] = None
    ref_logprobs: Optional[torch.Tensor] = None
    modality_inputs: Optional[Dict[str, Any]] = None
    seq_id: int = 0
    per_token_loss: Optional[torch.Tensor] = None  # filled by the engine after fwd_bwd (fp32, CPU)
    _active: Optional[int] = field(default=None, repr=False)

    def __post_init__(self):
        if self.targets is None:
            self.targets = torch.roll(self.tokens, -1)

    def __len__(self) -> int:
        return int(self.tokens.numel())

    @property
    def active_token_count(self) -> int:
        """Number of positions that contribute to the loss (targets != -100 and mask > 0); cached."""
        if self._active is None:
            a = self.targets != -100
            if self.loss_mask is not None:
                a = a & (self.loss_mask > 0)
            self._active = int(a.sum())
        return self._active


def as_sequence(obj) -> "Sequence":
    """A :class:`Sequence` for anything that carries ``tokens`` (duck typing, as the reference's engine allows:
    ``tokens``, optionally ``targets``, ``loss_mask``, ``advantages``, ``ref_logprobs``, ``modality_inputs``,
    ``seq_id``).  A :class:`Sequence` is returned as it is."""
    if isinstance(obj, Sequence):
        return obj
    if not hasattr(obj, "tokens"):
        raise TypeError(f"{type(obj).__name__} is not a sequence: it has no 'tokens'")
    pick = lambda name: getattr(obj, name, None)
    as64 = lambda t: None if t is None else torch.as_tensor(t).to(torch.int64)
    return Sequence(as64(obj.tokens), targets=as64(pick("targets")), loss_mask=pick("loss_mask"),
                    advantages=pick("advantages"), ref_logprobs=pick("ref_logprobs"),
                    modality_inputs=pick("modality_inputs"), seq_id=int(pick("seq_id") or 0))
