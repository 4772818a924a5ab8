"""Loss functions plugged into the LM head (flextrain/nn/loss.py:68-442).

A loss receives the logits of one micro-chunk and turns them *in place* into ``dZ`` scaled by
``grad_scale`` (the per-step ``1 / active_tokens`` factor), returning per-token losses; the
``(T, V)`` logits never exist for more than one micro-chunk.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Protocol

import torch

from .. import ops


@dataclass
class TokenSlice:
    targets: torch.Tensor
    loss_mask: Optional[torch.Tensor] = None
    advantages: Optional[torch.Tensor] = None
    ref_logprobs: Optional[torch.Tensor] = None


class LossFn(Protocol):
    def __call__(self, logits: torch.Tensor, sl: TokenSlice, grad_scale: float, softcap: float) -> torch.Tensor: ...


class CrossEntropyLoss:
    """Softmax cross-entropy; ``-100`` targets and ``loss_mask <= 0`` rows contribute neither loss nor gradient."""
    ignore_index = -100

    def __call__(self, logits, sl: TokenSlice, grad_scale: float, softcap: float = 0.0) -> torch.Tensor:
        return ops.softmax_ce_(logits, sl.targets, grad_scale=grad_scale, softcap=softcap, loss_mask=sl.loss_mask,
                               ignore_index=self.ignore_index)


class MSELoss:
    """Mean-squared error between logits and one-hot targets (regression / debugging head)."""

    def __call__(self, logits, sl: TokenSlice, grad_scale: float, softcap: float = 0.0) -> torch.Tensor:
        z = logits.to(torch.float32)
        valid = (sl.targets != -100)
        onehot = torch.zeros_like(z).scatter_(1, sl.targets.clamp(min=0).long().unsqueeze(1), 1.0)
        diff = (z - onehot) * valid.unsqueeze(1)
        logits.copy_((2.0 * diff * grad_scale / z.shape[1]).to(logits.dtype))
        return diff.pow(2).mean(-1)


class GRPOLoss:
    """Policy-gradient loss with per-token advantages and an optional KL penalty to reference log-probs:
    ``L = -A * logp(target) + beta * KL(pi || ref)`` using the k3 estimator on the taken token."""

    def __init__(self, kl_beta: float = 0.0):
        self.kl_beta = kl_beta

    def __call__(self, logits, sl: TokenSlice, grad_scale: float, softcap: float = 0.0) -> torch.Tensor:
        z = logits.to(torch.float32)
        valid = (sl.targets != -100).to(torch.float32)
        tgt = sl.targets.clamp(min=0).long()
        logp = torch.log_softmax(z, -1)
        lp = logp.gather(1, tgt.unsqueeze(1)).squeeze(1)
        adv = sl.advantages.to(torch.float32) if sl.advantages is not None else torch.ones_like(lp)
        coef = -adv
        loss = -adv * lp
        if self.kl_beta > 0 and sl.ref_logprobs is not None:
            d = sl.ref_logprobs.to(torch.float32) - lp
            loss = loss + self.kl_beta * (torch.exp(d) - d - 1)
            coef = coef + self.kl_beta * (1 - torch.exp(d))
        p = torch.exp(logp)
        onehot = torch.zeros_like(p).scatter_(1, tgt.unsqueeze(1), 1.0)
        dz = (onehot - p) * (coef * valid * grad_scale).unsqueeze(1)
        logits.copy_(dz.to(logits.dtype))
        return loss * valid
