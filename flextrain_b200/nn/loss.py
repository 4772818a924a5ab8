"""Loss functions plugged into the LM head (flextrain/nn/loss.py:68-442).

A loss receives the logits of one micro-chunk and turns them *in place* into ``dZ`` scaled by
``grad_scale`` (the per-step ``1 / active_tokens`` factor), returning per-token losses; the
``(T, V)`` logits never exist for more than one micro-chunk.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Protocol

import torch

from .. import ops


@dataclass
class TokenSlice:
    """What a loss needs for the rows of one micro-chunk (flextrain/nn/loss.py:66-106); ``labels`` is the
    reference's name for ``targets``."""
    targets: Optional[torch.Tensor] = None
    loss_mask: Optional[torch.Tensor] = None
    advantages: Optional[torch.Tensor] = None
    ref_logprobs: Optional[torch.Tensor] = None
    offset: int = 0
    size: Optional[int] = None
    extra: Dict[str, torch.Tensor] = field(default_factory=dict)
    labels: Optional[torch.Tensor] = field(default=None, repr=False)

    def __post_init__(self):
        if self.targets is None:
            self.targets = self.labels
        self.labels = self.targets
        if self.size is None and self.targets is not None:
            self.size = int(self.targets.shape[0])


@dataclass
class TokenContext:
    """The same fields for a whole training chunk; :meth:`slice_for` narrows them to a micro-chunk
    (flextrain/nn/loss.py:108-166)."""
    labels: Optional[torch.Tensor] = None
    loss_mask: Optional[torch.Tensor] = None
    advantages: Optional[torch.Tensor] = None
    ref_logprobs: Optional[torch.Tensor] = None
    extra: Dict[str, torch.Tensor] = field(default_factory=dict)

    def slice_for(self, offset: int, size: int) -> TokenSlice:
        cut = lambda t: None if t is None else t[offset:offset + size]
        return TokenSlice(cut(self.labels), cut(self.loss_mask), cut(self.advantages), cut(self.ref_logprobs),
                          offset=offset, size=size, extra={k: v[offset:offset + size] for k, v in self.extra.items()})

    @property
    def total_tokens(self) -> int:
        for t in (self.labels, self.loss_mask, self.advantages, self.ref_logprobs, *self.extra.values()):
            if t is not None:
                return int(t.shape[0])
        raise ValueError("TokenContext is empty; cannot infer total_tokens")


class LossFn(Protocol):
    """``loss(logits, token_slice, grad_scale, softcap) -> per-token losses``, with the logits overwritten by
    ``dZ * grad_scale``.  A loss written for the reference, an object with
    ``compute(logits, token_slice, *, loss_scale, per_token_loss_out) -> (dZ, aux)`` and UNscaled ``dZ``
    (flextrain/nn/loss.py:174-213), is accepted too: :func:`apply_loss` adapts it."""

    def __call__(self, logits: torch.Tensor, sl: TokenSlice, grad_scale: float, softcap: float) -> torch.Tensor: ...


def apply_loss(loss_fn, logits: torch.Tensor, sl: TokenSlice, grad_scale: float, softcap: float = 0.0) -> torch.Tensor:
    """Run either kind of loss on one micro-chunk: ``logits`` becomes ``dZ * grad_scale``, the per-token losses come
    back.  For a ``compute``-style loss the final soft-cap, which the built-in kernels fuse, is applied here: the loss
    sees the capped logits and its gradient is carried back through the cap."""
    if callable(loss_fn) and (getattr(loss_fn, "_native", False) or not hasattr(loss_fn, "compute")):
        return loss_fn(logits, sl, grad_scale, softcap)
    out = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
    slope = None
    if softcap and softcap > 0:
        capped = torch.tanh(logits.to(torch.float32) / softcap)
        slope = 1.0 - capped * capped
        logits.copy_((capped * softcap).to(logits.dtype))
    ret = loss_fn.compute(logits, sl, loss_scale=grad_scale, per_token_loss_out=out)
    dz = ret[0] if isinstance(ret, tuple) else ret
    if dz is not logits:
        logits.copy_(dz.to(logits.dtype))
    if slope is not None:
        logits.copy_((logits.to(torch.float32) * slope * grad_scale).to(logits.dtype))
    else:
        logits.mul_(grad_scale)
    return out


class _NativeLoss:
    """Built-in losses answer to both call styles."""
    _native = True

    def compute(self, logits, token_slice, *, loss_scale: float = 1.0, per_token_loss_out=None):
        """The reference's entry point: UNscaled ``dZ`` written over the logits; returns ``(dZ, {})``."""
        per_tok = self(logits, token_slice, 1.0, 0.0)
        if per_token_loss_out is not None:
            per_token_loss_out.copy_(per_tok)
        return logits, {}


class CrossEntropyLoss(_NativeLoss):
    """Softmax cross-entropy; ``-100`` targets and ``loss_mask <= 0`` rows contribute neither loss nor gradient."""

    def __init__(self, ignore_index: int = -100):
        self.ignore_index = int(ignore_index)

    def __call__(self, logits, sl: TokenSlice, grad_scale: float, softcap: float = 0.0) -> torch.Tensor:
        return ops.softmax_ce_(logits, sl.targets, grad_scale=grad_scale, softcap=softcap, loss_mask=sl.loss_mask,
                               ignore_index=self.ignore_index)


class MSELoss(_NativeLoss):
    """Mean-squared error between logits and one-hot targets (regression / debugging head)."""

    def __call__(self, logits, sl: TokenSlice, grad_scale: float, softcap: float = 0.0) -> torch.Tensor:
        z = logits.to(torch.float32)
        valid = (sl.targets != -100)
        onehot = torch.zeros_like(z).scatter_(1, sl.targets.clamp(min=0).long().unsqueeze(1), 1.0)
        diff = (z - onehot) * valid.unsqueeze(1)
        logits.copy_((2.0 * diff * grad_scale / z.shape[1]).to(logits.dtype))
        return diff.pow(2).mean(-1)


class GRPOLoss(_NativeLoss):
    """Policy-gradient loss with per-token advantages and an optional KL penalty to reference log-probs:
    ``L = -A * logp(target) + beta * KL(pi || ref)`` using the k3 estimator on the taken token
    (``kl_coef`` is the reference's name for ``kl_beta``)."""

    def __init__(self, kl_beta: float = 0.0, *, kl_coef: Optional[float] = None):
        self.kl_beta = float(kl_coef if kl_coef is not None else kl_beta)

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
