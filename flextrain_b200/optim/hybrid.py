"""Per-tensor choice between Muon and AdamW (flextrain/optim/hybrid.py:46-254)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..core.layer import ParamSpec, TensorSpec
from .adamw import AdamW, AdamWHyperparams
from .base import OptimizerStateSpec, _accept_hp_keyword, _grads_finite
from .muon import Muon, MuonHyperparams


@dataclass
class HybridMuonAdamWHyperparams:
    """(flextrain/optim/hybrid.py:147-153): the two optimizers' records; ``lr`` is the default of both."""
    lr: float = 1e-3
    adamw: Optional[AdamWHyperparams] = None
    muon: Optional[MuonHyperparams] = None

    def __post_init__(self):
        if self.adamw is None:
            self.adamw = AdamWHyperparams(lr=self.lr)
        if self.muon is None:
            self.muon = MuonHyperparams(lr=self.lr)


_ADAM_NAME_PARTS = ("_norm", "embed", "head", "router", "lm_head")


def uses_muon(t: TensorSpec) -> bool:
    """Per-tensor rule (flextrain/optim/hybrid.py:46-89): explicit hint wins; otherwise rank-2/3 tensors whose
    name has none of ``_norm / embed / head / router / lm_head`` go to Muon, everything else to AdamW."""
    if t.optimizer is not None:
        return t.optimizer == "muon"
    return len(t.shape) in (2, 3) and not any(p in t.name for p in _ADAM_NAME_PARTS)


def infer_optimizer_for_param(spec: TensorSpec, dims=None) -> str:
    """``"muon"`` or ``"adamw"`` for one tensor, by :func:`uses_muon`'s rule (flextrain/optim/hybrid.py:60-89; shapes are
    concrete here, so ``dims`` is not needed)."""
    return "muon" if uses_muon(spec) else "adamw"


@dataclass
class HybridMuonAdamW:
    muon: Muon = field(default_factory=Muon)
    adamw: AdamW = field(default_factory=lambda: AdamW(lr=3e-4))
    check_error: bool = False

    def __post_init__(self):
        if isinstance(self.muon, HybridMuonAdamWHyperparams):       # HybridMuonAdamW(HybridMuonAdamWHyperparams(...))
            hp = self.muon
            self.muon = Muon(hp.muon)
            self.adamw = AdamW(hp.adamw, state_dtype=torch.float32)   # the reference's hybrid keeps fp32 moments
            self.check_error = bool(hp.adamw.check_error or hp.muon.check_error)

    @property
    def lr(self) -> float:
        return self.muon.lr

    @lr.setter
    def lr(self, v: float) -> None:
        ratio = self.adamw.lr / self.muon.lr if self.muon.lr else 1.0
        self.muon.lr = v
        self.adamw.lr = v * ratio

    def _split(self, param_spec: ParamSpec):
        mu = [t.name for t in param_spec.trainable() if uses_muon(t)]
        ad = [t.name for t in param_spec.trainable() if not uses_muon(t)]
        return mu, ad

    def state_specs(self, param_spec: ParamSpec) -> List[OptimizerStateSpec]:
        mu, ad = self._split(param_spec)
        out = [s for s in self.muon.state_specs(param_spec) if s.param in mu]
        out += [s for s in self.adamw.state_specs(param_spec) if s.param in ad]
        return out

    def step(self, param_spec, params, grads, state, step_num: int, grad_scale: float = 1.0) -> int:
        mu, ad = self._split(param_spec)
        if self.check_error:
            gs = [grads[t.grad_name] for t in param_spec.trainable()]
            if gs and not _grads_finite(gs):
                return 1
        rc = self.muon.step(param_spec, params, grads, state, step_num, grad_scale, only=set(mu))
        rc |= self.adamw.step(param_spec, params, grads, state, step_num, grad_scale, only=set(ad))
        return rc

    def flops_per_param(self) -> float:
        return 12.0


_accept_hp_keyword(HybridMuonAdamW)
