"""Muon: momentum, Nesterov, quintic Newton-Schulz orthogonalisation (flextrain/optim/muon.py:20-81)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from .. import ops
from ..core.layer import ParamSpec
from .base import OptimizerStateSpec, _accept_hp_keyword, _grads_finite, _suffix


@dataclass
class MuonHyperparams:
    """(flextrain/optim/muon.py:22-33; the Newton-Schulz coefficients are fixed in the kernels here.)"""
    lr: float = 1e-3
    beta: float = 0.95
    eps: float = 1e-8
    ns_iters: int = 5
    weight_decay: float = 0.0
    nesterov: bool = True
    check_error: bool = False
    a: float = 3.4445                       # Newton-Schulz quintic coefficients: compiled into the kernels here,
    b: float = -4.7750                      # so other values are refused rather than ignored
    c: float = 2.0315

    def __post_init__(self):
        if (round(self.a, 4), round(self.b, 4), round(self.c, 4)) != (3.4445, -4.775, 2.0315):
            raise ValueError("the Newton-Schulz coefficients are fixed at (3.4445, -4.7750, 2.0315)")


@dataclass
class Muon:
    """Momentum + Nesterov + 5 quintic Newton-Schulz iterations, update scaled by ``0.2*sqrt(max(m,n))``
    (flextrain/optim/muon.py:20-81). One bf16 momentum buffer per tensor; 3-D tensors are batches of matrices."""
    lr: float = 1e-3
    beta: float = 0.95
    weight_decay: float = 0.0
    ns_iters: int = 5
    nesterov: bool = True
    state_dtype: torch.dtype = torch.bfloat16
    check_error: bool = False

    def __post_init__(self):
        if isinstance(self.lr, MuonHyperparams):             # Muon(MuonHyperparams(...))
            hp = self.lr
            self.lr, self.beta, self.weight_decay = hp.lr, hp.beta, hp.weight_decay
            self.ns_iters, self.nesterov, self.check_error = hp.ns_iters, hp.nesterov, hp.check_error

    def state_specs(self, param_spec: ParamSpec) -> List[OptimizerStateSpec]:
        return [OptimizerStateSpec(f"o_muon_{_suffix(t.name)}", t.shape, t.opt_state_dtype or self.state_dtype, t.name)
                for t in param_spec.trainable()]

    def step(self, param_spec, params, grads, state, step_num: int, grad_scale: float = 1.0, only=None) -> int:
        todo = [t for t in param_spec.trainable() if only is None or t.name in only]
        if self.check_error and todo and not _grads_finite([grads[t.grad_name] for t in todo]):
            return 1
        for t in todo:
            ops.muon_step(params[t.name], grads[t.grad_name], state[f"o_muon_{_suffix(t.name)}"], lr=self.lr,
                          beta=self.beta, weight_decay=self.weight_decay, ns_iters=self.ns_iters,
                          nesterov=self.nesterov, grad_scale=grad_scale)
        return 0

    def flops_per_param(self) -> float:
        return 0.0


_accept_hp_keyword(Muon)
