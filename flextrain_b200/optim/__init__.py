"""Optimizers: AdamW, Muon and the per-tensor hybrid (flextrain/optim/*.py).

An optimizer is stateless apart from its hyper-parameters; the engine owns the state tensors
(so they can live in HBM, in pinned host memory or in a data-parallel shard) and hands them in:

    code = opt.step(param_spec, params, grads, state, step_num, grad_scale=1.0)

State keys follow flextrain/optim/base.py:77-87: ``o_adam_m_<suffix>``, ``o_adam_v_<suffix>``,
``o_muon_<suffix>`` where ``w_q -> q``.  ``step`` returns non-zero when ``check_error`` finds a
NaN/Inf gradient, in which case nothing was updated.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Protocol, Tuple

import torch

from .. import ops
from ..core.layer import ParamSpec, TensorSpec


@dataclass
class OptimizerStateSpec:
    key: str
    shape: Tuple[int, ...]
    dtype: torch.dtype
    param: str


def _suffix(name: str) -> str:
    return name[2:] if name.startswith(("w_", "b_")) and not name.startswith("b_") else name


def state_key(state_tensor_name: str, param_name: str) -> str:
    """Key of an optimizer-state tensor: ``<state name>_<parameter name without its w_ prefix>`` (``o_adam_m_q`` for
    ``w_q``; flextrain/optim/base.py:78-87)."""
    return f"{state_tensor_name}_{_suffix(param_name)}"


@dataclass
class AdamWHyperparams:
    """Hyper-parameter record in the reference's spelling (flextrain/optim/adamw.py:25-37): ``AdamW(AdamWHyperparams(...),
    state_dtype=...)`` builds the same optimizer as ``AdamW(lr=..., ...)``."""
    lr: float = 1e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.001
    check_error: bool = False


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


class Optimizer(Protocol):
    def state_specs(self, param_spec: ParamSpec) -> List[OptimizerStateSpec]: ...
    def step(self, param_spec: ParamSpec, params, grads, state, step_num: int, grad_scale: float = 1.0) -> int: ...


def _grads_finite(grads: List[torch.Tensor]) -> bool:
    bad = torch.zeros((), dtype=torch.float32, device=grads[0].device)
    for g in grads:
        bad = bad + (~torch.isfinite(g.to(torch.float32))).any().to(torch.float32)
    return float(bad) == 0.0


@dataclass
class AdamW:
    """Decoupled-weight-decay AdamW; state dtype bf16 by default, per-tensor override via ``TensorSpec.opt_state_dtype``
    (flextrain/optim/adamw.py:24-154)."""
    lr: float = 3e-5
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.0
    state_dtype: torch.dtype = torch.bfloat16
    check_error: bool = False
    no_decay_1d: bool = True

    def __post_init__(self):
        if isinstance(self.lr, AdamWHyperparams):            # AdamW(AdamWHyperparams(...), state_dtype=...)
            hp = self.lr
            self.lr, self.beta1, self.beta2, self.eps = hp.lr, hp.beta1, hp.beta2, hp.eps
            self.weight_decay, self.check_error = hp.weight_decay, hp.check_error

    @property
    def hp(self) -> "AdamWHyperparams":
        return AdamWHyperparams(self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.check_error)

    def state_specs(self, param_spec: ParamSpec) -> List[OptimizerStateSpec]:
        out = []
        for t in param_spec.trainable():
            dt = t.opt_state_dtype or (torch.float32 if t.master_dtype == torch.float32 and "norm" in t.name
                                       else self.state_dtype)
            s = _suffix(t.name)
            out.append(OptimizerStateSpec(f"o_adam_m_{s}", t.shape, dt, t.name))
            out.append(OptimizerStateSpec(f"o_adam_v_{s}", t.shape, dt, t.name))
        return out

    def step(self, param_spec, params, grads, state, step_num: int, grad_scale: float = 1.0, only=None) -> int:
        P, G, M, V, lrs, wds = [], [], [], [], [], []
        for t in param_spec.trainable():
            if only is not None and t.name not in only:
                continue
            s = _suffix(t.name)
            P.append(params[t.name]); G.append(grads[t.grad_name])
            M.append(state[f"o_adam_m_{s}"]); V.append(state[f"o_adam_v_{s}"])
            lrs.append(self.lr)
            wds.append(0.0 if (self.no_decay_1d and len(t.shape) == 1) else self.weight_decay)
        if not P:
            return 0
        if self.check_error and not _grads_finite(G):
            return 1
        ops.adamw_multi(P, G, M, V, lrs=lrs, wds=wds, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                        step=step_num, grad_scale=grad_scale)
        return 0

    def flops_per_param(self) -> float:
        return 12.0


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


def _accept_hp_keyword(cls) -> None:
    """``Cls(hp=record)`` is the reference's spelling of ``Cls(record)``."""
    plain = cls.__init__

    def __init__(self, *args, hp=None, **kw):
        if hp is not None:
            args = (hp,) + args
        plain(self, *args, **kw)

    __init__.__doc__, __init__.__wrapped__ = plain.__doc__, plain
    cls.__init__ = __init__


for _cls in (AdamW, Muon, HybridMuonAdamW):
    _accept_hp_keyword(_cls)
