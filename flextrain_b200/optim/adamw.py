"""AdamW with decoupled weight decay over the multi-tensor kernel (flextrain/optim/adamw.py:24-154)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import torch

from .. import ops
from ..core.layer import ParamSpec
from .base import OptimizerStateSpec, _accept_hp_keyword, _grads_finite, _suffix


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


_accept_hp_keyword(AdamW)
