"""What every optimizer shares: the protocol, the state-tensor record and its key rule, the finite-gradient check
(flextrain/optim/base.py:14-87)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Protocol, Tuple

import torch

from ..core.layer import ParamSpec


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


class Optimizer(Protocol):
    def state_specs(self, param_spec: ParamSpec) -> List[OptimizerStateSpec]: ...
    def step(self, param_spec: ParamSpec, params, grads, state, step_num: int, grad_scale: float = 1.0) -> int: ...


def _grads_finite(grads: List[torch.Tensor]) -> bool:
    bad = torch.zeros((), dtype=torch.float32, device=grads[0].device)
    for g in grads:
        bad = bad + (~torch.isfinite(g.to(torch.float32))).any().to(torch.float32)
    return float(bad) == 0.0


def _accept_hp_keyword(cls) -> None:
    """``Cls(hp=record)`` is the reference's spelling of ``Cls(record)``."""
    plain = cls.__init__

    def __init__(self, *args, hp=None, **kw):
        if hp is not None:
            args = (hp,) + args
        plain(self, *args, **kw)

    __init__.__doc__, __init__.__wrapped__ = plain.__doc__, plain
    cls.__init__ = __init__
