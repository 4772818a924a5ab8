"""What every optimizer shares: the protocol, the state-tensor record and its key rule, the finite-gradient check
(flextrain/optim/base.py:14-87)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Protocol, Tuple

import torch

from ..core.layer import ParamSpec


@dataclass(frozen=True)
class OptStateTensor:
    """One kind of state tensor an optimizer keeps per parameter (``o_adam_m`` in fp32, say): the element of the
    reference-style ``OptimizerStateSpec(tensors=(...))`` (flextrain/optim/base.py:14-20)."""
    name: str
    dtype: torch.dtype


@dataclass
class OptimizerStateSpec:
    """One state tensor of one parameter (``key``, ``shape``, ``dtype``, owning ``param``): what
    ``optimizer.state_specs(param_spec)`` lists.  Built with ``tensors=(OptStateTensor, ...)`` instead, it is the
    reference's per-optimizer declaration "every parameter gets these", which :func:`as_engine_optimizer` expands."""
    key: Optional[str] = None
    shape: Optional[Tuple[int, ...]] = None
    dtype: Optional[torch.dtype] = None
    param: Optional[str] = None
    tensors: Optional[Tuple[OptStateTensor, ...]] = None


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


class ReferenceStyleOptimizer:
    """Adapter for an optimizer written to the reference's protocol (flextrain/optim/base.py:52-75): a class
    attribute ``state_spec = OptimizerStateSpec(tensors=(...))`` and
    ``step(param_spec, master, grads, state, *, step_num) -> int``.  The state of parameter ``w_x`` lives under
    ``<state name>_x``; the wrapped ``step`` sees the trainable tensors only, and a gradient-clipping scale is applied
    to the gradients before it runs."""

    def __init__(self, inner):
        object.__setattr__(self, "inner", inner)

    def __getattr__(self, name):
        return getattr(object.__getattribute__(self, "inner"), name)

    def __setattr__(self, name, value):
        setattr(self.inner, name, value)

    @property
    def lr(self):
        hp = getattr(self.inner, "hp", None)
        return getattr(self.inner, "lr", getattr(hp, "lr", None))

    @lr.setter
    def lr(self, v) -> None:
        hp = getattr(self.inner, "hp", None)
        if hasattr(self.inner, "lr") or hp is None:
            self.inner.lr = v
        else:
            try:
                hp.lr = v
            except Exception:                                   # a frozen record: replace it
                import dataclasses
                self.inner.hp = dataclasses.replace(hp, lr=v)

    def state_specs(self, param_spec: ParamSpec) -> List[OptimizerStateSpec]:
        return [OptimizerStateSpec(state_key(st.name, t.name), t.shape, st.dtype, t.name)
                for t in param_spec.trainable() for st in self.inner.state_spec.tensors]

    def step(self, param_spec: ParamSpec, params, grads, state, step_num: int, grad_scale: float = 1.0) -> int:
        live = ParamSpec(param_spec.trainable())
        if not live.tensors:
            return 0
        if grad_scale != 1.0:
            for t in live.tensors:
                grads[t.grad_name].mul_(grad_scale)
        return int(self.inner.step(live, params, grads, state, step_num=step_num) or 0)

    def flops_per_param(self) -> float:
        fn = getattr(self.inner, "flops_per_param", None)
        return float(fn()) if callable(fn) else 0.0


def as_engine_optimizer(opt):
    """The optimizer as the engine drives it: itself when it lists its state with ``state_specs``, wrapped when it
    follows the reference's protocol."""
    if hasattr(opt, "state_specs"):
        return opt
    spec = getattr(opt, "state_spec", None)
    if spec is not None and getattr(spec, "tensors", None) is not None and hasattr(opt, "step"):
        return ReferenceStyleOptimizer(opt)
    raise TypeError(f"{type(opt).__name__} is not an optimizer: it needs state_specs(param_spec) and step(...), or the "
                    "reference-style state_spec attribute")
