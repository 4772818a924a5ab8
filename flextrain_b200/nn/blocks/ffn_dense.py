"""Dense gated FFN (SwiGLU / tanh-GeGLU) with hand-written forward / recompute / backward.

``w_1`` = gate, ``w_3`` = up, ``w_2`` = down (names as in flextrain/io/arch/llama.py:10-28).  Gate and
up are one GEMM writing ``x13 (T, 2F) = [gate | up]`` (tier 3) whose epilogue also emits the activation; the
down projection adds the residual in its epilogue; in the backward the down projection's data gradient and the
activation backward are one GEMM whose epilogue writes ``[dgate | dup]`` and re-emits ``act`` for the down-proj
weight gradient (flextrain/nn/blocks/ffn_dense.py:58-304, fusions F1/F4, runs them as separate passes).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ... import ops
from ...core.activation_schema import ActivationField
from ...core.layer import TensorSpec
from .linear import LinearGroup, LoRAConfig


@dataclass
class DenseFFNConfig:
    d_model: int
    ffn_dim: int
    kind: str = "swiglu"           # "swiglu" | "geglu"


class GatedFFN:
    def __init__(self, cfg: DenseFFNConfig, *, dtype=torch.bfloat16, lora: Optional[LoRAConfig] = None):
        self.cfg = cfg
        self.dtype = dtype
        self.up = LinearGroup(["w_1", "w_3"], lora)
        self.down = LinearGroup(["w_2"], lora)
        self.up.tp_mode, self.down.tp_mode = "col", "row"    # used only when a tensor-parallel handle is bound

    def tensor_specs(self):
        c, dt = self.cfg, self.dtype
        return [TensorSpec("w_1", (c.ffn_dim, c.d_model), dt), TensorSpec("w_3", (c.ffn_dim, c.d_model), dt),
                TensorSpec("w_2", (c.d_model, c.ffn_dim), dt)]

    def activation_fields(self):
        c = self.cfg
        return [ActivationField("x13", lambda t: (t, 2 * c.ffn_dim), self.dtype, 3)]

    def fwd(self, h, x_resid, params, slot):
        F = self.cfg.ffn_dim
        if self.up.tp is None:
            x13, act = ops.linear_glu_fwd(h, self.up.weight(params), self.cfg.kind, x13=slot.out("x13", h.device))
        else:
            x13 = self.up.fwd(h, params, out=slot.out("x13", h.device))
            act = ops.glu_fwd(x13[:, :F], x13[:, F:], self.cfg.kind)
        return self.down.fwd(act, params, residual=x_resid)

    def recompute(self, h, params, slot) -> None:
        if not slot.has("x13"):
            slot._t["x13"] = self.up.fwd(h, params)

    def bwd(self, dx, params, grads, slot):
        """Returns ``(dh, dx13)``; the caller runs ``self.up.wgrad(dx13, h, ...)`` once ``h`` is re-emitted."""
        F = self.cfg.ffn_dim
        x13 = slot._t["x13"]
        if self.down.tp is None:
            dx13, act = ops.linear_glu_bwd(dx, self.down.weight(params), x13, self.cfg.kind)
        else:
            dact = self.down.dgrad(dx, params)
            dx13 = torch.empty_like(x13)
            _, _, act = ops.glu_bwd(dact, x13[:, :F], x13[:, F:], self.cfg.kind, dgate=dx13[:, :F], dup=dx13[:, F:])
        self.down.wgrad(dx, act, params, grads)
        dh = self.up.dgrad(dx13, params)
        return dh, dx13

    def flops(self, T: int):
        c = self.cfg
        return 2.0 * T * c.d_model * 2 * c.ffn_dim, 2.0 * T * c.ffn_dim * c.d_model
