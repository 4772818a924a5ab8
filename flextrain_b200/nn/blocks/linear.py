"""Linear-projection helper shared by all blocks: fused weight groups and LoRA.

* **Fused groups.**  Weights are ``(out, in)``; tensors that are adjacent in the layer's flat
  parameter buffer (``w_q, w_k, w_v`` and ``w_1, w_3``) form one taller matrix without any copy, so
  QKV and gate/up are each ONE GEMM in forward, dgrad and wgrad.  The reference issues them as
  separate cuBLAS calls (flextrain/nn/blocks/attention.py:424-435, ffn_dense.py:130-131).
* **LoRA.**  ``W' = W + s * B @ A`` with ``A = <t>_lora_a (r, in)``, ``B = <t>_lora_b (out, r)``
  (PEFT layout).  Forward / dgrad use the materialised ``W'``; the base weight gradient is skipped
  and the rank-r gradients come from the captured ``(x, dy)``:
  ``gA += s * (dy @ B).T @ x``,  ``gB += s * dy.T @ (x @ A.T)``
  (flextrain/nn/layers/lora_wrapper.py:106-148, 429, 602, 840).
* **Tensor parallelism** (no counterpart in the reference).  With a bound ``tp`` handle the activations between
  blocks are token-sharded ``(T/tp, d)``.  A ``"col"`` group holds ``out/tp`` rows of each weight: forward is the
  fused all-gather→GEMM, dgrad the fused GEMM→reduce-scatter, wgrad gathers its input.  A ``"row"`` group holds
  ``in/tp`` columns: forward is GEMM→reduce-scatter (+ local residual), dgrad all-gather→GEMM; the gathered ``dy``
  is kept for the weight gradient.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import torch

from ... import ops

# "all": every dense projection plus the routed-expert stacks of MoE layers (one rank-r pair per expert), as the
# reference's lora_targets="all" (flextrain/nn/layers/lora_wrapper.py:197-255); routers, shared experts and the
# bundled linear-attention projections are left out there too.
LORA_ALL_TARGETS = ("w_q", "w_k", "w_v", "w_o", "w_1", "w_2", "w_3", "w_up", "w_down")


@dataclass
class LoRAConfig:
    targets: Tuple[str, ...] = LORA_ALL_TARGETS
    rank: int = 16
    alpha: float = 16.0
    compute_dtype: torch.dtype = torch.bfloat16
    master_dtype: torch.dtype = torch.bfloat16
    grad_dtype: torch.dtype = torch.bfloat16
    opt_state_dtype: torch.dtype = torch.bfloat16

    @property
    def scale(self) -> float:
        return self.alpha / self.rank


def fused_view(tensors: Sequence[torch.Tensor]) -> Optional[torch.Tensor]:
    """Return one ``(sum out_i, in)`` view over row-adjacent ``(out_i, in)`` tensors, or None."""
    t0 = tensors[0]
    if any(t.dim() != 2 or t.shape[1] != t0.shape[1] or not t.is_contiguous() or t.dtype != t0.dtype
           or t.device != t0.device for t in tensors):
        return None
    ptr = t0.data_ptr()
    for t in tensors:
        if t.data_ptr() != ptr:
            return None
        ptr += t.numel() * t.element_size()
    rows = sum(t.shape[0] for t in tensors)
    try:
        return torch.as_strided(t0, (rows, t0.shape[1]), (t0.shape[1], 1))
    except RuntimeError:
        return None


class LinearGroup:
    """A projection made of one or more named ``(out_i, in)`` weights applied to the same input."""

    def __init__(self, names: Sequence[str], lora: Optional[LoRAConfig] = None, bias_names: Sequence[str] = ()):
        self.names = list(names)
        self.bias_names = list(bias_names)
        self.lora = lora
        self.lora_names = [n for n in self.names if lora is not None and n in lora.targets]
        self.tp = None                 # TensorParallel handle, bound by the layer when tensor parallelism is on
        self.tp_mode: Optional[str] = None      # "col" | "row"
        self._dy_full = None           # (data_ptr of the local dy, gathered dy) kept between dgrad and wgrad

    # -- effective weight ---------------------------------------------------------
    def weight(self, params: Dict[str, torch.Tensor]) -> torch.Tensor:
        """Effective (LoRA-merged) weight of the whole group as one matrix."""
        ws = [params[n] for n in self.names]
        if not self.lora_names:
            if len(ws) == 1:
                return ws[0]
            fv = fused_view(ws)
            return fv if fv is not None else torch.cat(ws, 0)
        key = "_eff_" + "+".join(self.names)
        cached = params.get(key)
        if cached is not None:
            return cached
        eff = torch.cat(ws, 0) if len(ws) > 1 else ws[0].clone()
        r0 = 0
        for n, w in zip(self.names, ws):
            if n in self.lora_names:
                a, b = params[n + "_lora_a"], params[n + "_lora_b"]
                ops.gemm(b.to(eff.dtype), a.to(eff.dtype), alpha=self.lora.scale, beta=1.0, out=eff[r0:r0 + w.shape[0]])
            r0 += w.shape[0]
        params[key] = eff
        return eff

    def bias(self, params) -> Optional[torch.Tensor]:
        if not self.bias_names:
            return None
        bs = [params[n] for n in self.bias_names]
        b = bs[0] if len(bs) == 1 else torch.cat(bs, 0)
        return b.to(torch.float32)

    # -- passes -------------------------------------------------------------------
    def fwd(self, x, params, *, residual=None, out=None):
        if self.tp is not None:
            return self._tp_fwd(x, params, residual, out)
        return ops.linear_fwd(x, self.weight(params), bias=self.bias(params), residual=residual, out=out)

    def dgrad(self, dy, params, *, out=None, accumulate=False):
        if self.tp is not None:
            return self._tp_dgrad(dy, params, out, accumulate)
        return ops.linear_dgrad(dy, self.weight(params), out=out, accumulate=accumulate)

    # -- tensor-parallel passes -----------------------------------------------------
    def _tp_fwd(self, x, params, residual, out):
        w = self.weight(params)
        if self.tp_mode == "col":
            y = self.tp.ag_gemm(x, w)                                   # (T, out/tp) from (T/tp, in)
            b = self.bias(params)
            if b is not None:
                y += b.to(y.dtype)
            if residual is not None:
                y += residual
        else:
            y = self.tp.gemm_rs(x, w, residual_local=residual)          # (T/tp, out) from (T, in/tp)
        if out is not None:
            out.copy_(y)
            return out
        return y

    def _tp_dgrad(self, dy, params, out, accumulate):
        w = self.weight(params)
        if self.tp_mode == "col":
            dx = self.tp.gemm_rs(dy, w, trans_w=False)                  # (T/tp, in)
        else:
            dx = self.tp.ag_gemm(dy, w, trans_w=False)                  # (T, in/tp); dy gathered on the way
            self._dy_full = (dy.data_ptr(), self.tp.last_gathered)
        if out is not None:
            if accumulate:
                out += dx
            else:
                out.copy_(dx)
            return out
        return dx

    def _tp_wgrad_operands(self, dy, x):
        """Full-token operands of the weight gradient: gather whichever side is token-sharded."""
        if self.tp_mode == "col":
            return dy, self.tp.all_gather(x)
        if self._dy_full is not None and self._dy_full[0] == dy.data_ptr():
            dyf = self._dy_full[1]
        else:
            dyf = self.tp.all_gather(dy)
        self._dy_full = None
        return dyf, x

    def wgrad(self, dy, x, params, grads, *, alpha: float = 1.0) -> None:
        """Accumulate weight (and bias / LoRA) gradients of every member from ``(x, dy)``."""
        if self.tp is not None:
            dy, x = self._tp_wgrad_operands(dy, x)
        gnames = ["g_" + n[2:] for n in self.names]
        trainable = [g in grads for g in gnames]
        if all(trainable) and not self.lora_names:
            gs = [grads[g] for g in gnames]
            fv = gs[0] if len(gs) == 1 else fused_view(gs)
            if fv is not None:
                ops.linear_wgrad(dy, x, fv, alpha=alpha)
                gs = None
            if gs is not None:
                r0 = 0
                for g in gs:
                    ops.linear_wgrad(dy[:, r0:r0 + g.shape[0]], x, g, alpha=alpha)
                    r0 += g.shape[0]
        else:
            r0 = 0
            for n, gname in zip(self.names, gnames):
                rows = params[n].shape[0]
                dyn = dy[:, r0:r0 + rows]
                if gname in grads:
                    ops.linear_wgrad(dyn, x, grads[gname], alpha=alpha)
                if n in self.lora_names:
                    self._lora_wgrad(n, dyn, x, params, grads, alpha)
                r0 += rows
        if self.bias_names:
            r0 = 0
            for n, bn in zip(self.names, self.bias_names):
                rows = params[n].shape[0]
                gb = "g_" + bn
                if gb in grads:
                    ops.bias_grad(dy[:, r0:r0 + rows], grads[gb], alpha=alpha)
                r0 += rows

    def _lora_wgrad(self, n, dy, x, params, grads, alpha):
        s = self.lora.scale * alpha
        a, b = params[n + "_lora_a"], params[n + "_lora_b"]
        ga, gb = grads.get("g_" + n[2:] + "_lora_a"), grads.get("g_" + n[2:] + "_lora_b")
        if ga is None:
            return
        dyb = ops.gemm(dy.contiguous() if dy.stride(-1) != 1 else dy, b.to(dy.dtype))          # (T, r)
        xa = ops.gemm(x, a.to(x.dtype), trans_b=True)                                            # (T, r)
        ops.gemm(dyb, x, trans_a=True, alpha=s, beta=1.0, out=ga)                                # (r, in)
        ops.gemm(dy, xa, trans_a=True, alpha=s, beta=1.0, out=gb)                                # (out, r)


def clear_effective_weights(params: Dict[str, torch.Tensor]) -> None:
    """Drop cached LoRA-merged weights (call after every optimizer step)."""
    for k in [k for k in params if k.startswith("_eff_")]:
        del params[k]
