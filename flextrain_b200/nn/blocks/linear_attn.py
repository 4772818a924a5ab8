"""Gated DeltaNet linear-attention block (Qwen3-Next / Qwen3.5 hybrid layers).

Pipeline (flextrain/nn/blocks/linear_attn.py:1-43, 1027-1184):
``h @ W_qkvz`` and ``h @ W_ba`` → depthwise causal conv1d (+SiLU) over ``[q‖k‖v]`` → L2-norm(q, k) →
gated delta rule with ``g = -exp(A_log) * softplus(a + dt_bias)``, ``beta = sigmoid(b)`` →
gated RMSNorm ``rmsnorm(o) * w * silu(z)`` → out-projection + residual.

Cross-chunk state: the recurrent state ``(HV, dk, dv)`` fp32 and the conv tail ``(conv_dim, W-1)`` at
the end of a chunk are tier-0 fields; the engine threads them (and their gradients, in reverse)
between the chunks of one sequence through ``LayerContext``.

Backward re-runs the block's forward under autograd on the saved input (an activation-
recompute backward): the only tensors kept per chunk are the boundary states, which is the
reference's tier-0 footprint (``lin_final_state``, ``lin_conv_state``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from ... import ops
from ...core.activation_schema import ActivationField
from ...core.layer import ChunkMeta, LayerContext, TensorSpec
from ...ops import reference as ref


@dataclass
class GDNConfig:
    d_model: int
    n_k_heads: int
    n_v_heads: int
    head_k_dim: int
    head_v_dim: int
    conv_width: int = 4
    norm_eps: float = 1e-6

    @property
    def key_dim(self):
        return self.n_k_heads * self.head_k_dim

    @property
    def value_dim(self):
        return self.n_v_heads * self.head_v_dim

    @property
    def conv_dim(self):
        return 2 * self.key_dim + self.value_dim


class GatedDeltaNetBlock:
    PARAMS = ("w_lin_qkvz", "w_lin_ba", "w_lin_conv", "w_lin_dt_bias", "w_lin_A_log", "w_lin_norm", "w_lin_out")

    def __init__(self, cfg: GDNConfig, *, dtype=torch.bfloat16, norm_dtype=torch.float32):
        self.cfg, self.dtype, self.norm_dtype = cfg, dtype, norm_dtype

    def tensor_specs(self):
        c, dt = self.cfg, self.dtype
        return [TensorSpec("w_lin_qkvz", (2 * c.key_dim + 2 * c.value_dim, c.d_model), dt),
                TensorSpec("w_lin_ba", (2 * c.n_v_heads, c.d_model), dt, optimizer="adamw"),
                TensorSpec("w_lin_conv", (c.conv_dim, c.conv_width), dt, optimizer="adamw"),
                TensorSpec("w_lin_dt_bias", (c.n_v_heads,), torch.float32, init="ones", optimizer="adamw"),
                TensorSpec("w_lin_A_log", (c.n_v_heads,), torch.float32, init="zeros", optimizer="adamw"),
                TensorSpec("w_lin_norm", (c.head_v_dim,), self.norm_dtype, init="ones"),
                TensorSpec("w_lin_out", (c.d_model, c.value_dim), dt)]

    def activation_fields(self):
        c = self.cfg
        return [ActivationField("lin_final_state", lambda t: (1, c.n_v_heads, c.head_k_dim, c.head_v_dim),
                                torch.float32, 0, per_seq=True),
                ActivationField("lin_conv_state", lambda t: (1, c.conv_dim, c.conv_width - 1), self.dtype, 0,
                                per_seq=True)]

    # ------------------------------------------------------------------------ core
    def _core(self, h, x_resid, meta: ChunkMeta, p, state_in, conv_in):
        """Differentiable forward. Returns ``(out, final_state, final_conv)``."""
        c = self.cfg
        T = h.shape[0]
        f32 = torch.float32
        qkvz = (h.to(f32) @ p["w_lin_qkvz"].to(f32).t())
        ba = (h.to(f32) @ p["w_lin_ba"].to(f32).t())
        qkv, z = qkvz[:, : c.conv_dim], qkvz[:, c.conv_dim:]
        b, a = ba[:, : c.n_v_heads], ba[:, c.n_v_heads:]
        qkv_c, conv_fin = ref.causal_conv1d_fwd(qkv, p["w_lin_conv"].to(f32), meta.cu_seqlens_q,
                                                conv_in.to(f32) if conv_in is not None else None, activation=True)
        q = qkv_c[:, : c.key_dim].reshape(T, c.n_k_heads, c.head_k_dim)
        k = qkv_c[:, c.key_dim: 2 * c.key_dim].reshape(T, c.n_k_heads, c.head_k_dim)
        v = qkv_c[:, 2 * c.key_dim:].reshape(T, c.n_v_heads, c.head_v_dim)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6)
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(b)
        g = -torch.exp(p["w_lin_A_log"].to(f32)) * F.softplus(a + p["w_lin_dt_bias"].to(f32))
        rule = ref.gated_delta_rule if T <= 64 else ref.gated_delta_rule_chunked
        o, fin = rule(q, k, v, g, beta, meta.cu_seqlens_q, state_in)
        o = o.to(f32)
        zz = z.reshape(T, c.n_v_heads, c.head_v_dim)
        r = torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + c.norm_eps)
        on = (o * r * p["w_lin_norm"].to(f32) * F.silu(zz)).reshape(T, c.value_dim)
        out = on @ p["w_lin_out"].to(f32).t()
        if x_resid is not None:
            out = out + x_resid.to(f32)
        return out, fin, conv_fin

    # --------------------------------------------------------------------- forward
    def fwd(self, h, x_resid, meta: ChunkMeta, params, slot, ctx: LayerContext):
        with torch.no_grad():
            out, fin, conv_fin = self._core(h, x_resid, meta, params, ctx.lin_state_in, ctx.lin_conv_in)
        if not ctx.lin_attn_recompute_only:
            slot.put("lin_final_state", fin[:1] if fin.shape[0] >= 1 else fin)
            slot.put("lin_conv_state", conv_fin[:1].to(self.dtype))
            ctx.out["lin_state"], ctx.out["lin_conv"] = fin, conv_fin.to(self.dtype)
        return out.to(h.dtype)

    def recompute(self, h, params, slot) -> None:      # nothing above tier 0 is stored
        return None

    # -------------------------------------------------------------------- backward
    def bwd(self, dx, h, meta: ChunkMeta, params, grads, slot, ctx: LayerContext):
        """Returns ``dh``; accumulates all parameter gradients; hands back state gradients via ``ctx.out``."""
        names = [n for n in self.PARAMS]
        leaf = {n: params[n].detach().to(torch.float32).requires_grad_("g_" + n[2:] in grads) for n in names}
        hh = h.detach().to(torch.float32).requires_grad_(True)
        s_in = ctx.lin_state_in.detach().to(torch.float32).requires_grad_(True) if ctx.lin_state_in is not None else None
        c_in = ctx.lin_conv_in.detach().to(torch.float32).requires_grad_(True) if ctx.lin_conv_in is not None else None
        with torch.enable_grad():
            out, fin, conv_fin = self._core(hh, None, meta, leaf, s_in, c_in)
            outs, gos = [out], [dx.to(torch.float32)]
            if ctx.lin_dstate_in is not None:
                outs.append(fin); gos.append(ctx.lin_dstate_in.to(torch.float32))
            if ctx.lin_dconv_in is not None:
                outs.append(conv_fin); gos.append(ctx.lin_dconv_in.to(torch.float32))
            wrt = [hh] + [leaf[n] for n in names if leaf[n].requires_grad]
            if s_in is not None:
                wrt.append(s_in)
            if c_in is not None:
                wrt.append(c_in)
            gr = torch.autograd.grad(outs, wrt, gos, allow_unused=True)
        it = iter(gr)
        dh = next(it)
        for n in names:
            if leaf[n].requires_grad:
                g = next(it)
                if g is not None:
                    grads["g_" + n[2:]].add_(g.to(grads["g_" + n[2:]].dtype))
        if s_in is not None:
            ctx.out["lin_dstate"] = next(it)
        if c_in is not None:
            ctx.out["lin_dconv"] = next(it)
        return dh.to(dx.dtype)

    def flops(self, T: int):
        c = self.cfg
        proj = 2.0 * T * c.d_model * (2 * c.key_dim + 2 * c.value_dim + 2 * c.n_v_heads)
        core = 2.0 * T * c.n_v_heads * c.head_k_dim * c.head_v_dim * 4
        return proj, core, 2.0 * T * c.value_dim * c.d_model
