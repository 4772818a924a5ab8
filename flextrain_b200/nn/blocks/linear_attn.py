"""Gated DeltaNet linear-attention block (Qwen3-Next / Qwen3.5 hybrid layers).

Pipeline (flextrain/nn/blocks/linear_attn.py:1-43, 1027-1184):
``h @ W_qkvz`` and ``h @ W_ba`` → depthwise causal conv1d (+SiLU) over ``[q‖k‖v]`` → L2-norm(q, k) →
gated delta rule with ``g = -exp(A_log) * softplus(a + dt_bias)``, ``beta = sigmoid(b)`` →
gated RMSNorm ``rmsnorm(o) * w * silu(z)`` → out-projection + residual.

Cross-chunk state: the recurrent state ``(HV, dk, dv)`` fp32 and the conv tail ``(conv_dim, W-1)`` at
the end of a chunk are tier-0 fields; the engine threads them (and their gradients, in reverse)
between the chunks of one sequence through ``LayerContext``.

The only tensors kept per chunk are the boundary states, which is the reference's tier-0 footprint
(``lin_final_state``, ``lin_conv_state``); backward recomputes the block from its input.

Two implementations of the same math:

* **CUDA (bf16)**: hand-written forward and backward, no autograd: tcgen05 GEMMs for the projections, the conv1d /
  L2-norm / gated-RMSNorm kernels of ``csrc/seqmix.cu`` and the recurrent delta-rule kernels of ``csrc/gdn.cu``
  (forward pass; backward = one reverse pass for the state adjoint + one forward-direction pass for the
  state-dependent terms; the gate gradient is a suffix sum of per-token scalars).
* **Reference (any device / dtype)**: the fp32 PyTorch formulation under autograd; it is the CPU path and the oracle
  the CUDA path is tested against.  ``FTB_GDN_BACKEND=reference`` forces it.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

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

    # ------------------------------------------------------------------- CUDA path
    def _use_cuda(self, h) -> bool:
        from ...ops import linattn_cuda as la
        c = self.cfg
        return (h.is_cuda and h.dtype == torch.bfloat16 and os.environ.get("FTB_GDN_BACKEND", "cuda") != "reference"
                and la.gdn_supported(c.head_k_dim, c.head_v_dim) and c.conv_width <= 8)

    def _cuda_forward(self, h, meta: ChunkMeta, p, state_in, conv_in, want_r: bool):
        """Everything up to the gated norm; returns the intermediates the backward needs."""
        from ...ops import linattn_cuda as la
        c = self.cfg
        T = h.shape[0]
        f32 = torch.float32
        cu = meta.cu_seqlens_q
        qkvz = ops.gemm(h, p["w_lin_qkvz"], trans_b=True)
        ba = ops.gemm(h, p["w_lin_ba"], trans_b=True)
        qkv, z2d = qkvz[:, : c.conv_dim], qkvz[:, c.conv_dim:]
        qkv_c, conv_fin = la.conv1d_fwd(qkv, p["w_lin_conv"], cu, conv_in, activation=True)
        qn, q_rn = la.l2norm_heads_fwd(qkv_c[:, : c.key_dim], c.n_k_heads, c.head_k_dim)
        kn, k_rn = la.l2norm_heads_fwd(qkv_c[:, c.key_dim: 2 * c.key_dim], c.n_k_heads, c.head_k_dim)
        v = qkv_c[:, 2 * c.key_dim:].contiguous().view(T, c.n_v_heads, c.head_v_dim)
        # gates in one launch straight from the bf16 projection (flextrain/ops/_kernels/gate_prep.py:29-80)
        beta, g = la.gate_prep_fwd(ba.contiguous(), p["w_lin_dt_bias"].to(f32), p["w_lin_A_log"].to(f32))
        o, fin, r = la.gdn_fwd(qn, kn, v, g, beta, cu, state_in, want_r=want_r)
        z = z2d.contiguous().view(T * c.n_v_heads, c.head_v_dim)
        on = ops.gated_rmsnorm_fwd(o.view(T * c.n_v_heads, c.head_v_dim), z, p["w_lin_norm"].to(f32), c.norm_eps)
        return dict(qkvz=qkvz, qkv_c=qkv_c, conv_fin=conv_fin, qn=qn, kn=kn, q_rn=q_rn, k_rn=k_rn, v=v, ba=ba,
                    beta=beta, g=g, o=o, fin=fin, r=r, on=on.view(T, c.value_dim))

    def _fwd_cuda(self, h, x_resid, meta, params, slot, ctx):
        s = self._cuda_forward(h, meta, params, ctx.lin_state_in, ctx.lin_conv_in, want_r=False)
        out = ops.linear_fwd(s["on"], params["w_lin_out"], residual=x_resid)
        if not ctx.lin_attn_recompute_only:
            slot.put("lin_final_state", s["fin"][:1])
            slot.put("lin_conv_state", s["conv_fin"][:1].to(self.dtype))
            ctx.out["lin_state"], ctx.out["lin_conv"] = s["fin"], s["conv_fin"].to(self.dtype)
        return out

    def _bwd_cuda(self, dx, h, meta, params, grads, slot, ctx):
        from ...ops import linattn_cuda as la
        c = self.cfg
        T = h.shape[0]
        f32 = torch.float32
        cu = meta.cu_seqlens_q
        s = self._cuda_forward(h, meta, params, ctx.lin_state_in, ctx.lin_conv_in, want_r=True)
        acc = lambda name, val: grads[name].add_(val.to(grads[name].dtype)) if name in grads else None
        # ---- out-projection and gated norm
        d_on = ops.linear_dgrad(dx, params["w_lin_out"])
        if "g_lin_out" in grads:
            ops.linear_wgrad(dx, s["on"], grads["g_lin_out"])
        dqkvz = torch.empty_like(s["qkvz"])
        dwn = torch.zeros(c.head_v_dim, dtype=f32, device=h.device)
        d_o = la.gated_rmsnorm_bwd(d_on.view(T, c.n_v_heads, c.head_v_dim), s["o"], s["qkvz"][:, c.conv_dim:],
                                   params["w_lin_norm"].to(f32), dqkvz[:, c.conv_dim:], dwn, c.n_v_heads,
                                   c.head_v_dim, c.norm_eps)
        acc("g_lin_norm", dwn)
        # ---- recurrence
        dq, dk, dv, dg, dbeta, dstate_in = la.gdn_bwd(s["qn"], s["kn"], s["v"], s["g"], s["beta"], cu, ctx.lin_state_in,
                                                      s["fin"], s["r"], d_o, dstate_final=ctx.lin_dstate_in)
        # ---- L2 norms and conv
        dqkv_c = torch.empty(T, c.conv_dim, dtype=h.dtype, device=h.device)
        la.l2norm_heads_bwd(dq.contiguous(), s["qkv_c"][:, : c.key_dim], s["q_rn"], dqkv_c[:, : c.key_dim],
                            c.n_k_heads, c.head_k_dim)
        la.l2norm_heads_bwd(dk.contiguous(), s["qkv_c"][:, c.key_dim: 2 * c.key_dim], s["k_rn"],
                            dqkv_c[:, c.key_dim: 2 * c.key_dim], c.n_k_heads, c.head_k_dim)
        dqkv_c[:, 2 * c.key_dim:].copy_(dv.view(T, c.value_dim))
        dwc = torch.zeros(c.conv_dim, c.conv_width, dtype=f32, device=h.device)
        dconv_in = la.conv1d_bwd(s["qkvz"][:, : c.conv_dim], params["w_lin_conv"], cu, ctx.lin_conv_in, dqkv_c,
                                 ctx.lin_dconv_in, dqkvz[:, : c.conv_dim], dwc, want_dinit=ctx.lin_conv_in is not None)
        acc("g_lin_conv", dwc)
        # ---- gates:  beta = sigmoid(b);  g = -exp(A_log) * softplus(a + dt_bias)
        d_alog = torch.zeros(c.n_v_heads, dtype=f32, device=h.device)
        d_dtb = torch.zeros(c.n_v_heads, dtype=f32, device=h.device)
        dba = la.gate_prep_bwd(s["ba"].contiguous(), params["w_lin_dt_bias"].to(f32), params["w_lin_A_log"].to(f32),
                               s["g"], dbeta, dg, d_alog, d_dtb)
        acc("g_lin_A_log", d_alog)
        acc("g_lin_dt_bias", d_dtb)
        # ---- input projections
        dh = ops.linear_dgrad(dqkvz, params["w_lin_qkvz"])
        dh = ops.linear_dgrad(dba, params["w_lin_ba"], out=dh, accumulate=True)
        if "g_lin_qkvz" in grads:
            ops.linear_wgrad(dqkvz, h, grads["g_lin_qkvz"])
        if "g_lin_ba" in grads:
            ops.linear_wgrad(dba, h, grads["g_lin_ba"])
        if ctx.lin_state_in is not None:
            ctx.out["lin_dstate"] = dstate_in
        if ctx.lin_conv_in is not None:
            ctx.out["lin_dconv"] = dconv_in
        return dh

    # --------------------------------------------------------------------- forward
    def fwd(self, h, x_resid, meta: ChunkMeta, params, slot, ctx: LayerContext):
        if self._use_cuda(h):
            return self._fwd_cuda(h, x_resid, meta, params, slot, ctx)
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
        if self._use_cuda(h):
            return self._bwd_cuda(dx, h, meta, params, grads, slot, ctx)
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
