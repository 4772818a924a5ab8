"""Routed mixture-of-experts SwiGLU FFN (optionally with a gated shared expert).

Weights follow flextrain/nn/blocks/ffn_moe.py:12-19 transposed to (out, in):
``w_router (E, d)``, ``w_up (E, 2F, d)`` with the 2F axis ``[up ‖ gate]`` (value first, gate second),
``w_down (E, d, F)``.  The reference runs a Python loop of per-expert cuBLASLt calls after a
host sync on the expert counts (flextrain/ops/full_moe.py:134-148, 393-466); here routing,
the counting sort, both grouped GEMMs and the weighted combine stay on the device:

    logits -> top-k -> plan (expert-major rows, each expert padded to a tile multiple)
    x_sorted = gather(h)             up = grouped_gemm(x_sorted, w_up)       act = glu(up)
    y = grouped_gemm(act, w_down)    out = resid + sum_k weight * y[row(t,k)]

Under expert parallelism (``ctx.ep``) the gather / combine become the all-to-all dispatch and
combine of ``flextrain_b200.parallel.ep``.
Saved tiers (flextrain/nn/blocks/ffn_moe.py:176-223): routing state tier 0, ``x_up`` tier 3.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ... import ops
from ...core.activation_schema import ActivationField
from ...core.layer import LayerContext, TensorSpec
from ...ops import moe_dump
from ...ops import reference as ref
from .ffn_dense import DenseFFNConfig, GatedFFN
from .linear import LinearGroup, LoRAConfig

ROW_PAD = 128        # expert row segments are padded to the GEMM tile height


@dataclass
class MoEConfig:
    d_model: int
    num_experts: int
    top_k: int
    expert_dim: int
    routing: str = "topk_then_softmax"        # or "softmax_then_topk"
    aux_loss_alpha: float = 0.0
    shared_dim: int = 0                        # > 0: one shared expert of this width
    shared_gate: bool = True                   # sigmoid(h @ w_shared_gate) scales the shared expert
    kind: str = "swiglu"


class MoEFFN:
    def __init__(self, cfg: MoEConfig, *, dtype=torch.bfloat16, lora: Optional[LoRAConfig] = None):
        self.cfg = cfg
        self.dtype = dtype
        # per-expert LoRA on the routed stacks (flextrain/nn/layers/lora_wrapper.py:656-838)
        self.lora = lora if (lora is not None and any(t in lora.targets for t in ("w_up", "w_down"))) else None
        self.shared = None
        if cfg.shared_dim > 0:
            self.shared = GatedFFN(DenseFFNConfig(cfg.d_model, cfg.shared_dim, cfg.kind), dtype=dtype, lora=None)
            self.shared.up = LinearGroup(["w_shared_1", "w_shared_3"], None)
            self.shared.down = LinearGroup(["w_shared_2"], None)

    # ------------------------------------------------------------------ declarations
    def tensor_specs(self):
        c, dt = self.cfg, self.dtype
        specs = [TensorSpec("w_router", (c.num_experts, c.d_model), dt, optimizer="adamw"),
                 TensorSpec("w_up", (c.num_experts, 2 * c.expert_dim, c.d_model), dt),
                 TensorSpec("w_down", (c.num_experts, c.d_model, c.expert_dim), dt)]
        for s in specs[1:]:
            s.shard = type(s.shard)(ep_dim=0)
        if self.shared is not None:
            specs += [TensorSpec("w_shared_1", (c.shared_dim, c.d_model), dt),
                      TensorSpec("w_shared_3", (c.shared_dim, c.d_model), dt),
                      TensorSpec("w_shared_2", (c.d_model, c.shared_dim), dt)]
            if c.shared_gate:
                specs.append(TensorSpec("w_shared_gate", (1, c.d_model), dt, optimizer="adamw"))
        return specs

    ep_world = 1                   # set by the API under expert parallelism (with the receive capacity factor)
    ep_capacity_factor = 1.0

    def rows_bound(self, T: int) -> int:
        c = self.cfg
        if self.ep_world > 1:
            # rows this rank is PLANNED to receive for its experts from all ranks' chunks of T tokens (the saved
            # x_up is sized by what actually arrives; the receive buffers by the worst case)
            from ...parallel.ep import PLANNING_FACTOR, ep_capacity
            return ep_capacity(T, c.top_k, c.num_experts, self.ep_world, PLANNING_FACTOR)
        return ref.moe_rows_bound(T, c.top_k, c.num_experts, ROW_PAD)

    def activation_fields(self):
        c, dt = self.cfg, self.dtype
        f = [ActivationField("router_weights", lambda t: (t, c.top_k), torch.float32, 0),
             ActivationField("chosen_experts", lambda t: (t, c.top_k), torch.int32, 0),
             ActivationField("x_up", lambda t: (self.rows_bound(t), 2 * c.expert_dim), dt, 3)]
        if self.shared is not None:
            f.append(ActivationField("x13_shared", lambda t: (t, 2 * c.shared_dim), dt, 3))
        return f

    # ------------------------------------------------------------------ per-expert LoRA
    def weight(self, params, name: str) -> torch.Tensor:
        """Effective expert stack ``W'[e] = W[e] + s * B[e] @ A[e]`` (cached in ``params`` until the optimizer step).
        The merge is ONE grouped GEMM with K = r over the stacked ``B`` rows (expert e owns rows ``e*out .. (e+1)*out``),
        accumulated in place into a copy of the base stack."""
        w = params[name]
        a = params.get(name + "_lora_a")
        if self.lora is None or a is None:
            return w
        key = "_eff_" + name
        eff = params.get(key)
        if eff is None:
            b = params[name + "_lora_b"]
            n_e, out_f, in_f = w.shape
            eff = w.clone()
            offs = torch.arange(n_e + 1, dtype=torch.int32, device=w.device) * out_f
            ops.grouped_gemm(b.to(w.dtype).reshape(n_e * out_f, -1), a.to(w.dtype).contiguous(), offs, trans_w=False,
                             out=eff.view(n_e * out_f, in_f), alpha=self.lora.scale, beta=1.0)
            params[key] = eff
        return eff

    def lora_wgrad(self, name: str, dy, x, offsets, params, grads, pad: int) -> None:
        """Rank-r gradients of one expert stack from the expert-major rows ``x (R, in)`` / ``dy (R, out)``:
        ``gB[e] += s * dy_e^T (x_e A_e^T)``, ``gA[e] += s * (dy_e B_e)^T x_e`` -- two grouped GEMMs with N = r and two
        grouped weight-gradient launches, for all experts at once."""
        ga = grads.get("g_" + name[2:] + "_lora_a")
        if self.lora is None or ga is None:
            return
        gb = grads["g_" + name[2:] + "_lora_b"]
        s = self.lora.scale
        a, b = params[name + "_lora_a"].to(x.dtype), params[name + "_lora_b"].to(x.dtype)
        xa = ops.grouped_gemm(x, a, offsets, trans_w=True)               # (R, r)
        ops.grouped_wgrad(dy, xa, offsets, gb, alpha=s, pad=pad)
        dyb = ops.grouped_gemm(dy, b, offsets, trans_w=False)            # (R, r)
        ops.grouped_wgrad(dyb, x, offsets, ga, alpha=s, pad=pad)

    # --------------------------------------------------------------------- helpers
    def _route(self, h, params):
        c = self.cfg
        logits = ops.gemm(h, params["w_router"], trans_b=True)
        w, idx = ops.topk_route(logits, c.top_k, c.routing)
        return logits, w, idx

    def _experts_fwd(self, h, params, plan, x_up_out=None):
        F = self.cfg.expert_dim
        xs = ops.gather_rows(h, plan.row_src, idx_div=self.cfg.top_k)
        up = ops.grouped_gemm(xs, self.weight(params, "w_up"), plan.offsets)
        if x_up_out is not None and x_up_out.data_ptr() != up.data_ptr():
            x_up_out.copy_(up)
            up = x_up_out
        act = ops.glu_fwd(up[:, F:], up[:, :F], self.cfg.kind)
        return xs, up, act

    def _shared_fwd(self, h, params, slot):
        c = self.cfg
        y = self.shared.fwd(_Rename(h), None, _SharedParams(params), _SharedSlot(slot))
        if c.shared_gate:
            g = torch.sigmoid(ops.gemm(h, params["w_shared_gate"], trans_b=True).to(torch.float32))
            return y, g
        return y, None

    # --------------------------------------------------------------------- forward
    def fwd(self, h, x_resid, params, slot, ctx: LayerContext):
        c = self.cfg
        logits, w, idx = self._route(h, params)
        slot.put("router_weights", w)
        slot.put("chosen_experts", idx)
        if ctx.ep is not None:
            out = ctx.ep.moe_forward(self, h, x_resid, w, idx, params, slot)
        else:
            plan = ops.moe_plan(idx, c.num_experts, ROW_PAD)
            _, up, act = self._experts_fwd(h, params, plan, slot.out("x_up", h.device))
            y = ops.grouped_gemm(act, self.weight(params, "w_down"), plan.offsets)
            out = ops.moe_combine(y, plan.inv, w, x_resid)
        if self.shared is not None:
            ys, g = self._shared_fwd(h, params, slot)
            out = (out.to(torch.float32) + (ys.to(torch.float32) * g if g is not None else ys.to(torch.float32))).to(out.dtype)
        if moe_dump.DUMP_DIR is not None:
            moe_dump.dump(router_logits=logits, router_weights=w, chosen_experts=idx, output=out)
        return out

    def recompute(self, h, params, slot) -> None:
        if not slot.has("x_up"):
            plan = ops.moe_plan(slot._t["chosen_experts"], self.cfg.num_experts, ROW_PAD)
            _, up, _ = self._experts_fwd(h, params, plan)
            slot._t["x_up"] = up
        if self.shared is not None and not slot.has("x13_shared"):
            slot._t["x13_shared"] = self.shared.up.fwd(h, _SharedParams(params))

    # -------------------------------------------------------------------- backward
    def bwd(self, dx, h, params, grads, slot, ctx: LayerContext):
        """Full backward including weight gradients (``h`` = normed FFN input). Returns ``dh``."""
        c = self.cfg
        F, K, E = c.expert_dim, c.top_k, c.num_experts
        w, idx = slot._t["router_weights"], slot._t["chosen_experts"]
        if ctx.ep is not None:
            dh, dw = ctx.ep.moe_backward(self, dx, h, w, idx, params, grads, slot)
        else:
            plan = ops.moe_plan(idx, E, ROW_PAD)
            up = slot._t["x_up"]
            xs = ops.gather_rows(h, plan.row_src, idx_div=K)
            dy_u = ops.gather_rows(dx, plan.row_src, idx_div=K)                         # unweighted dL/dy rows
            dact_u = ops.grouped_gemm(dy_u, self.weight(params, "w_down"), plan.offsets, trans_w=False)
            # activation (re-emitted), router-weight gradient and weighted dact in one pass
            wrow = ref.moe_row_weights(w, plan)
            dup = torch.empty_like(up)
            act_w, dw_rows = ops.glu_bwd_weighted(dact_u, up[:, F:], up[:, :F], wrow, c.kind, dgate=dup[:, F:],
                                                  dup=dup[:, :F])
            dw = ref.moe_rows_to_slots(dw_rows, plan, w.shape)
            if "g_down" in grads:       # g_down += dy^T (w * act): the router weight rides on the activation
                ops.grouped_wgrad(dy_u, act_w, plan.offsets, grads["g_down"], pad=ROW_PAD)
            if "g_up" in grads:
                ops.grouped_wgrad(dup, xs, plan.offsets, grads["g_up"], pad=ROW_PAD)
            self.lora_wgrad("w_down", dy_u, act_w, plan.offsets, params, grads, ROW_PAD)
            self.lora_wgrad("w_up", dup, xs, plan.offsets, params, grads, ROW_PAD)
            dxs = ops.grouped_gemm(dup, self.weight(params, "w_up"), plan.offsets, trans_w=False)
            dh = ops.moe_combine(dxs, plan.inv, None, None)
        # router
        logits = ops.gemm(h, params["w_router"], trans_b=True)
        dlogits = ops.topk_route_bwd(dw, logits, w, idx, c.routing)
        if c.aux_loss_alpha > 0 and ctx.total_tokens_per_step > 0:
            dlogits = ops.load_balance_bwd_(dlogits.contiguous(), logits, idx, c.aux_loss_alpha,
                                            ctx.total_tokens_per_step)
        dl = dlogits.to(h.dtype)
        dh = ops.gemm(dl, params["w_router"], beta=1.0, out=dh)
        if "g_router" in grads:
            ops.gemm(dl, h, trans_a=True, beta=1.0, out=grads["g_router"])
        if self.shared is not None:
            dh = self._shared_bwd(dx, h, dh, params, grads, slot)
        return dh

    def _shared_bwd(self, dx, h, dh, params, grads, slot):
        c = self.cfg
        sp, ss = _SharedParams(params), _SharedSlot(slot)
        if c.shared_gate:
            F = c.shared_dim
            x13 = slot._t["x13_shared"]
            act = ops.glu_fwd(x13[:, :F], x13[:, F:], c.kind)
            ys = self.shared.down.fwd(act, sp)
            z = ops.gemm(h, params["w_shared_gate"], trans_b=True).to(torch.float32)
            g = torch.sigmoid(z)
            dg = (dx.to(torch.float32) * ys.to(torch.float32)).sum(-1, keepdim=True) * g * (1 - g)
            dgb = dg.to(h.dtype)
            dh = ops.gemm(dgb, params["w_shared_gate"], beta=1.0, out=dh)
            if "g_shared_gate" in grads:
                ops.gemm(dgb, h, trans_a=True, beta=1.0, out=grads["g_shared_gate"])
            dxs = (dx.to(torch.float32) * g).to(dx.dtype)
        else:
            dxs = dx
        dhs, dx13 = self.shared.bwd(dxs, sp, _SharedGrads(grads), ss)
        self.shared.up.wgrad(dx13, h, sp, _SharedGrads(grads))
        return (dh.to(torch.float32) + dhs.to(torch.float32)).to(dh.dtype)

    def flops(self, T: int):
        c = self.cfg
        routed = 2.0 * T * c.top_k * c.d_model * 3 * c.expert_dim
        router = 2.0 * T * c.d_model * c.num_experts
        shared = 2.0 * T * c.d_model * 3 * c.shared_dim
        return router, routed, shared


class _Rename:
    """Identity wrapper kept for readability at call sites (``h`` passes through)."""

    def __new__(cls, x):
        return x


class _SharedParams(dict):
    """View of the layer's params where the shared expert's tensors appear under their own names."""

    def __init__(self, params):
        super().__init__(params)


class _SharedGrads(dict):
    def __init__(self, grads):
        super().__init__(grads)


class _SharedSlot:
    """Maps the dense FFN's ``x13`` field onto ``x13_shared`` of the MoE slot."""

    def __init__(self, slot):
        self.s = slot
        self._t = _SharedSlotDict(slot)

    def out(self, name, device):
        return self.s.out("x13_shared", device)

    def has(self, name):
        return self.s.has("x13_shared")


class _SharedSlotDict:
    def __init__(self, slot):
        self.s = slot

    def __getitem__(self, k):
        return self.s._t["x13_shared"]

    def __setitem__(self, k, v):
        self.s._t["x13_shared"] = v
