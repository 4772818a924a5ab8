"""Config-driven decoder layer: one class composes the blocks for every supported family.

The reference has one hand-written class per family (``nn/layers/llama.py``, ``mistral.py``,
``qwen2.py``, ``qwen3.py``, ``qwen3_moe.py``, ``olmoe.py``, ``gemma2.py``, ``gemma3.py``,
``qwen3_5.py``, ``qwen3_next.py``); they differ only in which options of the same blocks are on.
Here a :class:`DecoderConfig` selects:

* mixer: GQA attention (bias / QK-norm / soft-cap / sliding window / output gate) or Gated DeltaNet
* FFN:   dense SwiGLU / GeGLU, or routed MoE (+ shared expert)
* norms: pre-norm (Llama) or sandwich pre+post norms (Gemma 2/3)

and the layer provides the engine contract: ``forward`` / ``forward_recompute`` / ``backward`` /
``compute_cost`` (canonical shape: flextrain/nn/layers/llama.py:95-479).  Tier layout of the
Llama-shaped layer (flextrain/nn/layers/llama.py:98-104): 0 ``x_inp, rstd's, xk, xv``;
1 ``attn_result, softmax_lse``; 2 ``xq, xo``; 3 ``x13``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ... import ops
from ...core.activation_schema import ActivationField, ActivationSchema
from ...core.layer import ChunkMeta, ComputeCost, LayerContext, ParamSpec, TensorSpec
from ..blocks.attention import AttentionConfig, GQAAttentionBlock
from ..blocks.ffn_dense import DenseFFNConfig, GatedFFN
from ..blocks.ffn_moe import MoEConfig, MoEFFN
from ..blocks.linear import LoRAConfig, clear_effective_weights
from ..blocks.linear_attn import GatedDeltaNetBlock, GDNConfig


@dataclass
class DecoderConfig:
    d_model: int
    attn: Optional[AttentionConfig] = None
    gdn: Optional[GDNConfig] = None
    ffn: Optional[DenseFFNConfig] = None
    moe: Optional[MoEConfig] = None
    norm_eps: float = 1e-5
    post_norms: bool = False
    dtype: torch.dtype = torch.bfloat16
    norm_dtype: torch.dtype = torch.float32
    grad_dtype: Optional[torch.dtype] = None
    norm_grad_dtype: torch.dtype = torch.float32
    master_dtype: Optional[torch.dtype] = None
    lora: Optional[LoRAConfig] = None
    family: str = "llama"
    layer_scalar: bool = False       # Gemma 4: the layer's output is multiplied by a stored, untrained scalar
    seq_parallel: int = 1            # tensor-parallel degree: the residual stream and norm statistics hold T / seq_parallel tokens


class DecoderLayer:
    def __init__(self, cfg: DecoderConfig, layer_id: int = 0):
        self.cfg = cfg
        self.layer_id = layer_id
        dt, nd = cfg.dtype, cfg.norm_dtype
        self.attn = GQAAttentionBlock(cfg.attn, dtype=dt, norm_dtype=nd, lora=cfg.lora) if cfg.attn else None
        self.gdn = GatedDeltaNetBlock(cfg.gdn, dtype=dt, norm_dtype=nd) if cfg.gdn else None
        self.ffn = GatedFFN(cfg.ffn, dtype=dt, lora=cfg.lora) if cfg.ffn else None
        self.moe = MoEFFN(cfg.moe, dtype=dt, lora=cfg.lora) if cfg.moe else None
        assert (self.attn is None) != (self.gdn is None) and (self.ffn is None) != (self.moe is None)
        self.param_spec = self._build_param_spec()
        self.activation_schema = self._build_schema()

    # ------------------------------------------------------------------ declarations
    def _build_param_spec(self) -> ParamSpec:
        c = self.cfg
        norm = lambda n: TensorSpec(n, (c.d_model,), c.norm_dtype, master_dtype=c.norm_dtype,
                                    grad_dtype=c.norm_grad_dtype, init="ones")
        specs = [norm("w_attn_norm")]
        specs += (self.attn or self.gdn).tensor_specs()
        if c.post_norms:
            specs.append(norm("w_post_attn_norm"))
        specs.append(norm("w_ffn_norm"))
        specs += (self.ffn or self.moe).tensor_specs()
        if c.post_norms:
            specs.append(norm("w_post_ffn_norm"))
        if c.layer_scalar:
            specs.append(TensorSpec("w_layer_scalar", (1,), torch.float32, master_dtype=torch.float32, init="ones",
                                    frozen=True))
        for s in specs:
            if "norm" in s.name:
                s.grad_dtype = c.norm_grad_dtype
                s.master_dtype = c.norm_dtype
            else:
                if c.grad_dtype is not None and s.compute_dtype != torch.float32:
                    s.grad_dtype = c.grad_dtype
                if c.master_dtype is not None and s.compute_dtype != torch.float32:
                    s.master_dtype = c.master_dtype
        if c.lora is not None:
            lo, extra = c.lora, []
            for s in specs:
                s.frozen = True
                if s.name in lo.targets and len(s.shape) == 2:
                    out_f, in_f = s.shape
                    extra.append(TensorSpec(s.name + "_lora_a", (lo.rank, in_f), lo.compute_dtype,
                                            master_dtype=lo.master_dtype, grad_dtype=lo.grad_dtype,
                                            opt_state_dtype=lo.opt_state_dtype, optimizer="adamw"))
                    extra.append(TensorSpec(s.name + "_lora_b", (out_f, lo.rank), lo.compute_dtype,
                                            master_dtype=lo.master_dtype, grad_dtype=lo.grad_dtype,
                                            opt_state_dtype=lo.opt_state_dtype, optimizer="adamw", init="zeros"))
                elif s.name in lo.targets and len(s.shape) == 3 and s.shard.ep_dim == 0:
                    # routed-expert stack (E, out, in): one rank-r pair per expert, sharded with the experts
                    n_e, out_f, in_f = s.shape
                    for suffix, shape, init in (("_lora_a", (n_e, lo.rank, in_f), None),
                                                ("_lora_b", (n_e, out_f, lo.rank), "zeros")):
                        t = TensorSpec(s.name + suffix, shape, lo.compute_dtype, master_dtype=lo.master_dtype,
                                       grad_dtype=lo.grad_dtype, opt_state_dtype=lo.opt_state_dtype, optimizer="adamw",
                                       **({"init": init} if init else {}))
                        t.shard = type(s.shard)(ep_dim=0)
                        extra.append(t)
            specs += extra
        return ParamSpec(specs)

    def _build_schema(self) -> ActivationSchema:
        c, d, dt = self.cfg, self.cfg.d_model, self.cfg.dtype
        f32 = torch.float32
        sp = max(1, c.seq_parallel)
        fields = [ActivationField("x_inp", lambda t: (t // sp, d), dt, 0),
                  ActivationField("attn_norm_rstd", lambda t: (t // sp,), f32, 0),
                  ActivationField("ffn_norm_rstd", lambda t: (t // sp,), f32, 0)]
        fields += (self.attn or self.gdn).activation_fields()
        fields.append(ActivationField("xo", lambda t: (t // sp, d), dt, 2))
        fields += (self.ffn or self.moe).activation_fields()
        if c.post_norms:
            # the branch outputs come out of the row-parallel projections, i.e. already token-sharded
            fields += [ActivationField("post_attn_rstd", lambda t: (t // sp,), f32, 0),
                       ActivationField("post_ffn_rstd", lambda t: (t // sp,), f32, 0),
                       ActivationField("attn_branch", lambda t: (t // sp, d), dt, 2),
                       ActivationField("ffn_branch", lambda t: (t // sp, d), dt, 3)]
        return ActivationSchema(fields, max_tier=3)

    # --------------------------------------------------------------------- forward
    def _mixer_fwd(self, h1, resid, meta, params, slot, ctx):
        if self.attn is not None:
            qkv = None
            if ctx.param_gather is not None:
                # first use of this layer's weights in the step: the QKV projection also gathers the layer's parameters
                qkv = ctx.param_gather(self.layer_id, h1, self.attn.qkv.weight(params))
            return self.attn.fwd(h1, resid, meta, params, slot, ctx, qkv=qkv)
        return self.gdn.fwd(h1, resid, meta, params, slot, ctx)

    def _ffn_fwd(self, h2, resid, params, slot, ctx):
        if self.ffn is not None:
            return self.ffn.fwd(h2, resid, params, slot)
        return self.moe.fwd(h2, resid, params, slot, ctx)

    def forward(self, x, meta: ChunkMeta, params: Dict[str, torch.Tensor], slot, ctx: LayerContext):
        out = self._forward(x, meta, params, slot, ctx)
        if self.cfg.layer_scalar:
            out = (out * params["w_layer_scalar"]).to(out.dtype)
        return out

    def _forward(self, x, meta: ChunkMeta, params: Dict[str, torch.Tensor], slot, ctx: LayerContext):
        c = self.cfg
        x = slot.put("x_inp", x)
        h1, r1 = ops.rmsnorm_fwd(x, params["w_attn_norm"], c.norm_eps)
        slot.put("attn_norm_rstd", r1)
        if c.post_norms:
            a = slot.put("attn_branch", self._mixer_fwd(h1, None, meta, params, slot, ctx))
            an, ra = ops.rmsnorm_fwd(a, params["w_post_attn_norm"], c.norm_eps)
            slot.put("post_attn_rstd", ra)
            xo = x + an
        else:
            xo = self._mixer_fwd(h1, x, meta, params, slot, ctx)
        xo = slot.put("xo", xo)
        h2, r2 = ops.rmsnorm_fwd(xo, params["w_ffn_norm"], c.norm_eps)
        slot.put("ffn_norm_rstd", r2)
        if c.post_norms:
            f = slot.put("ffn_branch", self._ffn_fwd(h2, None, params, slot, ctx))
            fn, rf = ops.rmsnorm_fwd(f, params["w_post_ffn_norm"], c.norm_eps)
            slot.put("post_ffn_rstd", rf)
            return xo + fn
        return self._ffn_fwd(h2, xo, params, slot, ctx)

    # ------------------------------------------------------------------- recompute
    def forward_recompute(self, meta: ChunkMeta, params, slot, ctx: LayerContext) -> None:
        """Re-materialise every field above the slot's save level from the tier-0 fields."""
        c = self.cfg
        t = slot._t
        x = slot.get("x_inp")
        need_xo = not slot.has("xo")
        if self.attn is not None:
            need_out = not slot.has("attn_result")
            need_q = not slot.has("xq")
            if need_out or need_q or need_xo:
                h1 = None
                if need_q or (c.attn.gated and not slot.has("xgate")):
                    h1, _ = ops.rmsnorm_fwd(x, params["w_attn_norm"], c.norm_eps)
                self.attn.recompute(h1, meta, params, slot, ctx, need_out=need_out)
            if need_xo:
                attn_in = t["attn_result"]
                if c.attn.gated:
                    attn_in = (attn_in.to(torch.float32) * torch.sigmoid(t["xgate"].to(torch.float32))).to(attn_in.dtype)
                if c.post_norms:
                    a = self.attn.o.fwd(attn_in, params)
                    t["attn_branch"] = a
                    an, _ = ops.rmsnorm_fwd(a, params["w_post_attn_norm"], c.norm_eps)
                    t["xo"] = x + an
                else:
                    t["xo"] = self.attn.o.fwd(attn_in, params, residual=x)
        elif need_xo:
            h1, _ = ops.rmsnorm_fwd(x, params["w_attn_norm"], c.norm_eps)
            sub = LayerContext(**{**ctx.__dict__, "lin_attn_recompute_only": True, "out": {}})
            if c.post_norms:
                a = self.gdn.fwd(h1, None, meta, params, slot, sub)
                t["attn_branch"] = a
                an, _ = ops.rmsnorm_fwd(a, params["w_post_attn_norm"], c.norm_eps)
                t["xo"] = x + an
            else:
                t["xo"] = self.gdn.fwd(h1, x, meta, params, slot, sub)
        ffn = self.ffn or self.moe
        need_ffn = (not slot.has("x13")) if self.ffn is not None else \
            (not slot.has("x_up") or (self.moe.shared is not None and not slot.has("x13_shared")))
        if need_ffn or (c.post_norms and not slot.has("ffn_branch")):
            h2, _ = ops.rmsnorm_fwd(t["xo"], params["w_ffn_norm"], c.norm_eps)
            ffn.recompute(h2, params, slot)
            if c.post_norms and not slot.has("ffn_branch"):
                sc = _Passthrough(slot)
                t["ffn_branch"] = self._ffn_fwd(h2, None, params, sc, ctx)

    # -------------------------------------------------------------------- backward
    def backward(self, dx, meta: ChunkMeta, params, grads, slot, ctx: LayerContext):
        c = self.cfg
        t = slot._t
        x, xo = t["x_inp"], t["xo"]
        if c.layer_scalar:
            dx = (dx * params["w_layer_scalar"]).to(dx.dtype)
        # ---- FFN half
        d_branch = dx
        if c.post_norms:
            d_branch, _ = ops.rmsnorm_bwd(dx, t["ffn_branch"], params["w_post_ffn_norm"], t["post_ffn_rstd"],
                                          dw_out=grads.get("g_post_ffn_norm"))
        if self.ffn is not None:
            dh2, dx13 = self.ffn.bwd(d_branch, params, grads, slot)
            dxo, h2 = ops.rmsnorm_bwd(dh2, xo, params["w_ffn_norm"], t["ffn_norm_rstd"], dx_add=dx, emit_y=True,
                                      dw_out=grads.get("g_ffn_norm"))
            self.ffn.up.wgrad(dx13, h2, params, grads)
        else:
            h2, _ = ops.rmsnorm_fwd(xo, params["w_ffn_norm"], c.norm_eps)
            dh2 = self.moe.bwd(d_branch, h2, params, grads, slot, ctx)
            dxo, _ = ops.rmsnorm_bwd(dh2, xo, params["w_ffn_norm"], t["ffn_norm_rstd"], dx_add=dx,
                                     dw_out=grads.get("g_ffn_norm"))
        # ---- mixer half
        d_branch = dxo
        if c.post_norms:
            d_branch, _ = ops.rmsnorm_bwd(dxo, t["attn_branch"], params["w_post_attn_norm"], t["post_attn_rstd"],
                                          dw_out=grads.get("g_post_attn_norm"))
        if self.attn is not None:
            cache = {}

            def h_fn():
                if "h" not in cache:
                    cache["h"], _ = ops.rmsnorm_fwd(x, params["w_attn_norm"], c.norm_eps)
                return cache["h"]

            dh1, dqkv = self.attn.bwd(d_branch, h_fn, meta, params, grads, slot, ctx)
            dx_in, h1 = ops.rmsnorm_bwd(dh1, x, params["w_attn_norm"], t["attn_norm_rstd"], dx_add=dxo, emit_y=True,
                                        dw_out=grads.get("g_attn_norm"))
            self.attn.qkv.wgrad(dqkv, h1, params, grads)
        else:
            h1, _ = ops.rmsnorm_fwd(x, params["w_attn_norm"], c.norm_eps)
            dh1 = self.gdn.bwd(d_branch, h1, meta, params, grads, slot, ctx)
            dx_in, _ = ops.rmsnorm_bwd(dh1, x, params["w_attn_norm"], t["attn_norm_rstd"], dx_add=dxo,
                                       dw_out=grads.get("g_attn_norm"))
        return dx_in

    def end_of_step(self, params) -> None:
        clear_effective_weights(params)

    def bind_tp(self, tp) -> None:
        """Route the projections through the tensor-parallel handle (fused all-gather→GEMM / GEMM→reduce-scatter)."""
        if tp is None:
            return
        if self.attn is None or self.ffn is None:
            raise NotImplementedError("tensor parallelism covers dense attention + gated-FFN layers")
        for g in (self.attn.qkv, self.attn.o, self.ffn.up, self.ffn.down):
            g.tp = tp

    # ------------------------------------------------------------------------ cost
    def compute_cost(self, num_tokens: int, avg_ctx: float) -> ComputeCost:
        T = num_tokens
        if self.attn is not None:
            proj, core, oproj = self.attn.flops(T, avg_ctx)
        else:
            proj, core, oproj = self.gdn.flops(T)
        if self.ffn is not None:
            up, down = self.ffn.flops(T)
        else:
            router, routed, shared = self.moe.flops(T)
            up, down = router + (routed + shared) * 2 / 3, (routed + shared) / 3
        total = proj + core + oproj + up + down
        if self.attn is not None:
            avoided = (0.0, core, core + proj + oproj, core + proj + oproj + up)
        else:   # linear attention keeps only boundary states; xo (tier 2) avoids the whole mixer
            avoided = (0.0, 0.0, proj + core + oproj, proj + core + oproj + up)
        return ComputeCost(total, avoided, attn_fwd_flops=core if self.attn is not None else 0.0)


class _Passthrough:
    """Slot wrapper used when a block forward is re-run only for its output: nothing is stored."""

    def __init__(self, slot):
        self.s = slot
        self._t = dict(slot._t)
        self.buffer = None
        self.schema, self.num_tokens = slot.schema, slot.num_tokens

    def put(self, name, value):
        self._t[name] = value
        return value

    def out(self, name, device):
        f = self.schema.by_name(name)
        tt = torch.empty(f.shape_fn(self.num_tokens), dtype=f.dtype, device=device)
        self._t[name] = tt
        return tt

    def get(self, name):
        return self._t[name]

    def has(self, name):
        return name in self._t
