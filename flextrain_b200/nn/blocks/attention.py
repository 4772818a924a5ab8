"""Grouped-query attention block with hand-written forward / recompute / backward.

One class covers what the reference splits across ``nn/blocks/attention.py`` (GQA, QK-norm per
head or per row, QKV bias, logit soft-cap, sliding window), ``attention_gated.py`` (doubled
``w_q`` = query ‖ gate with ``sigmoid(gate)`` on the attention output, partial rotary, MRoPE) and
the Gemma scale override.  Save tiers follow flextrain/nn/blocks/attention.py:236-294:
``xk, xv`` tier 0; ``attn_result, softmax_lse`` tier 1; ``xq`` (and the gate) tier 2.

Long sequences: a chunk whose sequence started in an earlier chunk appends its K/V to the rolling
window and attends over ``window[:prior+len]``; in backward the dK/dV of earlier chunks' keys are
accumulated in the window and each chunk collects (then clears) its own slice
(flextrain/nn/blocks/attention.py:463-487, 636-696).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional, Tuple

import torch

from ... import ops
from ...core.activation_schema import ActivationField
from ...core.layer import ChunkMeta, LayerContext, TensorSpec
from .linear import LinearGroup, LoRAConfig
from .rope import RopeConfig


@dataclass
class AttentionConfig:
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    rope: RopeConfig = field(default_factory=RopeConfig)
    qkv_bias: bool = False
    qk_norm: Optional[str] = None            # None | "head" (Qwen3, Gemma3) | "row" (OLMoE)
    norm_eps: float = 1e-6
    softcap: float = 0.0
    window: int = 0                          # sliding window (0 = full causal)
    scale: Optional[float] = None            # default head_dim ** -0.5
    gated: bool = False                      # Qwen3-Next / Qwen3.5 output gate
    causal: bool = True
    v_norm: bool = False                     # Gemma 4: per-head RMSNorm of V without a learned scale

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim


class GQAAttentionBlock:
    def __init__(self, cfg: AttentionConfig, *, dtype=torch.bfloat16, norm_dtype=torch.float32,
                 lora: Optional[LoRAConfig] = None, prefix: str = ""):
        self.cfg = cfg
        self.dtype = dtype
        self.norm_dtype = norm_dtype
        self.scale = cfg.scale if cfg.scale is not None else cfg.head_dim ** -0.5
        bias = ["b_q", "b_k", "b_v"] if cfg.qkv_bias else []
        self.qkv = LinearGroup(["w_q", "w_k", "w_v"], lora, bias)
        self.o = LinearGroup(["w_o"], lora)
        self.qkv.tp_mode, self.o.tp_mode = "col", "row"      # used only when a tensor-parallel handle is bound
        self.inv_freq_cache: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ declarations
    def tensor_specs(self):
        c, dt = self.cfg, self.dtype
        qrows = c.q_dim * (2 if c.gated else 1)
        specs = [TensorSpec("w_q", (qrows, c.d_model), dt), TensorSpec("w_k", (c.kv_dim, c.d_model), dt),
                 TensorSpec("w_v", (c.kv_dim, c.d_model), dt), TensorSpec("w_o", (c.d_model, c.q_dim), dt)]
        if c.qkv_bias:
            specs += [TensorSpec("b_q", (qrows,), dt, init="zeros"), TensorSpec("b_k", (c.kv_dim,), dt, init="zeros"),
                      TensorSpec("b_v", (c.kv_dim,), dt, init="zeros")]
        if c.qk_norm == "head":
            specs += [TensorSpec("w_q_norm", (c.head_dim,), self.norm_dtype, init="ones"),
                      TensorSpec("w_k_norm", (c.head_dim,), self.norm_dtype, init="ones")]
        elif c.qk_norm == "row":
            specs += [TensorSpec("w_q_norm", (c.q_dim,), self.norm_dtype, init="ones"),
                      TensorSpec("w_k_norm", (c.kv_dim,), self.norm_dtype, init="ones")]
        return specs

    def activation_fields(self):
        c, dt = self.cfg, self.dtype
        f = [ActivationField("xk", lambda t: (t, c.n_kv_heads, c.head_dim), dt, 0),
             ActivationField("xv", lambda t: (t, c.n_kv_heads, c.head_dim), dt, 0),
             ActivationField("attn_result", lambda t: (t, c.q_dim), dt, 1),
             ActivationField("softmax_lse", lambda t: (c.n_heads, t), torch.float32, 1),
             ActivationField("xq", lambda t: (t, c.n_heads, c.head_dim), dt, 2)]
        if c.gated:
            f.append(ActivationField("xgate", lambda t: (t, c.q_dim), dt, 2))
        if c.qk_norm == "head":
            f += [ActivationField("q_rstd", lambda t: (t, c.n_heads), torch.float32, 0),
                  ActivationField("k_rstd", lambda t: (t, c.n_kv_heads), torch.float32, 0)]
        elif c.qk_norm == "row":
            f += [ActivationField("q_rstd", lambda t: (t,), torch.float32, 0),
                  ActivationField("k_rstd", lambda t: (t,), torch.float32, 0)]
        if c.v_norm:
            f.append(ActivationField("v_rstd", lambda t: (t, c.n_kv_heads), torch.float32, 0))
        return f

    # --------------------------------------------------------------------- helpers
    def _inv_freq(self, device) -> torch.Tensor:
        key = str(device)
        if key not in self.inv_freq_cache:
            self.inv_freq_cache[key] = self.cfg.rope.inv_freq(self.cfg.head_dim).to(device)
        return self.inv_freq_cache[key]

    def _unit_gain(self, device) -> torch.Tensor:
        """The all-ones gain of the scale-free V norm (the norm kernels take a gain operand)."""
        key = "ones:" + str(device)
        if key not in self.inv_freq_cache:
            self.inv_freq_cache[key] = torch.ones(self.cfg.head_dim, dtype=self.norm_dtype, device=device)
        return self.inv_freq_cache[key]

    def _project_qkv(self, h, params, qkv=None):
        """QKV projection (one GEMM) -> pre-norm, pre-RoPE ``(q, gate, k, v)`` views of one buffer.  ``qkv`` may carry
        a projection that was already computed (without bias) by a fused gather-GEMM."""
        c = self.cfg
        if qkv is None:
            qkv = self.qkv.fwd(h, params)
        elif self.qkv.bias_names:
            qkv += self.qkv.bias(params).to(qkv.dtype)
        T = qkv.shape[0]                 # all tokens of the chunk (h holds T/tp of them under tensor parallelism)
        if c.gated:
            # w_q rows are per-head [query(hd) ‖ gate(hd)] (HF Qwen3-Next layout)
            qg = qkv[:, : 2 * c.q_dim].reshape(T, c.n_heads, 2 * c.head_dim)
            q = qg[:, :, : c.head_dim]
            gate = qg[:, :, c.head_dim:].reshape(T, c.q_dim)
            off = 2 * c.q_dim
        else:
            q = qkv[:, : c.q_dim].unflatten(1, (c.n_heads, c.head_dim))
            gate, off = None, c.q_dim
        k = qkv[:, off: off + c.kv_dim].unflatten(1, (c.n_kv_heads, c.head_dim))
        v = qkv[:, off + c.kv_dim: off + 2 * c.kv_dim].unflatten(1, (c.n_kv_heads, c.head_dim))
        return q, gate, k, v

    def _qk_norm_fwd(self, q, k, params):
        c = self.cfg
        if c.qk_norm == "head":
            qn, qr = ops.rmsnorm_fwd(q.contiguous(), params["w_q_norm"], c.norm_eps)
            kn, kr = ops.rmsnorm_fwd(k.contiguous(), params["w_k_norm"], c.norm_eps)
        else:
            T = q.shape[0]
            qn, qr = ops.rmsnorm_fwd(q.reshape(T, -1).contiguous(), params["w_q_norm"], c.norm_eps)
            kn, kr = ops.rmsnorm_fwd(k.reshape(T, -1).contiguous(), params["w_k_norm"], c.norm_eps)
            qn, kn = qn.view(T, c.n_heads, c.head_dim), kn.view(T, c.n_kv_heads, c.head_dim)
        return qn, qr, kn, kr

    def _qkv_post(self, h, meta: ChunkMeta, params, slot, *, want_q=True, qkv=None):
        """Compute post-norm, post-RoPE q / k / v (+gate) from the normed input and store them in the slot."""
        c = self.cfg
        q, gate, k, v = self._project_qkv(h, params, qkv)
        if c.qk_norm:
            q, qr, k, kr = self._qk_norm_fwd(q, k, params)
            slot.put("q_rstd", qr)
            slot.put("k_rstd", kr)
        inv = self._inv_freq(h.device)
        pos, sec = meta.positions, c.rope.mrope_sections
        xk = ops.rope(k, pos, inv, out=slot.out("xk", h.device), mrope_sections=sec)
        xv = slot.out("xv", h.device)
        if c.v_norm:
            vn, vr = ops.rmsnorm_fwd(v.contiguous(), self._unit_gain(h.device), c.norm_eps)
            slot.put("v_rstd", vr)
            xv.copy_(vn)
        else:
            xv.copy_(v)
        xq = None
        if want_q:
            xq = ops.rope(q, pos, inv, out=slot.out("xq", h.device), mrope_sections=sec)
            if c.gated:
                slot.put("xgate", gate.contiguous() if slot.buffer is None else gate)
        return xq, xk, xv

    def _kv_for_attention(self, meta: ChunkMeta, xk, xv, ctx: LayerContext, *, write: bool):
        """K/V seen by this chunk's queries: its own, or the rolling window when prior chunks exist."""
        if not (meta.has_prior or any(meta.has_more_chunks)):
            return xk, xv
        if len(meta.seq_lens) != 1:
            raise ValueError("a chunk with prior context must hold exactly one sequence")
        P, L = meta.prior_lens[0], meta.seq_lens[0]
        w = ctx.kv_window
        if write:
            w.k[P:P + L].copy_(xk)
            w.v[P:P + L].copy_(xv)
        return w.k[:P + L], w.v[:P + L]

    def _attend(self, xq, K, V, meta):
        c = self.cfg
        return ops.attention_fwd(xq, K, V, meta.cu_seqlens_q, meta.cu_seqlens_k, meta.max_seqlen_q, meta.max_seqlen_k,
                                 scale=self.scale, causal=c.causal, window=c.window, softcap=c.softcap)

    # --------------------------------------------------------------------- forward
    def fwd(self, h, x_resid, meta: ChunkMeta, params, slot, ctx: LayerContext, qkv=None) -> torch.Tensor:
        """``h`` = normed input, ``x_resid`` = residual stream. Returns ``x_resid + attn(h) @ w_o.T``."""
        c = self.cfg
        xq, xk, xv = self._qkv_post(h, meta, params, slot, qkv=qkv)
        K, V = self._kv_for_attention(meta, xk, xv, ctx, write=True)
        out, lse = self._attend(xq, K, V, meta)
        out2 = out.reshape(out.shape[0], c.q_dim)
        if c.gated:
            g = slot.get("xgate")
            raw = slot.put("attn_result", out2)
            out2 = (raw.to(torch.float32) * torch.sigmoid(g.to(torch.float32))).to(raw.dtype)
        else:
            out2 = slot.put("attn_result", out2)
        slot.put("softmax_lse", lse)
        return self.o.fwd(out2, params, residual=x_resid)

    # ------------------------------------------------------------------- recompute
    def recompute(self, h, meta: ChunkMeta, params, slot, ctx: LayerContext, *, need_out: bool) -> None:
        """Re-materialise ``xq`` (tier 2) and, if asked, ``attn_result`` / ``softmax_lse`` (tier 1)."""
        if not slot.has("xq") or (self.cfg.gated and not slot.has("xgate")):
            tmp = _ScratchSlot(slot)
            self._qkv_post(h, meta, params, tmp)
            slot._t["xq"] = tmp._t["xq"]
            if self.cfg.gated:
                slot._t["xgate"] = tmp._t["xgate"]
        if need_out and not slot.has("attn_result"):
            K, V = self._kv_for_attention(meta, slot._t["xk"], slot._t["xv"], ctx, write=False)
            out, lse = self._attend(slot._t["xq"], K, V, meta)
            slot._t["attn_result"] = out.reshape(out.shape[0], self.cfg.q_dim)
            slot._t["softmax_lse"] = lse

    # -------------------------------------------------------------------- backward
    def bwd(self, dxo, h_fn, meta: ChunkMeta, params, grads, slot, ctx: LayerContext):
        """Backward from ``dxo`` (grad of the block output). Returns ``(dh, dqkv, wgrad_closure_inputs)``.

        ``h_fn()`` lazily provides the normed input (needed only for the QK-norm pre-activation
        recompute).  The caller owns the residual path and the deferred QKV weight gradient:
        it calls ``self.qkv.wgrad(dqkv, h, ...)`` once the norm backward has re-emitted ``h``.
        """
        c = self.cfg
        t = slot._t
        attn_raw = t["attn_result"]
        T = attn_raw.shape[0]
        if c.gated:
            sg = torch.sigmoid(t["xgate"].to(torch.float32))
            attn_in = (attn_raw.to(torch.float32) * sg).to(attn_raw.dtype)
        else:
            attn_in = attn_raw
        dattn = self.o.dgrad(dxo, params)                                        # (T, q_dim)
        self.o.wgrad(dxo, attn_in, params, grads)
        dgate = None
        if c.gated:
            df = dattn.to(torch.float32)
            dgate = (df * attn_raw.to(torch.float32) * sg * (1 - sg)).to(dattn.dtype)
            dattn = (df * sg).to(dattn.dtype)
        K, V = self._kv_for_attention(meta, t["xk"], t["xv"], ctx, write=False)
        dq, dk, dv = ops.attention_bwd(dattn.view(T, c.n_heads, c.head_dim), t["xq"], K, V,
                                       attn_raw.view(T, c.n_heads, c.head_dim), t["softmax_lse"], meta.cu_seqlens_q,
                                       meta.cu_seqlens_k, meta.max_seqlen_q, meta.max_seqlen_k, scale=self.scale,
                                       causal=c.causal, window=c.window, softcap=c.softcap)
        if meta.has_prior or (ctx.kv_window is not None and ctx.kv_window.dk is not None and any(meta.has_more_chunks)):
            dk, dv = self._cross_chunk_dkv(dk, dv, meta, ctx)
        # inverse RoPE, then QK-norm backward, assembling dqkv in projection-row order
        inv = self._inv_freq(dxo.device)
        pos, sec = meta.positions, c.rope.mrope_sections
        qrows = c.q_dim * (2 if c.gated else 1)
        dqkv = torch.empty(T, qrows + 2 * c.kv_dim, dtype=dxo.dtype, device=dxo.device)
        if c.gated:
            qg = dqkv[:, :qrows].view(T, c.n_heads, 2 * c.head_dim)
            dq_dst = qg[:, :, : c.head_dim]
            qg[:, :, c.head_dim:].copy_(dgate.view(T, c.n_heads, c.head_dim))
        else:
            dq_dst = dqkv[:, :qrows].unflatten(1, (c.n_heads, c.head_dim))
        dk_dst = dqkv[:, qrows: qrows + c.kv_dim].unflatten(1, (c.n_kv_heads, c.head_dim))
        dv_dst = dqkv[:, qrows + c.kv_dim:].unflatten(1, (c.n_kv_heads, c.head_dim))
        pre = self._project_qkv(h_fn(), params) if (c.qk_norm or c.v_norm) else None   # pre-norm recompute (one GEMM)
        if c.v_norm:
            dvp, _ = ops.rmsnorm_bwd(dv.contiguous(), pre[3].contiguous(), self._unit_gain(dxo.device), t["v_rstd"])
            dv_dst.copy_(dvp.view(T, c.n_kv_heads, c.head_dim))
        else:
            dv_dst.copy_(dv)
        if not c.qk_norm:
            if c.gated:
                dq_dst.copy_(ops.rope(dq.contiguous(), pos, inv, inverse=True, mrope_sections=sec))
            else:
                ops.rope(dq, pos, inv, out=dq_dst, inverse=True, mrope_sections=sec)
            ops.rope(dk, pos, inv, out=dk_dst, inverse=True, mrope_sections=sec)
        else:
            dqn = ops.rope(dq.contiguous(), pos, inv, inverse=True, mrope_sections=sec)
            dkn = ops.rope(dk.contiguous(), pos, inv, inverse=True, mrope_sections=sec)
            q_pre, _, k_pre, _ = pre
            if c.qk_norm == "head":
                dqp, _ = ops.rmsnorm_bwd(dqn, q_pre.contiguous(), params["w_q_norm"], t["q_rstd"],
                                         dw_out=grads.get("g_q_norm"))
                dkp, _ = ops.rmsnorm_bwd(dkn, k_pre.contiguous(), params["w_k_norm"], t["k_rstd"],
                                         dw_out=grads.get("g_k_norm"))
            else:
                dqp, _ = ops.rmsnorm_bwd(dqn.view(T, -1), q_pre.reshape(T, -1).contiguous(), params["w_q_norm"],
                                         t["q_rstd"], dw_out=grads.get("g_q_norm"))
                dkp, _ = ops.rmsnorm_bwd(dkn.view(T, -1), k_pre.reshape(T, -1).contiguous(), params["w_k_norm"],
                                         t["k_rstd"], dw_out=grads.get("g_k_norm"))
            dq_dst.copy_(dqp.view(T, c.n_heads, c.head_dim))
            dk_dst.copy_(dkp.view(T, c.n_kv_heads, c.head_dim))
        dh = self.qkv.dgrad(dqkv, params)
        return dh, dqkv

    def _cross_chunk_dkv(self, dk, dv, meta: ChunkMeta, ctx: LayerContext):
        """Fold this chunk's dK/dV for earlier keys into the window; return the totals for its own keys."""
        w = ctx.kv_window
        P, L = meta.prior_lens[0], meta.seq_lens[0]
        if P > 0:
            w.dk[:P] += dk[:P]
            w.dv[:P] += dv[:P]
        own_k, own_v = dk[P:P + L], dv[P:P + L]
        if meta.has_more_chunks[0]:
            own_k = own_k + w.dk[P:P + L]
            own_v = own_v + w.dv[P:P + L]
        w.dk[P:P + L].zero_()
        w.dv[P:P + L].zero_()
        return own_k.contiguous(), own_v.contiguous()

    # ------------------------------------------------------------------------ cost
    def flops(self, T: int, avg_ctx: float) -> Tuple[float, float, float]:
        """(qkv_proj, attention core, o_proj) forward FLOPs for ``T`` tokens at mean context ``avg_ctx``."""
        c = self.cfg
        qrows = c.q_dim * (2 if c.gated else 1)
        proj = 2.0 * T * c.d_model * (qrows + 2 * c.kv_dim)
        ctxlen = min(avg_ctx, c.window) if c.window else avg_ctx
        core = 4.0 * T * ctxlen * c.q_dim
        return proj, core, 2.0 * T * c.q_dim * c.d_model


class _ScratchSlot:
    """Slot stand-in whose outputs are fresh tensors (used while recomputing into a lower-level slot)."""

    def __init__(self, slot):
        self.schema, self.num_tokens, self.buffer, self._t = slot.schema, slot.num_tokens, None, {}

    def put(self, name, value):
        self._t[name] = value
        return value

    def out(self, name, device):
        f = self.schema.by_name(name)
        t = torch.empty(f.shape_fn(self.num_tokens), dtype=f.dtype, device=device)
        self._t[name] = t
        return t

    def get(self, name):
        return self._t[name]
