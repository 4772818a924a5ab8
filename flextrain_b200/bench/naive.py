"""Naive autograd PyTorch models used as the parity oracle (flextrain/bench/parity.py:142-385).

A plain ``nn.Module``-free functional decoder over the *same* parameter tensors the engine holds:
``naive_loss(am, seqs)`` runs every sequence on its own through ordinary PyTorch ops with autograd,
so the engine's hand-written backward, chunking, save tiers, rings and packing can all be checked
against ``torch.autograd`` + ``torch.optim.AdamW`` on CPU in fp32.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from ..ops import reference as ref


def clone_params(am, requires_grad: bool = True):
    """Deep copy of every master tensor as fp32 autograd leaves: ``{(scope, layer, name): tensor}``."""
    out = {}
    for scope, l, name, t in am.named_master_params():
        out[(scope, l, name)] = t.detach().to(torch.float32).clone().requires_grad_(requires_grad)
    return out


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, inv_freq, sections=None):
    rot = 2 * inv_freq.numel()
    ang = ref._rope_angles(pos, inv_freq, sections)
    cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
    x1, x2 = x[..., : rot // 2], x[..., rot // 2: rot]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin, x[..., rot:]], -1)


def _lin(P, l, name, x, lora_scale=None):
    w = P[("layer", l, name)]
    a = P.get(("layer", l, name + "_lora_a"))
    if a is not None:
        b = P[("layer", l, name + "_lora_b")]
        w = w + lora_scale * (b @ a)
    return x @ w.t()


def _attention(layer, l, P, h, pos):
    c = layer.attn.cfg
    T = h.shape[0]
    ls = layer.cfg.lora.scale if layer.cfg.lora is not None else None
    q, k, v = _lin(P, l, "w_q", h, ls), _lin(P, l, "w_k", h, ls), _lin(P, l, "w_v", h, ls)
    if c.qkv_bias:
        q, k, v = q + P[("layer", l, "b_q")], k + P[("layer", l, "b_k")], v + P[("layer", l, "b_v")]
    gate = None
    if c.gated:
        qg = q.view(T, c.n_heads, 2 * c.head_dim)
        q, gate = qg[..., : c.head_dim].reshape(T, -1), qg[..., c.head_dim:].reshape(T, -1)
    if c.qk_norm == "row":
        q = _rms(q, P[("layer", l, "w_q_norm")], c.norm_eps)
        k = _rms(k, P[("layer", l, "w_k_norm")], c.norm_eps)
    q, k, v = q.view(T, c.n_heads, c.head_dim), k.view(T, c.n_kv_heads, c.head_dim), v.view(T, c.n_kv_heads, c.head_dim)
    if c.qk_norm == "head":
        q = _rms(q, P[("layer", l, "w_q_norm")], c.norm_eps)
        k = _rms(k, P[("layer", l, "w_k_norm")], c.norm_eps)
    if c.v_norm:
        v = _rms(v, torch.ones(c.head_dim, dtype=v.dtype), c.norm_eps)
    inv = c.rope.inv_freq(c.head_dim)
    q, k = _rope(q, pos, inv, c.rope.mrope_sections), _rope(k, pos, inv, c.rope.mrope_sections)
    rep = c.n_heads // c.n_kv_heads
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    sc = torch.einsum("qhd,khd->hqk", q, kk) * layer.attn.scale
    if c.softcap:
        sc = c.softcap * torch.tanh(sc / c.softcap)
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    mask = j <= i
    if c.window:
        mask = mask & (j > i - c.window)
    sc = sc.masked_fill(~mask, float("-inf"))
    o = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), vv).reshape(T, -1)
    if gate is not None:
        o = o * torch.sigmoid(gate)
    return _lin(P, l, "w_o", o, ls)


def _gdn(layer, l, P, h):
    from ..core.layer import ChunkMeta
    T = h.shape[0]
    meta = ChunkMeta.build(0, [0], [T], [0], [False], h.device)
    p = {n: P[("layer", l, n)] for n in layer.gdn.PARAMS}
    out, _, _ = layer.gdn._core(h, None, meta, p, None, None)
    return out


def _ffn(layer, l, P, h, aux=None):
    ls = layer.cfg.lora.scale if layer.cfg.lora is not None else None
    if layer.ffn is not None:
        g, u = _lin(P, l, "w_1", h, ls), _lin(P, l, "w_3", h, ls)
        act = F.silu(g) if layer.ffn.cfg.kind == "swiglu" else F.gelu(g, approximate="tanh")
        return _lin(P, l, "w_2", act * u, ls)
    c = layer.moe.cfg
    logits = h @ P[("layer", l, "w_router")].t()
    if c.routing == "softmax_then_topk":
        probs = torch.softmax(logits, -1)
        w, idx = torch.sort(probs, dim=-1, descending=True, stable=True)
        w, idx = w[:, : c.top_k], idx[:, : c.top_k]
    else:
        vals, idx = torch.sort(logits, dim=-1, descending=True, stable=True)
        w, idx = torch.softmax(vals[:, : c.top_k], -1), idx[:, : c.top_k]
    if aux is not None and c.aux_loss_alpha > 0:
        # load-balance term of this layer over these tokens: alpha * E * sum_e f_e * sum_t p_te, with the routed
        # fraction f_e a constant; the caller divides by the step's token count
        E = logits.shape[-1]
        f = torch.bincount(idx.reshape(-1), minlength=E).to(logits.dtype) / idx.numel()
        aux.append(c.aux_loss_alpha * E * (f.detach() * torch.softmax(logits, -1).sum(0)).sum())
    up, down = P[("layer", l, "w_up")], P[("layer", l, "w_down")]
    if ls is not None and ("layer", l, "w_up_lora_a") in P:        # per-expert adapters: W'[e] = W[e] + s B[e] A[e]
        up = up + ls * torch.bmm(P[("layer", l, "w_up_lora_b")], P[("layer", l, "w_up_lora_a")])
        down = down + ls * torch.bmm(P[("layer", l, "w_down_lora_b")], P[("layer", l, "w_down_lora_a")])
    out = torch.zeros_like(h)
    for k in range(c.top_k):
        e = idx[:, k]
        uw = up[e]                                  # (T, 2F, d)
        x = torch.einsum("tfd,td->tf", uw, h)
        F_ = c.expert_dim
        val, gate = x[:, :F_], x[:, F_:]
        act = (F.silu(gate) if c.kind == "swiglu" else F.gelu(gate, approximate="tanh")) * val
        out = out + w[:, k: k + 1] * torch.einsum("tdf,tf->td", down[e], act)
    if c.shared_dim > 0:
        g, u = h @ P[("layer", l, "w_shared_1")].t(), h @ P[("layer", l, "w_shared_3")].t()
        ys = (F.silu(g) * u) @ P[("layer", l, "w_shared_2")].t()
        if c.shared_gate:
            ys = ys * torch.sigmoid(h @ P[("layer", l, "w_shared_gate")].t())
        out = out + ys
    return out


def naive_forward(am, P, tokens: torch.Tensor, positions: Optional[torch.Tensor] = None, aux=None) -> torch.Tensor:
    """Logits ``(T, V)`` of one sequence through plain autograd ops; ``aux`` (a list) collects the MoE layers'
    un-normalised load-balance terms."""
    T = tokens.numel()
    pos = positions if positions is not None else torch.arange(T)
    x = P[("embed", -1, "w_tok_embeddings")][tokens.long()] * am.embed.scale
    for l, layer in enumerate(am.layers):
        c = layer.cfg
        h = _rms(x, P[("layer", l, "w_attn_norm")], c.norm_eps)
        a = _attention(layer, l, P, h, pos) if layer.attn is not None else _gdn(layer, l, P, h)
        if c.post_norms:
            a = _rms(a, P[("layer", l, "w_post_attn_norm")], c.norm_eps)
        x = x + a
        h = _rms(x, P[("layer", l, "w_ffn_norm")], c.norm_eps)
        f = _ffn(layer, l, P, h, aux)
        if c.post_norms:
            f = _rms(f, P[("layer", l, "w_post_ffn_norm")], c.norm_eps)
        x = x + f
        if c.layer_scalar:
            x = x * P[("layer", l, "w_layer_scalar")]
    h = _rms(x, P[("head", -1, "w_final_norm")], am.head.norm_eps)
    z = h @ P[("head", -1, "w_head_proj")].t()
    if am.head.final_softcap:
        z = am.head.final_softcap * torch.tanh(z / am.head.final_softcap)
    return z


def naive_loss(am, P, seqs) -> torch.Tensor:
    """Mean cross-entropy over the active tokens of ``seqs`` (each sequence run on its own)."""
    total, active = 0.0, 0
    for s in seqs:
        z = naive_forward(am, P, s.tokens)
        tgt = s.targets.clone()
        if s.loss_mask is not None:
            tgt[s.loss_mask <= 0] = -100
        total = total + F.cross_entropy(z, tgt, ignore_index=-100, reduction="sum")
        active += int((tgt != -100).sum())
    return total / max(active, 1)
