"""Shared checkpoint-name map builders for the decoder families."""
from __future__ import annotations

from typing import List

import torch

from ..hf_weights import WeightMapEntry as E


def embed_entries(mc, prefix="model.") -> List[E]:
    return [E("w_tok_embeddings", [f"{prefix}embed_tokens.weight"],
              alternates=[[f"model.language_model.embed_tokens.weight"], [f"language_model.model.embed_tokens.weight"]])]


def head_entries(mc, prefix="model.") -> List[E]:
    return [E("w_final_norm", [f"{prefix}norm.weight"], plus_one=mc.norm_plus_one,
              alternates=[["model.language_model.norm.weight"], ["language_model.model.norm.weight"]]),
            E("w_head_proj", ["lm_head.weight"], alternates=[["language_model.lm_head.weight"]])]


def _alts(i: int, tail: str):
    return [[f"model.language_model.layers.{i}.{tail}"], [f"language_model.model.layers.{i}.{tail}"]]


def attn_entries(i: int, mc, *, bias=False, qk_norm=False, prefix="model.") -> List[E]:
    p = f"{prefix}layers.{i}.self_attn."
    out = []
    for ours, theirs in (("w_q", "q_proj"), ("w_k", "k_proj"), ("w_v", "v_proj"), ("w_o", "o_proj")):
        out.append(E(ours, [f"{p}{theirs}.weight"], alternates=_alts(i, f"self_attn.{theirs}.weight")))
        if bias and ours != "w_o":
            out.append(E("b_" + ours[2:], [f"{p}{theirs}.bias"], alternates=_alts(i, f"self_attn.{theirs}.bias")))
    if qk_norm:
        out.append(E("w_q_norm", [f"{p}q_norm.weight"], plus_one=mc.norm_plus_one,
                     alternates=_alts(i, "self_attn.q_norm.weight")))
        out.append(E("w_k_norm", [f"{p}k_norm.weight"], plus_one=mc.norm_plus_one,
                     alternates=_alts(i, "self_attn.k_norm.weight")))
    return out


def norm_entries(i: int, mc, *, sandwich=False, prefix="model.") -> List[E]:
    p = f"{prefix}layers.{i}."
    po = mc.norm_plus_one
    if sandwich:   # Gemma 2/3: four norms per layer
        names = (("w_attn_norm", "input_layernorm"), ("w_post_attn_norm", "post_attention_layernorm"),
                 ("w_ffn_norm", "pre_feedforward_layernorm"), ("w_post_ffn_norm", "post_feedforward_layernorm"))
    else:
        names = (("w_attn_norm", "input_layernorm"), ("w_ffn_norm", "post_attention_layernorm"))
    return [E(o, [f"{p}{t}.weight"], plus_one=po, alternates=_alts(i, f"{t}.weight")) for o, t in names]


def dense_ffn_entries(i: int, mc, prefix="model.") -> List[E]:
    p = f"{prefix}layers.{i}.mlp."
    return [E(o, [f"{p}{t}.weight"], alternates=_alts(i, f"mlp.{t}.weight"))
            for o, t in (("w_1", "gate_proj"), ("w_3", "up_proj"), ("w_2", "down_proj"))]


def moe_entries(i: int, mc, *, prefix="model.", router="mlp.gate", experts="mlp.experts",
                shared="mlp.shared_expert", shared_gate="mlp.shared_expert_gate") -> List[E]:
    p = f"{prefix}layers.{i}."
    n, F = mc.num_experts, mc.expert_dim
    up_names, down_names = [], []
    for e in range(n):
        up_names += [f"{p}{experts}.{e}.up_proj.weight", f"{p}{experts}.{e}.gate_proj.weight"]
        down_names.append(f"{p}{experts}.{e}.down_proj.weight")

    def comb_up(ts):       # (E, 2F, d) with the 2F axis [up ‖ gate]
        if len(ts) == 1:   # stacked checkpoint (transformers >= 5 writes experts.gate_up_proj as [gate ‖ up])
            return torch.cat([ts[0][:, F:], ts[0][:, :F]], 1)
        return torch.stack([torch.cat([ts[2 * e], ts[2 * e + 1]], 0) for e in range(n)], 0)

    def split_up(t):
        out = []
        for e in range(n):
            out += [t[e, :F], t[e, F:]]
        return out

    out = [E("w_router", [f"{p}{router}.weight"]),
           E("w_up", up_names, combine=comb_up, split=split_up, alternates=[[f"{p}{experts}.gate_up_proj"]]),
           E("w_down", down_names, combine=lambda ts: ts[0] if len(ts) == 1 else torch.stack(ts, 0),
             split=lambda t: list(t.unbind(0)), alternates=[[f"{p}{experts}.down_proj"]])]
    if mc.shared_dim > 0:
        out += [E("w_shared_1", [f"{p}{shared}.gate_proj.weight"]), E("w_shared_3", [f"{p}{shared}.up_proj.weight"]),
                E("w_shared_2", [f"{p}{shared}.down_proj.weight"])]
        if mc.shared_gate:
            out.append(E("w_shared_gate", [f"{p}{shared_gate}.weight"]))
    return out


def gdn_entries(i: int, mc, prefix="model.") -> List[E]:
    """Gated DeltaNet: HF ``in_proj_qkvz`` / ``in_proj_ba`` are stored per key-head group
    ``[q(hk) k(hk) v(r*hv) z(r*hv)]`` (r = value heads per key head); the engine uses flat ``[Q‖K‖V‖Z]`` and
    ``[B‖A]`` (flextrain/nn/blocks/linear_attn.py:448-535)."""
    p = f"{prefix}layers.{i}.linear_attn."
    g = mc.gdn
    r = g.n_v_heads // g.n_k_heads
    hk, hv = g.head_k_dim, g.head_v_dim
    grp = 2 * hk + 2 * r * hv

    def perm_qkvz():
        q, k, v, z = [], [], [], []
        for h in range(g.n_k_heads):
            b = h * grp
            q += range(b, b + hk); k += range(b + hk, b + 2 * hk)
            v += range(b + 2 * hk, b + 2 * hk + r * hv); z += range(b + 2 * hk + r * hv, b + grp)
        return torch.tensor(q + k + v + z, dtype=torch.long)

    def perm_ba():
        bb, aa = [], []
        for h in range(g.n_k_heads):
            b = h * 2 * r
            bb += range(b, b + r); aa += range(b + r, b + 2 * r)
        return torch.tensor(bb + aa, dtype=torch.long)

    pq, pb = perm_qkvz(), perm_ba()
    iq, ib = torch.argsort(pq), torch.argsort(pb)
    # Qwen3-Next bundles the projections per key-head group; Qwen3.5 stores them separately and already flat.  Either
    # form loads; export writes the family's own.
    bundled_qkvz, bundled_ba = [f"{p}in_proj_qkvz.weight"], [f"{p}in_proj_ba.weight"]
    flat_qkvz, flat_ba = [f"{p}in_proj_qkv.weight", f"{p}in_proj_z.weight"], [f"{p}in_proj_b.weight", f"{p}in_proj_a.weight"]
    n_qkv, n_b = 2 * g.n_k_heads * hk + g.n_v_heads * hv, g.n_v_heads
    flat = mc.arch in ("qwen3_5", "qwen3_5_moe")
    return [
        E("w_lin_qkvz", flat_qkvz if flat else bundled_qkvz,
          combine=lambda ts: torch.cat(ts, 0) if len(ts) == 2 else ts[0][pq],
          split=(lambda t: [t[:n_qkv], t[n_qkv:]]) if flat else (lambda t: [t[iq]]),
          alternates=[bundled_qkvz if flat else flat_qkvz]),
        E("w_lin_ba", flat_ba if flat else bundled_ba,
          combine=lambda ts: torch.cat(ts, 0) if len(ts) == 2 else ts[0][pb],
          split=(lambda t: [t[:n_b], t[n_b:]]) if flat else (lambda t: [t[ib]]),
          alternates=[bundled_ba if flat else flat_ba]),
        E("w_lin_conv", [f"{p}conv1d.weight"], combine=lambda ts: ts[0].reshape(ts[0].shape[0], -1),
          split=lambda t: [t.unsqueeze(1)]),
        E("w_lin_dt_bias", [f"{p}dt_bias"]), E("w_lin_A_log", [f"{p}A_log"]),
        E("w_lin_norm", [f"{p}norm.weight"]), E("w_lin_out", [f"{p}out_proj.weight"]),
    ]
