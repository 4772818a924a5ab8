"""Qwen3-Next: hybrid Gated-DeltaNet / gated full attention (3 linear : 1 full), partial rotary, (1+w) norms,
routed MoE with one sigmoid-gated shared expert (flextrain/nn/layers/qwen3_next.py)."""
from __future__ import annotations

from typing import List

from ...nn.blocks.linear_attn import GDNConfig
from ...nn.blocks.rope import RopeConfig
from ..hf_weights import ArchSpec
from . import _maps as M
from .common import ModelConfig, config_from_dims as _cfd

FAMILY = "qwen3_next"


def default_hyperparams() -> dict:
    return {"rope_theta": 10000000.0, "norm_eps": 1e-6, "qk_norm": "head", "gated_attn": True,
            "partial_rotary_factor": 0.25, "layer_pattern": "3L1F", "routing": "topk_then_softmax"}


def config_from_dims(dims, hyper):
    mc = _cfd(dims, FAMILY, hyper)
    mc.norm_plus_one = True
    if mc.gdn is None and any(t == "linear" for t in (mc.layer_types or [])):
        mc.gdn = GDNConfig(d_model=mc.d_model, n_k_heads=max(1, mc.n_kv_heads), n_v_heads=mc.n_heads,
                           head_k_dim=mc.head_dim, head_v_dim=mc.head_dim, norm_eps=mc.norm_eps)
    return mc


def hybrid_from_hf(hf: dict, family: str) -> ModelConfig:
    txt = hf.get("text_config", hf)
    d, H = txt["hidden_size"], txt["num_attention_heads"]
    hd = txt.get("head_dim") or d // H
    mc = ModelConfig(arch=family, vocab_size=txt["vocab_size"], n_layers=txt["num_hidden_layers"], d_model=d,
                     n_heads=H, n_kv_heads=txt.get("num_key_value_heads", H), head_dim=hd,
                     ffn_dim=txt.get("intermediate_size", 0), norm_eps=txt.get("rms_norm_eps", 1e-6),
                     rope=RopeConfig.from_hf(txt, hd), qk_norm="head", gated_attn=True, norm_plus_one=True,
                     tie_embeddings=bool(txt.get("tie_word_embeddings", False)), hf=hf)
    lt = txt.get("layer_types")
    if lt:
        mc.layer_types = ["linear" if t == "linear_attention" else "full" for t in lt]
    else:
        k = int(txt.get("full_attention_interval", 4))
        mc.layer_types = ["full" if (i + 1) % k == 0 else "linear" for i in range(mc.n_layers)]
    mc.gdn = GDNConfig(d_model=d, n_k_heads=txt["linear_num_key_heads"], n_v_heads=txt["linear_num_value_heads"],
                       head_k_dim=txt["linear_key_head_dim"], head_v_dim=txt["linear_value_head_dim"],
                       conv_width=txt.get("linear_conv_kernel_dim", 4), norm_eps=mc.norm_eps)
    if mc.rope.mrope_sections:
        mc.mrope_sections = mc.rope.mrope_sections
    if txt.get("num_experts", 0):
        mc.num_experts, mc.top_k = int(txt["num_experts"]), int(txt["num_experts_per_tok"])
        mc.expert_dim = int(txt["moe_intermediate_size"])
        mc.shared_dim = int(txt.get("shared_expert_intermediate_size", 0) or 0)
        mc.shared_gate = True
        mc.routing = "topk_then_softmax" if txt.get("norm_topk_prob", True) else "softmax_then_topk"
    return mc


def config_from_hf(hf: dict) -> ModelConfig:
    return hybrid_from_hf(hf, FAMILY)


def to_hf_config(mc: ModelConfig) -> dict:
    g = mc.gdn
    c = {"architectures": ["Qwen3NextForCausalLM"], "model_type": "qwen3_next", "vocab_size": mc.vocab_size,
         "num_hidden_layers": mc.n_layers, "hidden_size": mc.d_model, "num_attention_heads": mc.n_heads,
         "num_key_value_heads": mc.n_kv_heads, "head_dim": mc.head_dim, "intermediate_size": mc.ffn_dim,
         "rms_norm_eps": mc.norm_eps, "rope_theta": mc.rope.theta,
         "partial_rotary_factor": mc.rope.partial_rotary_factor,
         "layer_types": ["linear_attention" if t == "linear" else "full_attention" for t in (mc.layer_types or [])],
         "tie_word_embeddings": mc.tie_embeddings, "torch_dtype": "bfloat16"}
    if g is not None:
        c.update({"linear_num_key_heads": g.n_k_heads, "linear_num_value_heads": g.n_v_heads,
                  "linear_key_head_dim": g.head_k_dim, "linear_value_head_dim": g.head_v_dim,
                  "linear_conv_kernel_dim": g.conv_width})
    if mc.num_experts:
        c.update({"num_experts": mc.num_experts, "num_experts_per_tok": mc.top_k,
                  "moe_intermediate_size": mc.expert_dim, "shared_expert_intermediate_size": mc.shared_dim,
                  "norm_topk_prob": mc.routing == "topk_then_softmax"})
    return c


def _layer(i: int, mc: ModelConfig) -> List:
    out = M.norm_entries(i, mc)
    if mc.layer_type(i) == "linear":
        out += M.gdn_entries(i, mc)
    else:
        out += M.attn_entries(i, mc, qk_norm=True)
    out += M.moe_entries(i, mc) if mc.is_moe_layer(i) else M.dense_ffn_entries(i, mc)
    return out


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _layer, ("Qwen3NextForCausalLM",))
