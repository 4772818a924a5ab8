"""Gemma 3 (text tower): Gemma-2 sandwich norms + per-head QK-norm, no soft-caps, 5 sliding : 1 global layers
with a separate RoPE base for sliding layers (flextrain/nn/layers/gemma3.py)."""
from __future__ import annotations

from ...nn.blocks.rope import RopeConfig
from ..hf_weights import ArchSpec
from . import _maps as M
from . import gemma2 as _g
from .common import ModelConfig

FAMILY = "gemma3"


def default_hyperparams() -> dict:
    return {"rope_theta": 1000000.0, "norm_eps": 1e-6, "ffn_kind": "geglu", "post_norms": True, "qk_norm": "head",
            "tie_embeddings": True}


def config_from_dims(dims, hyper):
    mc = _g.config_from_dims(dims, {**default_hyperparams(), **hyper})
    mc.arch = FAMILY
    mc.rope_local = RopeConfig(theta=float(hyper.get("rope_local_theta", 10000.0)))   # sliding layers' own base
    return mc


def config_from_hf(hf: dict) -> ModelConfig:
    txt = hf.get("text_config", hf)
    mc = _g._common(txt, FAMILY)
    mc.qk_norm = "head"
    mc.hf = hf
    lt = txt.get("layer_types")
    if lt:
        mc.layer_types = ["sliding" if t == "sliding_attention" else "full" for t in lt]
    else:
        pat = int(txt.get("sliding_window_pattern", 6))
        mc.layer_types = ["full" if (i + 1) % pat == 0 else "sliding" for i in range(mc.n_layers)]
    mc.rope_local = RopeConfig(theta=float(txt.get("rope_local_base_freq", 10000.0)))
    rp = txt.get("rope_parameters") or {}
    if "full_attention" in rp or "sliding_attention" in rp:       # transformers >= 5: one parameter set per layer type
        mc.rope = RopeConfig.from_hf({"rope_parameters": rp.get("full_attention", {})}, mc.head_dim)
        mc.rope_local = RopeConfig.from_hf({"rope_parameters": rp.get("sliding_attention", {})}, mc.head_dim)
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _g.to_hf_config(mc)
    c.update({"architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
              "rope_local_base_freq": mc.rope_local.theta if mc.rope_local else 10000.0,
              "layer_types": ["sliding_attention" if t == "sliding" else "full_attention" for t in (mc.layer_types or [])],
              "rope_scaling": mc.rope.scaling})
    c.pop("attn_logit_softcapping", None); c.pop("final_logit_softcapping", None)
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _g._layer,
                     ("Gemma3ForCausalLM", "Gemma3ForConditionalGeneration"))
