"""Gemma 2: sandwich (pre+post) norms stored as gamma-1, tanh-GeGLU, attention and final logit soft-caps,
``query_pre_attn_scalar`` scale, alternating sliding / full layers, ``sqrt(d)`` embedding scale, tied head
(flextrain/nn/layers/gemma2.py:26-30)."""
from __future__ import annotations

import math
from typing import List

from ...nn.blocks.rope import RopeConfig
from ..hf_weights import ArchSpec
from . import _maps as M
from .common import ModelConfig, config_from_dims as _cfd

FAMILY = "gemma2"


def default_hyperparams() -> dict:
    return {"rope_theta": 10000.0, "norm_eps": 1e-6, "ffn_kind": "geglu", "post_norms": True,
            "attn_softcap": 50.0, "final_softcap": 30.0, "tie_embeddings": True}


def config_from_dims(dims, hyper):
    mc = _cfd(dims, FAMILY, hyper)
    mc.norm_plus_one = True
    mc.embed_scale = math.sqrt(mc.d_model)
    return mc


def _common(hf: dict, family: str) -> ModelConfig:
    d, H = hf["hidden_size"], hf["num_attention_heads"]
    hd = hf.get("head_dim") or d // H
    qpas = hf.get("query_pre_attn_scalar", hd)
    return ModelConfig(arch=family, vocab_size=hf["vocab_size"], n_layers=hf["num_hidden_layers"], d_model=d,
                       n_heads=H, n_kv_heads=hf.get("num_key_value_heads", H), head_dim=hd,
                       ffn_dim=hf["intermediate_size"], norm_eps=hf.get("rms_norm_eps", 1e-6),
                       rope=RopeConfig.from_hf(hf, hd), ffn_kind="geglu", post_norms=True, norm_plus_one=True,
                       attn_scale=float(qpas) ** -0.5, embed_scale=math.sqrt(d),
                       tie_embeddings=bool(hf.get("tie_word_embeddings", True)),
                       sliding_window=int(hf.get("sliding_window") or 0), hf=hf)


def config_from_hf(hf: dict) -> ModelConfig:
    mc = _common(hf, FAMILY)
    mc.attn_softcap = float(hf.get("attn_logit_softcapping") or 0.0)
    mc.final_softcap = float(hf.get("final_logit_softcapping") or 0.0)
    lt = hf.get("layer_types")
    if lt:
        mc.layer_types = ["sliding" if t == "sliding_attention" else "full" for t in lt]
    else:
        mc.layer_types = ["sliding" if i % 2 == 0 else "full" for i in range(mc.n_layers)]
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    return {"architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "vocab_size": mc.vocab_size,
            "num_hidden_layers": mc.n_layers, "hidden_size": mc.d_model, "num_attention_heads": mc.n_heads,
            "num_key_value_heads": mc.n_kv_heads, "head_dim": mc.head_dim, "intermediate_size": mc.ffn_dim,
            "rms_norm_eps": mc.norm_eps, "rope_theta": mc.rope.theta, "hidden_activation": "gelu_pytorch_tanh",
            "attn_logit_softcapping": mc.attn_softcap or None, "final_logit_softcapping": mc.final_softcap or None,
            "query_pre_attn_scalar": round((mc.attn_scale or mc.head_dim ** -0.5) ** -2),
            "sliding_window": mc.sliding_window, "tie_word_embeddings": mc.tie_embeddings, "torch_dtype": "bfloat16"}


def _layer(i: int, mc: ModelConfig) -> List:
    return (M.norm_entries(i, mc, sandwich=True) + M.attn_entries(i, mc, qk_norm=mc.qk_norm is not None)
            + M.dense_ffn_entries(i, mc))


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _layer, ("Gemma2ForCausalLM",))
