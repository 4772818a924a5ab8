"""Llama family (Llama 2/3/3.1/3.2): pre-norm GQA + SwiGLU (flextrain/io/arch/llama.py:51-402).

No Q/K row permutation is needed on load or export: the kernels use the checkpoint's rotate-half
RoPE layout directly.
"""
from __future__ import annotations

from typing import List

from ...nn.blocks.rope import RopeConfig
from ..hf_weights import ArchSpec
from . import _maps as M
from .common import ModelConfig, config_from_dims as _cfd

FAMILY = "llama"


def default_hyperparams() -> dict:
    return {"rope_theta": 500000.0, "norm_eps": 1e-5}


def config_from_dims(dims: dict, hyper: dict) -> ModelConfig:
    return _cfd(dims, FAMILY, hyper)


def config_from_hf(hf: dict) -> ModelConfig:
    d, H = hf["hidden_size"], hf["num_attention_heads"]
    hd = hf.get("head_dim") or d // H
    return ModelConfig(arch=FAMILY, vocab_size=hf["vocab_size"], n_layers=hf["num_hidden_layers"], d_model=d,
                       n_heads=H, n_kv_heads=hf.get("num_key_value_heads", H), head_dim=hd,
                       ffn_dim=hf["intermediate_size"], norm_eps=hf.get("rms_norm_eps", 1e-5),
                       rope=RopeConfig.from_hf(hf, hd), qkv_bias=bool(hf.get("attention_bias", False)),
                       tie_embeddings=bool(hf.get("tie_word_embeddings", False)), hf=hf)


def to_hf_config(mc: ModelConfig) -> dict:
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": mc.vocab_size,
           "num_hidden_layers": mc.n_layers, "hidden_size": mc.d_model, "num_attention_heads": mc.n_heads,
           "num_key_value_heads": mc.n_kv_heads, "head_dim": mc.head_dim, "intermediate_size": mc.ffn_dim,
           "rms_norm_eps": mc.norm_eps, "rope_theta": mc.rope.theta, "rope_scaling": mc.rope.scaling,
           "hidden_act": "silu", "attention_bias": mc.qkv_bias, "tie_word_embeddings": mc.tie_embeddings,
           "torch_dtype": "bfloat16", "max_position_embeddings": 131072}
    return cfg


def _layer(i: int, mc: ModelConfig) -> List:
    return (M.norm_entries(i, mc) + M.attn_entries(i, mc, bias=mc.qkv_bias, qk_norm=mc.qk_norm is not None)
            + (M.moe_entries(i, mc) if mc.is_moe_layer(i) else M.dense_ffn_entries(i, mc)))


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _layer, ("LlamaForCausalLM",))
