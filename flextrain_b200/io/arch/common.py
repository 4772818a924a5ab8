"""Family-independent model description and the block builder every architecture shares.

An architecture module (``io/arch/<family>.py``) only has to translate between its HuggingFace
``config.json`` / dims dict and a :class:`ModelConfig`, and to declare its checkpoint name map; the
layers themselves are built here from the same blocks.  This plays the role of the reference's
per-arch ``hf_config_to_flextrain`` / ``hf_config_to_hyperparams`` / ``expand_dims`` /
``default_hyperparams`` / ``BLOCK_BUILDER`` set (flextrain/io/arch/llama.py:139-323).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import List, Optional, Tuple

import torch

from ...nn.blocks.attention import AttentionConfig
from ...nn.blocks.ffn_dense import DenseFFNConfig
from ...nn.blocks.ffn_moe import MoEConfig
from ...nn.blocks.linear import LORA_ALL_TARGETS, LoRAConfig
from ...nn.blocks.linear_attn import GDNConfig
from ...nn.blocks.rope import RopeConfig
from ...nn.embed import TokenEmbedLayer
from ...nn.head import LMHead
from ...nn.layers.decoder import DecoderConfig, DecoderLayer


@dataclass
class ModelConfig:
    arch: str
    vocab_size: int
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn_dim: int
    norm_eps: float = 1e-5
    rope: RopeConfig = field(default_factory=RopeConfig)
    rope_local: Optional[RopeConfig] = None          # Gemma-3 sliding layers use their own base
    layer_types: Optional[List[str]] = None          # per layer: "full" | "sliding" | "linear"
    sliding_window: int = 0
    qkv_bias: bool = False
    qk_norm: Optional[str] = None
    attn_softcap: float = 0.0
    final_softcap: float = 0.0
    attn_scale: Optional[float] = None
    gated_attn: bool = False
    ffn_kind: str = "swiglu"
    # MoE
    num_experts: int = 0
    top_k: int = 0
    expert_dim: int = 0
    routing: str = "topk_then_softmax"
    shared_dim: int = 0
    shared_gate: bool = True
    aux_loss_alpha: float = 0.0
    moe_layers: Optional[List[bool]] = None          # which layers are MoE (default: all when num_experts > 0)
    # Gated DeltaNet
    gdn: Optional[GDNConfig] = None
    # misc
    post_norms: bool = False
    embed_scale: float = 1.0
    tie_embeddings: bool = False
    norm_plus_one: bool = False                      # checkpoint stores gamma - 1 (Gemma, Qwen3.5/Next)
    is_causal: bool = True
    v_norm: bool = False                             # Gemma 4: scale-free per-head RMSNorm of V
    layer_scalar: bool = False                       # Gemma 4: stored per-layer output multiplier
    mrope_sections: Optional[Tuple[int, int, int]] = None
    hf: Optional[dict] = None

    def layer_type(self, i: int) -> str:
        return self.layer_types[i] if self.layer_types else "full"

    def is_moe_layer(self, i: int) -> bool:
        if self.num_experts <= 0:
            return False
        return True if self.moe_layers is None else bool(self.moe_layers[i])


@dataclass
class DTypePolicy:
    compute: torch.dtype = torch.bfloat16
    master: Optional[torch.dtype] = torch.bfloat16
    grad: Optional[torch.dtype] = torch.bfloat16
    norm: torch.dtype = torch.float32
    norm_grad: torch.dtype = torch.float32


def expand_layer_pattern(pattern: str, n_layers: int) -> List[str]:
    """``"3L1F"`` → ``[linear, linear, linear, full] * (n/4)`` (flextrain/io/arch/__init__.py:92-141).
    Letters: ``L`` linear attention, ``F`` full attention, ``S`` sliding-window attention."""
    names = {"L": "linear", "F": "full", "S": "sliding"}
    unit: List[str] = []
    num = ""
    for ch in pattern:
        if ch.isdigit():
            num += ch
        else:
            unit += [names[ch.upper()]] * int(num or "1")
            num = ""
    if not unit:
        raise ValueError(f"empty layer pattern {pattern!r}")
    return [unit[i % len(unit)] for i in range(n_layers)]


def resolve_lora(lora_targets, rank: int, alpha: float, compute, master, grad, opt) -> Optional[LoRAConfig]:
    if not lora_targets:
        return None
    if lora_targets in ("all", True):
        targets = LORA_ALL_TARGETS
    else:
        alias = {"q_proj": "w_q", "k_proj": "w_k", "v_proj": "w_v", "o_proj": "w_o", "gate_proj": "w_1",
                 "down_proj": "w_2", "up_proj": "w_3"}
        targets = tuple(alias.get(t, t if t.startswith("w_") else "w_" + t) for t in lora_targets)
    return LoRAConfig(targets=targets, rank=rank, alpha=alpha, compute_dtype=compute or torch.bfloat16,
                      master_dtype=master or torch.bfloat16, grad_dtype=grad or torch.bfloat16,
                      opt_state_dtype=opt or torch.bfloat16)


TP_COL_TENSORS = ("w_q", "w_k", "w_v", "b_q", "b_k", "b_v", "w_1", "w_3")     # split along dim 0 (output features)
TP_ROW_TENSORS = ("w_o", "w_2")                                              # split along dim 1 (input features)


def localize_for_tp(mc: ModelConfig, tp: int) -> ModelConfig:
    """The per-rank model of a ``tp``-way tensor-parallel layout: heads and FFN width divided by ``tp``."""
    if tp <= 1:
        return mc
    if mc.n_heads % tp or mc.n_kv_heads % tp or mc.ffn_dim % tp:
        raise ValueError(f"tensor parallel degree {tp} must divide n_heads {mc.n_heads}, n_kv_heads {mc.n_kv_heads} "
                         f"and ffn_dim {mc.ffn_dim}")
    if mc.num_experts > 0 or mc.gdn is not None or mc.qk_norm == "row":
        raise NotImplementedError("tensor parallelism covers dense attention + gated-FFN models (per-head QK-norm, "
                                  "sandwich norms, windows and soft-caps included; no MoE, linear attention or "
                                  "full-row QK-norm)")
    return replace(mc, n_heads=mc.n_heads // tp, n_kv_heads=mc.n_kv_heads // tp, ffn_dim=mc.ffn_dim // tp)


def build_decoder_config(mc: ModelConfig, i: int, dt: DTypePolicy, lora: Optional[LoRAConfig]) -> DecoderConfig:
    lt = mc.layer_type(i)
    attn = gdn = None
    if lt == "linear":
        gdn = mc.gdn
    else:
        rope = mc.rope_local if (lt == "sliding" and mc.rope_local is not None) else mc.rope
        if mc.mrope_sections is not None:
            rope = replace(rope, mrope_sections=mc.mrope_sections)
        attn = AttentionConfig(d_model=mc.d_model, n_heads=mc.n_heads, n_kv_heads=mc.n_kv_heads, head_dim=mc.head_dim,
                               rope=rope, qkv_bias=mc.qkv_bias, qk_norm=mc.qk_norm, norm_eps=mc.norm_eps,
                               softcap=mc.attn_softcap, window=mc.sliding_window if lt == "sliding" else 0,
                               scale=mc.attn_scale, gated=mc.gated_attn, causal=mc.is_causal, v_norm=mc.v_norm)
    ffn = moe = None
    if mc.is_moe_layer(i):
        moe = MoEConfig(d_model=mc.d_model, num_experts=mc.num_experts, top_k=mc.top_k, expert_dim=mc.expert_dim,
                        routing=mc.routing, aux_loss_alpha=mc.aux_loss_alpha, shared_dim=mc.shared_dim,
                        shared_gate=mc.shared_gate, kind=mc.ffn_kind)
    else:
        ffn = DenseFFNConfig(mc.d_model, mc.ffn_dim, mc.ffn_kind)
    return DecoderConfig(d_model=mc.d_model, attn=attn, gdn=gdn, ffn=ffn, moe=moe, norm_eps=mc.norm_eps,
                         post_norms=mc.post_norms, dtype=dt.compute, norm_dtype=dt.norm, grad_dtype=dt.grad,
                         norm_grad_dtype=dt.norm_grad, master_dtype=dt.master, lora=lora, family=mc.arch,
                         layer_scalar=mc.layer_scalar)


def build_model_parts(mc: ModelConfig, dt: DTypePolicy, lora: Optional[LoRAConfig], head_chunk_size: int = 4096,
                      block_builder=None, tp: int = 1, tp_rank: int = 0):
    """Returns ``(embed, layers, head)``; under LoRA the embedding and head are frozen
    (flextrain/api.py:568-582).  With ``tp > 1`` the layers are this rank's part of a tensor-parallel model."""
    mc = localize_for_tp(mc, tp)
    frozen = lora is not None
    embed = TokenEmbedLayer(mc.vocab_size, mc.d_model, dtype=dt.compute, grad_dtype=dt.grad, master_dtype=dt.master,
                            scale=mc.embed_scale, frozen=frozen)
    head = LMHead(mc.vocab_size, mc.d_model, dtype=dt.compute, norm_dtype=dt.norm, grad_dtype=dt.grad,
                  master_dtype=dt.master, norm_eps=mc.norm_eps, head_chunk_size=head_chunk_size,
                  final_softcap=mc.final_softcap, frozen=frozen, tied=mc.tie_embeddings)
    layers = []
    for i in range(mc.n_layers):
        cfg = build_decoder_config(mc, i, dt, lora)
        if tp > 1:
            cfg.seq_parallel = tp
        layer = block_builder(i, cfg, mc) if block_builder is not None else DecoderLayer(cfg, i)
        if tp > 1:
            for t in layer.param_spec.tensors:
                if t.name in TP_COL_TENSORS:
                    t.mark_local(0, tp_rank, tp)
                elif t.name in TP_ROW_TENSORS:
                    t.mark_local(1, tp_rank, tp)
                # LoRA on a sharded weight W (out, in): W + s * B @ A stays local when the adapter on the sharded side
                # is sharded with it (B rows for column-parallel W, A columns for row-parallel W); the other adapter is
                # replicated and its gradient, a partial sum on every rank, goes through the data-parallel reduction
                elif t.name.endswith("_lora_b") and t.name[: -len("_lora_b")] in TP_COL_TENSORS:
                    t.mark_local(0, tp_rank, tp)
                elif t.name.endswith("_lora_a") and t.name[: -len("_lora_a")] in TP_ROW_TENSORS:
                    t.mark_local(1, tp_rank, tp)
        layers.append(layer)
    return embed, layers, head


def config_from_dims(dims: dict, arch: str, hyper: Optional[dict] = None) -> ModelConfig:
    """FlexTrain dims dict (``orig/model_dims.json`` keys) + hyper-parameters → :class:`ModelConfig`."""
    h = dict(hyper or {})
    E = int(dims.get("num_routed_experts", 0) or 0)
    rope = RopeConfig(theta=float(h.get("rope_theta", 10000.0)), scaling=h.get("rope_scaling"),
                      partial_rotary_factor=float(h.get("partial_rotary_factor", 1.0)))
    mc = ModelConfig(
        arch=arch, vocab_size=int(dims["vocab_size"]), n_layers=int(dims["n_layers"]), d_model=int(dims["d_model"]),
        n_heads=int(dims["n_heads"]), n_kv_heads=int(dims["n_kv_heads"]), head_dim=int(dims["head_dim"]),
        ffn_dim=int(dims.get("ffn_dim", dims.get("expert_dim", 0))), norm_eps=float(h.get("norm_eps", 1e-5)),
        rope=rope, num_experts=E, top_k=int(dims.get("top_k", 0) or 0),
        expert_dim=int(dims.get("expert_dim", 0)) if E > 0 else 0,
        shared_dim=int(dims.get("shared_dim", dims.get("expert_dim", 0))) * int(
            dims.get("num_shared_experts", 0) or 0) if E > 0 else 0,
        is_causal=bool(dims.get("is_causal", True)))
    for k in ("qkv_bias", "qk_norm", "attn_softcap", "final_softcap", "sliding_window", "routing", "ffn_kind",
              "post_norms", "embed_scale", "gated_attn", "shared_gate", "aux_loss_alpha", "tie_embeddings", "v_norm",
              "layer_scalar", "attn_scale"):
        if k in h:
            setattr(mc, k, h[k])
    if "layer_pattern" in h:
        mc.layer_types = expand_layer_pattern(h["layer_pattern"], mc.n_layers)
    if "gdn" in h:
        g = h["gdn"]
        mc.gdn = GDNConfig(d_model=mc.d_model, n_k_heads=g["n_k_heads"], n_v_heads=g["n_v_heads"],
                           head_k_dim=g["head_k_dim"], head_v_dim=g["head_v_dim"], conv_width=g.get("conv_width", 4),
                           norm_eps=mc.norm_eps)
    return mc
