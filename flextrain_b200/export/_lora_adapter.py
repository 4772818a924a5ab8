"""PEFT-format LoRA adapter export (flextrain/export/_lora_adapter.py:198): ``adapter_config.json`` +
``adapter_model.safetensors`` with ``base_model.model.<module>.lora_A/B.weight``.  Adapter tensors are already
in PEFT orientation (``A (r, in)``, ``B (out, r)``).

Per-expert adapters of mixture-of-experts layers (stacked ``w_up_lora_a (E, r, d)`` / ``w_up_lora_b (E, 2F, r)`` with the
rows ``[up ‖ gate]``, ``w_down_lora_a (E, r, F)`` / ``w_down_lora_b (E, d, r)``) are written one module per expert under
the family's checkpoint names (``...mlp.experts.<e>.{gate,up,down}_proj``): gate and up share the expert's ``A`` and
take their halves of ``B``, which is exactly the adapter that was trained on the fused projection.  (The reference's
exporter covers the Llama-style modules only.)"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch

_MODULE = {"w_q": "self_attn.q_proj", "w_k": "self_attn.k_proj", "w_v": "self_attn.v_proj", "w_o": "self_attn.o_proj",
           "w_1": "mlp.gate_proj", "w_3": "mlp.up_proj", "w_2": "mlp.down_proj"}


def _wrapper_module_prefix(am):
    """Adapter keys follow the MODULE tree of the class the base checkpoint loads as, not the tensor names in its
    files: a vision-language wrapper (``...ForConditionalGeneration``) holds the decoder under the nested prefix the
    checkpoint uses, while the family's causal-LM class has ``model.layers`` even when its files spell the nested
    names.  Returns the nested prefix for the former, ``None`` otherwise."""
    nested = getattr(am, "hf_nested_prefix", None)
    if not nested or not getattr(am, "model_dir", None):
        return None
    try:
        with open(os.path.join(am.model_dir, "config.json")) as f:
            archs = json.load(f).get("architectures") or []
    except OSError:
        return None
    return nested if any(a.endswith("ForConditionalGeneration") for a in archs) else None


def save_lora_adapter(am, out_dir: str, base_model_name_or_path: Optional[str] = "", *, arch=None,
                      rank: Optional[int] = None, alpha: Optional[float] = None, bias: str = "none") -> str:
    """``rank`` / ``alpha`` override what ``adapter_config.json`` records (default: the values the model was built
    with); ``bias`` is written through; ``arch`` is accepted and not needed (flextrain/export/_lora_adapter.py:198)."""
    from safetensors.torch import save_file
    from ..io.hf_weights import gather_local_parts, is_export_writer
    lora = am.layers[0].cfg.lora
    if lora is None:
        raise ValueError("model was not built with LoRA")
    state = {}

    def whole(l, key, t):
        spec = am.layers[l].param_spec.get(key)
        if spec is not None and spec.is_local_part:            # tensor parallel: every rank takes part in the gather
            t = gather_local_parts(t.detach(), spec, am)
        return t.detach().to("cpu", torch.float32).contiguous()

    for l in range(len(am.layers)):
        p = am.buffers.host_params(l)
        for name, mod in _MODULE.items():
            if name + "_lora_a" in p:
                base = f"base_model.model.model.layers.{l}.{mod}"
                state[f"{base}.lora_A.weight"] = whole(l, name + "_lora_a", p[name + "_lora_a"])
                state[f"{base}.lora_B.weight"] = whole(l, name + "_lora_b", p[name + "_lora_b"])
    # per-expert adapters on the routed expert stacks
    expert_targets = set()
    mc = getattr(am, "model_config", None)
    if mc is not None and getattr(mc, "num_experts", 0) > 0:
        from ..io.arch import select_arch_module
        spec_of = select_arch_module(mc.arch).ARCH_SPEC.layer
        for l in range(len(am.layers)):
            p = am.buffers.host_params(l)
            if "w_up_lora_a" not in p and "w_down_lora_a" not in p:
                continue
            entries = {e.name: e for e in spec_of(l, mc)}
            mod = lambda hf_name: "base_model.model." + hf_name[: -len(".weight")] if hf_name.endswith(".weight") \
                else "base_model.model." + hf_name
            if "w_up_lora_a" in p and "w_up" in entries:
                a, b = whole(l, "w_up_lora_a", p["w_up_lora_a"]), whole(l, "w_up_lora_b", p["w_up_lora_b"])
                names = list(entries["w_up"].hf_names)                 # [e0.up, e0.gate, e1.up, e1.gate, ...]
                F = b.shape[1] // 2
                for e in range(a.shape[0]):
                    for half, hf_name in ((b[e, :F], names[2 * e]), (b[e, F:], names[2 * e + 1])):
                        state[f"{mod(hf_name)}.lora_A.weight"] = a[e].clone()
                        state[f"{mod(hf_name)}.lora_B.weight"] = half.clone()
                expert_targets |= {"gate_proj", "up_proj"}
            if "w_down_lora_a" in p and "w_down" in entries:
                a, b = whole(l, "w_down_lora_a", p["w_down_lora_a"]), whole(l, "w_down_lora_b", p["w_down_lora_b"])
                names = list(entries["w_down"].hf_names)
                for e in range(a.shape[0]):
                    state[f"{mod(names[e])}.lora_A.weight"] = a[e].clone()
                    state[f"{mod(names[e])}.lora_B.weight"] = b[e].clone()
                expert_targets.add("down_proj")
    if not is_export_writer(am):
        return out_dir
    nested = _wrapper_module_prefix(am)
    if nested:                      # vision-language wrappers: the decoder's modules live under the wrapper's prefix
        head = "base_model.model.model."
        state = {("base_model.model." + nested + k[len(head):] if k.startswith(head) else k): v
                 for k, v in state.items()}
    os.makedirs(out_dir, exist_ok=True)
    save_file(state, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
    cfg = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": int(rank or lora.rank),
           "lora_alpha": float(alpha if alpha is not None else lora.alpha), "lora_dropout": 0.0, "bias": bias, "fan_in_fan_out": False, "inference_mode": True,
           "target_modules": sorted({_MODULE[t].split(".")[-1] for t in lora.targets if t in _MODULE} | expert_targets),
           "base_model_name_or_path": base_model_name_or_path or (am.model_dir or "")}
    with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return out_dir
