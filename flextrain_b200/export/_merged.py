"""Merged export: fold ``W += scale * B @ A`` into the base weights in fp32 on the CPU, then write a full HF
directory (flextrain/export/_merged.py:63,133)."""
from __future__ import annotations

import torch


def merged_weight(params, name: str, am) -> torch.Tensor:
    lora = am.layers[0].cfg.lora
    w = params[name].detach().to("cpu", torch.float32)
    a = params[name + "_lora_a"].detach().to("cpu", torch.float32)
    b = params[name + "_lora_b"].detach().to("cpu", torch.float32)
    if w.dim() == 3:      # per-expert adapters: (E, out, r) @ (E, r, in)
        return (w + lora.scale * torch.bmm(b, a)).to(params[name].dtype)
    return (w + lora.scale * (b @ a)).to(params[name].dtype)


def merge_lora_into_base(am) -> int:
    """In-place merge on the engine's master weights; adapters are reset to the identity (B = 0).  Returns the number
    of weights merged (flextrain/export/_merged.py:63-130)."""
    n = 0
    for l in range(len(am.layers)):
        p = am.buffers.host_params(l)
        for name in [n_ for n_ in list(p) if (n_ + "_lora_a") in p]:
            p[name].copy_(merged_weight(p, name, am).to(p[name].device))
            p[name + "_lora_b"].zero_()
            n += 1
    return n


def save_hf_merged(am, out_dir: str, *, keep_lora_after_merge: bool = True, **kw) -> str:
    """Full HF directory with ``W + scale * B A`` folded in.  The merge happens on the way out: the engine's weights
    and adapters stay as they are (``keep_lora_after_merge=False`` also merges them in memory, which is what the
    reference's default leaves behind; the model computes the same function either way)."""
    from ._hf_full import save_hf_full
    out = save_hf_full(am, out_dir, _merge_lora=True, **kw)
    if not keep_lora_after_merge:
        merge_lora_into_base(am)
    return out
