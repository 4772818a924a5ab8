"""Sharded safetensors writer and auxiliary-file copy (flextrain/export/_common.py:62)."""
from __future__ import annotations

import json
import os
import shutil
from typing import Dict, Optional

import torch

AUX_FILES = ("tokenizer.json", "tokenizer_config.json", "tokenizer.model", "special_tokens_map.json", "vocab.json",
             "merges.txt", "generation_config.json", "chat_template.jinja", "preprocessor_config.json",
             "added_tokens.json")


def write_sharded_safetensors(state: Dict[str, torch.Tensor], out_dir: str, max_shard_bytes: int = 5 << 30) -> Dict:
    """Write ``state`` as ``model-0000i-of-0000n.safetensors`` (+ index) or a single ``model.safetensors``."""
    from safetensors.torch import save_file
    os.makedirs(out_dir, exist_ok=True)
    shards, cur, cur_bytes = [], {}, 0
    for name, t in state.items():
        nb = t.numel() * t.element_size()
        if cur and cur_bytes + nb > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[name] = t.contiguous()
        cur_bytes += nb
    if cur:
        shards.append(cur)
    total = sum(t.numel() * t.element_size() for t in state.values())
    if len(shards) == 1:
        save_file(shards[0], os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
        return {"metadata": {"total_size": total}, "weight_map": {k: "model.safetensors" for k in state}}
    index = {"metadata": {"total_size": total}, "weight_map": {}}
    for i, sh in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(out_dir, fn), metadata={"format": "pt"})
        for k in sh:
            index["weight_map"][k] = fn
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
        json.dump(index, f, indent=2)
    return index


def copy_aux_files(src_dir: Optional[str], out_dir: str) -> None:
    if not src_dir or not os.path.isdir(src_dir):
        return
    for fn in AUX_FILES:
        p = os.path.join(src_dir, fn)
        if os.path.exists(p):
            shutil.copy2(p, os.path.join(out_dir, fn))
