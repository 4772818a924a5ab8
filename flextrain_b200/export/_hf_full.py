"""Full HF-directory export (flextrain/export/_hf_full.py:311): sharded safetensors in checkpoint names,
``config.json`` and tokenizer files.  No Q/K permutation has to be undone (weights never left the checkpoint's
rotate-half layout); (1+w) norms are written back as ``gamma - 1``; MoE stacks and bundled linear-attention
projections are split by the arch map's ``split`` callables."""
from __future__ import annotations

import json
import os
from typing import Optional

from ..io.arch import select_arch_module
from ..io.hf_weights import checkpoint_names, collect_hf_state, is_export_writer, passthrough_tensors
from ._common import copy_aux_files, write_sharded_safetensors


def save_hf_full(am, out_dir: str, *, max_shard_bytes: Optional[int] = None, source_dir: Optional[str] = None,
                 _merge_lora: bool = False, hf_source_dir: Optional[str] = None, shard_size_bytes: Optional[int] = None,
                 arch=None) -> str:
    """``hf_source_dir`` / ``shard_size_bytes`` are the reference's names for ``source_dir`` / ``max_shard_bytes``; the
    family's name map comes from the model's own configuration, so ``arch`` is accepted and not needed."""
    source_dir = source_dir or hf_source_dir
    max_shard_bytes = max_shard_bytes or shard_size_bytes or (5 << 30)
    state = collect_hf_state(am, lora_merge=_merge_lora)          # collective under tensor / expert parallelism
    if not is_export_writer(am):
        return out_dir
    src = source_dir or am.model_dir
    # a checkpoint that nests its decoder (vision-language wrappers) gets its own names back, and what the engine does
    # not hold (vision tower, extra heads) is copied over from the source, so the directory loads where the source did
    state = checkpoint_names(state, getattr(am, "hf_nested_prefix", None))
    encoders = getattr(am.embed, "encoder_export_state", None)
    if encoders is not None:
        state.update(encoders())
    passthrough_tensors(src, state)
    write_sharded_safetensors(state, out_dir, max_shard_bytes)
    cfg = None
    if src and os.path.exists(os.path.join(src, "config.json")):
        with open(os.path.join(src, "config.json")) as f:
            cfg = json.load(f)
    if cfg is None:
        cfg = select_arch_module(am.model_config.arch).to_hf_config(am.model_config)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    copy_aux_files(src, out_dir)
    return out_dir
