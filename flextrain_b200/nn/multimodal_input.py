"""Multimodal input layer (flextrain/nn/multimodal_input.py:1-52): token embedding + frozen modality encoders.

Once per round the images of the round's sequences are encoded (``torch.inference_mode``); each chunk's embedded
text then has its placeholder rows replaced by the encoder rows (concat splice).  In backward the placeholder rows
of ``dx`` are zeroed before the embedding scatter-add."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..core.layer import ChunkMeta
from .embed import TokenEmbedLayer
from .splices.concat import splice_backward, splice_forward


class MultimodalInputLayer:
    def __init__(self, text: TokenEmbedLayer, encoders: Dict[str, object], placeholder_token_id: int):
        self.text = text
        self.encoders = encoders
        self.placeholder_token_id = placeholder_token_id
        self.param_spec = text.param_spec
        self.vocab_size, self.d_model, self.scale = text.vocab_size, text.d_model, text.scale
        self._rows: Dict[int, torch.Tensor] = {}           # seq_id -> encoder rows for this round

    def begin_round(self, seqs) -> None:
        """Encode every image of the round once."""
        self._rows.clear()
        enc = self.encoders.get("image")
        for s in seqs:
            mi = s.modality_inputs or {}
            if "pixel_values" in mi and enc is not None:
                self._rows[s.seq_id] = enc.encode(mi["pixel_values"], mi["grid_thw"])

    def forward(self, meta: ChunkMeta, params) -> torch.Tensor:
        x = self.text.forward(meta, params)
        ph = (meta.tokens == self.placeholder_token_id).nonzero(as_tuple=True)[0]
        meta.extra["placeholder_rows"] = ph
        if ph.numel() == 0:
            return x
        rows, used = [], meta.extra.setdefault("mm_row_cursor", {})
        cu = meta.cu_seqlens_q.tolist()
        for j, sid in enumerate(meta.seq_ids):
            n = int(((ph >= cu[j]) & (ph < cu[j + 1])).sum())
            if n:
                start = meta.extra.get("mm_row_start", {}).get(sid, 0)
                rows.append(self._rows[sid][start:start + n])
        return splice_forward(x, ph, torch.cat(rows, 0).to(x.device))

    def backward(self, dx, meta: ChunkMeta, params, grads) -> None:
        ph = meta.extra.get("placeholder_rows")
        if ph is not None and ph.numel():
            dx, _ = splice_backward(dx, ph)
        self.text.backward(dx, meta, params, grads)


def attach_multimodal_input(am, hf: dict, model_dir: str, freeze: bool = True, required: bool = False) -> None:
    """Swap the engine's token embedding for a :class:`MultimodalInputLayer` with a Qwen-VL vision tower."""
    from ..io.hf_weights import SafetensorsDir
    from .encoders.qwen_vl_vit import QwenVLViT, ViTConfig
    vc = hf.get("vision_config")
    if not vc:
        if required:
            raise ValueError("enable_multimodal=True but config.json has no vision_config")
        return
    vit = QwenVLViT(ViTConfig.from_hf(vc), device=am.device, dtype=torch.bfloat16 if am.device.type == "cuda" else torch.float32)
    try:
        vit.load(SafetensorsDir(model_dir))
    except KeyError:
        if required:
            raise
        return
    am.embed = MultimodalInputLayer(am.embed, {"image": vit}, int(hf.get("image_token_id", -1)))
