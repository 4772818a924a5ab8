"""Multimodal input layer (flextrain/nn/multimodal_input.py:83-355): token embedding + frozen modality encoders.

Once per round (:meth:`setup_round`) the images of the round's sequences are batched, copied to the device and
encoded under ``torch.inference_mode``; the host builds, per chunk, the map from placeholder rows to encoder rows.
Each chunk's embedded text then has its placeholder rows replaced by encoder rows (concat splice).  In backward the
placeholder rows of ``dx`` are zeroed before the embedding's scatter-add.  :meth:`finalize_round` drops the round's
encoder output."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..core.layer import ChunkMeta
from ..core.modality import ImageEmbeddings, ImageInputCPU, ImageInputs, InputsSummary
from .embed import TokenEmbedLayer
from .splices.concat import build_splice_maps, splice_backward, splice_forward


def images_of(seq) -> List[ImageInputCPU]:
    """The images a data adapter attached to a sequence, as :class:`ImageInputCPU` objects."""
    mi = seq.modality_inputs or {}
    if "images" in mi:
        return list(mi["images"])
    if "pixel_values" not in mi:
        return []
    out, off = [], 0
    for g in mi["grid_thw"]:
        n = int(g[0]) * int(g[1]) * int(g[2])
        out.append(ImageInputCPU(mi["pixel_values"][off:off + n], tuple(int(v) for v in g)))
        off += n
    return out


class MultimodalInputLayer:
    def __init__(self, text: TokenEmbedLayer, encoders: Dict[str, object], image_token_id: int,
                 video_token_id: Optional[int] = None):
        self.text = text
        self.encoders = encoders
        self.image_token_id = int(image_token_id)
        self.video_token_id = None if video_token_id is None else int(video_token_id)
        self.param_spec = text.param_spec
        self.vocab_size, self.d_model, self.scale = text.vocab_size, text.d_model, text.scale
        self._embeds: Optional[ImageEmbeddings] = None
        self.last_summary = InputsSummary()

    @property
    def placeholder_ids(self) -> List[int]:
        return [t for t in (self.image_token_id, self.video_token_id) if t is not None and t >= 0]

    def num_vision_layers(self) -> int:
        enc = self.encoders.get("image")
        return enc.cfg.depth if enc is not None else 0

    # ------------------------------------------------------------------ per round
    def setup_round(self, seqs, metas: List[ChunkMeta], device) -> InputsSummary:
        """Encode every image of the round once and attach the splice maps to the chunks."""
        enc = self.encoders.get("image")
        images, owner, row_offset, acc = [], [], {}, 0
        merge = enc.cfg.merge if enc is not None else 1
        for i, s in enumerate(seqs):
            ims = images_of(s)
            if not ims:
                continue
            if enc is None:
                raise RuntimeError("a sequence carries images but the model has no image encoder")
            row_offset[i] = acc
            for im in ims:
                im.validate(enc.cfg.patch_dim, merge)
                images.append(im)
                owner.append(i)
                acc += im.num_placeholders(merge)
        summary = InputsSummary(n_text_tokens=sum(len(s) for s in seqs) - acc, n_image_tokens=acc,
                                n_images=len(images), n_patches=sum(im.pixel_values.shape[0] for im in images))
        self.last_summary = summary
        self._embeds = None
        if not images:
            return summary
        batch = ImageInputs.pack(images, owner, enc.device, enc.dtype, pin=True)
        rows = enc.encode(batch.pixel_values, batch.grid_thw)
        self._embeds = ImageEmbeddings(rows.to(device), enc.rows_per_image(batch.grid_thw))
        maps = build_splice_maps(seqs, [m.extra["pieces"] for m in metas], self.placeholder_ids, row_offset)
        for i in row_offset:                                   # every image row must be consumed exactly once
            n_ph = int(torch.isin(seqs[i].tokens, torch.tensor(self.placeholder_ids)).sum())
            n_rows = sum(im.num_placeholders(merge) for im in images_of(seqs[i]))
            if n_ph != n_rows:
                raise ValueError(f"sequence {seqs[i].seq_id}: {n_ph} placeholder tokens but {n_rows} image rows")
        for m, mp in zip(metas, maps):
            if mp is not None:
                m.extra["mm_rows"] = mp[0].to(device, non_blocking=True)
                m.extra["mm_src"] = mp[1].to(device, non_blocking=True)
        return summary

    def finalize_round(self) -> None:
        self._embeds = None

    # ------------------------------------------------------------------ per chunk
    def forward(self, meta: ChunkMeta, params) -> torch.Tensor:
        x = self.text.forward(meta, params)
        rows = meta.extra.get("mm_rows")
        if rows is None:
            return x
        return splice_forward(x, rows, self._embeds.embeds.index_select(0, meta.extra["mm_src"]))

    def backward(self, dx, meta: ChunkMeta, params, grads) -> None:
        rows = meta.extra.get("mm_rows")
        if rows is not None:
            dx, _ = splice_backward(dx, rows)
        self.text.backward(dx, meta, params, grads)


def attach_multimodal_input(am, hf: dict, model_dir: str, freeze: bool = True, required: bool = False) -> None:
    """Swap the engine's token embedding for a :class:`MultimodalInputLayer` with the checkpoint's vision tower."""
    from ..io.hf_weights import SafetensorsDir
    from .encoders.qwen_vl_vit import QwenVLViT, ViTConfig
    vc = hf.get("vision_config")
    if not vc:
        if required:
            raise ValueError("enable_multimodal=True but config.json has no vision_config")
        return
    if not freeze:
        raise NotImplementedError("the vision tower is frozen in this phase (freeze_modality_encoders=False)")
    if am.tp is not None:
        raise NotImplementedError("multimodal input with tensor parallelism is not supported")
    vit = QwenVLViT(ViTConfig.from_hf(vc), device=am.device,
                    dtype=torch.bfloat16 if am.device.type == "cuda" else torch.float32)
    try:
        vit.load(SafetensorsDir(model_dir))
    except KeyError:
        if required:
            raise
        return
    am.embed = MultimodalInputLayer(am.embed, {"image": vit}, int(hf.get("image_token_id", -1)),
                                    hf.get("video_token_id"))
