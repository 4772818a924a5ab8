"""Image pre-processing for multimodal SFT (flextrain/io/image_processing.py:40-278): resize to a multiple of
``patch * merge``, normalise, cut into ``temporal x patch x patch`` patches, and build a :class:`Sequence` whose
text holds one placeholder token per merged patch."""
from __future__ import annotations

from typing import List, Sequence as Seq, Tuple

import torch

from ..core.modality import ImageInputCPU
from .sequence import Sequence

MEAN = (0.48145466, 0.4578275, 0.40821073)
STD = (0.26862954, 0.26130258, 0.27577711)


def patchify(img: torch.Tensor, patch: int = 14, temporal_patch: int = 2, merge: int = 2) -> ImageInputCPU:
    """``img (3, H, W)`` float in [0, 1] → ``ImageInputCPU`` with rows ordered (merge-block-major) like the HF processor."""
    c, H, W = img.shape
    q = patch * merge
    Hn, Wn = max(q, round(H / q) * q), max(q, round(W / q) * q)
    if (Hn, Wn) != (H, W):
        img = torch.nn.functional.interpolate(img[None], size=(Hn, Wn), mode="bicubic", align_corners=False)[0]
    mean, std = torch.tensor(MEAN).view(3, 1, 1), torch.tensor(STD).view(3, 1, 1)
    img = (img - mean) / std
    frames = img[None].repeat(temporal_patch, 1, 1, 1)                       # a still image fills the temporal patch
    gh, gw = Hn // patch, Wn // patch
    x = frames.view(temporal_patch, c, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(2, 5, 3, 6, 1, 0, 4, 7).reshape(gh * gw, c * temporal_patch * patch * patch)
    return ImageInputCPU(pixel_values=x.contiguous(), grid_thw=(1, gh, gw))


def build_multimodal_sequence(text_ids_before: Seq[int], image: ImageInputCPU, text_ids_after: Seq[int],
                              placeholder_id: int, merge: int = 2, seq_id: int = 0) -> Sequence:
    t, gh, gw = image.grid_thw
    n_ph = t * (gh // merge) * (gw // merge)
    ids = list(text_ids_before) + [placeholder_id] * n_ph + list(text_ids_after)
    toks = torch.tensor(ids, dtype=torch.int64)
    tgt = torch.roll(toks, -1)
    tgt[-1] = -100
    first = len(text_ids_before)
    tgt[max(first - 1, 0): first + n_ph] = -100                              # never predict placeholder tokens
    return Sequence(toks, targets=tgt, seq_id=seq_id,
                    modality_inputs={"pixel_values": image.pixel_values, "grid_thw": [image.grid_thw],
                                     "image_spans": [(first, t, gh // merge, gw // merge)]})
