"""Modality containers for multimodal inputs (flextrain/core/modality.py:37-189).

``ImageInputCPU`` is what the data adapter attaches to a :class:`~flextrain_b200.io.sequence.Sequence`; the input
layer batches the images of one round into ``ImageInputs`` (one host-to-device copy), the encoder returns
``ImageEmbeddings`` and the splice consumes them.  ``InputsSummary`` is the per-step accounting the trainer prints."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence as Seq, Tuple

import torch


@dataclass
class ImageInputCPU:
    """Pre-processed patches of ONE image (or video clip) on the host.

    ``pixel_values (t*h*w, C*tp*p*p)`` rows in merge-block-major order; ``grid_thw`` counts patches, so the image
    occupies ``t * (h/merge) * (w/merge)`` placeholder tokens in the text."""
    pixel_values: torch.Tensor
    grid_thw: Tuple[int, int, int]
    first_token: int = 0                 # index of the first placeholder token in the sequence
    kind: str = "image"                  # "image" | "video"
    frame_prefix_ids: Optional[List[List[int]]] = None   # video: token ids written before each temporal patch's block

    def num_placeholders(self, merge: int) -> int:
        t, h, w = self.grid_thw
        return t * (h // merge) * (w // merge)

    def validate(self, patch_dim: int, merge: int) -> None:
        t, h, w = self.grid_thw
        if h % merge or w % merge:
            raise ValueError(f"grid {self.grid_thw} is not a multiple of the merge size {merge}")
        if tuple(self.pixel_values.shape) != (t * h * w, patch_dim):
            raise ValueError(f"pixel_values {tuple(self.pixel_values.shape)} != ({t * h * w}, {patch_dim})")


@dataclass
class ImageInputs:
    """The images of one round, batched for the encoder."""
    pixel_values: torch.Tensor                               # (sum patches, patch_dim)
    grid_thw: List[Tuple[int, int, int]] = field(default_factory=list)
    seq_index: List[int] = field(default_factory=list)      # which sequence of the round each image belongs to

    @staticmethod
    def pack(images: Seq[ImageInputCPU], seq_index: Seq[int], device, dtype, pin: bool = False) -> "ImageInputs":
        if not images:
            return ImageInputs(torch.empty(0, 0, dtype=dtype, device=device))
        host = torch.cat([im.pixel_values for im in images], 0)
        if pin and torch.device(device).type == "cuda":
            host = host.pin_memory()
        return ImageInputs(host.to(device=device, dtype=dtype, non_blocking=True), [tuple(im.grid_thw) for im in images],
                           list(seq_index))

    @property
    def n_images(self) -> int:
        return len(self.grid_thw)


@dataclass
class ImageEmbeddings:
    """Encoder output rows in placeholder order: ``(sum merged patches, d_model)``."""
    embeds: torch.Tensor
    rows_per_image: List[int] = field(default_factory=list)

    def offsets(self) -> List[int]:
        out, acc = [], 0
        for n in self.rows_per_image:
            out.append(acc)
            acc += n
        return out


@dataclass
class ImageGradInputs:
    """Gradient with respect to the encoder rows (unused while the encoder is frozen)."""
    d_embeds: Optional[torch.Tensor] = None


@dataclass
class InputsSummary:
    n_text_tokens: int = 0
    n_image_tokens: int = 0
    n_images: int = 0
    n_patches: int = 0

    def add(self, other: "InputsSummary") -> "InputsSummary":
        return InputsSummary(self.n_text_tokens + other.n_text_tokens, self.n_image_tokens + other.n_image_tokens,
                             self.n_images + other.n_images, self.n_patches + other.n_patches)
