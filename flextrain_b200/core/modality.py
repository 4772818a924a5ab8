"""Modality containers for multimodal inputs (flextrain/core/modality.py:37-189)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch


@dataclass
class ImageInputCPU:
    """Pre-processed image patches on the host: ``pixel_values (n_patches, patch_dim)``, grid ``(t, h, w)``."""
    pixel_values: torch.Tensor
    grid_thw: Tuple[int, int, int]
    first_token: int = 0                 # index of the first placeholder token in the sequence


@dataclass
class ImageInputs:
    """Device-side batch of the images of one round."""
    pixel_values: torch.Tensor
    grid_thw: torch.Tensor               # (n_images, 3)
    seq_index: List[int] = field(default_factory=list)


@dataclass
class ImageEmbeddings:
    """Encoder output rows, in placeholder order: ``(n_merged_patches, d_model)``."""
    embeds: torch.Tensor
    rows_per_image: List[int] = field(default_factory=list)


@dataclass
class ImageGradInputs:
    """Gradient w.r.t. the embeddings (unused while the encoder is frozen)."""
    d_embeds: Optional[torch.Tensor] = None


@dataclass
class InputsSummary:
    n_text_tokens: int = 0
    n_image_tokens: int = 0
    n_images: int = 0
