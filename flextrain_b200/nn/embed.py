"""Token embedding input layer: gather forward (optional Gemma ``sqrt(d)`` scale), sorted
scatter-add backward (flextrain/nn/embed.py:67-169)."""
from __future__ import annotations

import torch

from .. import ops
from ..core.layer import ChunkMeta, ParamSpec, TensorSpec


class TokenEmbedLayer:
    def __init__(self, vocab_size: int, d_model: int, *, dtype=torch.bfloat16, grad_dtype=None, master_dtype=None,
                 scale: float = 1.0, frozen: bool = False):
        self.vocab_size, self.d_model, self.scale = vocab_size, d_model, scale
        self.param_spec = ParamSpec([TensorSpec("w_tok_embeddings", (vocab_size, d_model), dtype,
                                                master_dtype=master_dtype, grad_dtype=grad_dtype, frozen=frozen,
                                                optimizer="adamw")])

    def forward(self, meta: ChunkMeta, params) -> torch.Tensor:
        return ops.embedding_fwd(meta.tokens, params["w_tok_embeddings"], self.scale)

    def backward(self, dx, meta: ChunkMeta, params, grads) -> None:
        g = grads.get("g_tok_embeddings")
        if g is not None:
            ops.embedding_bwd(dx, meta.tokens, g, self.scale)
