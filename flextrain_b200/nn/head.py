"""LM head with fused forward + loss + backward per micro-chunk (flextrain/nn/head.py:155-393).

Per ``head_chunk_size`` tokens: RMSNorm → logits GEMM → loss (logits become ``dZ`` in place,
``loss_scale`` folded in) → ``g_head_proj += dZᵀ·h`` → ``dh = dZ·W`` → RMSNorm backward; the input
buffer is overwritten with ``dx``.  ``(T, V)`` is never materialised beyond one micro-chunk.
"""
from __future__ import annotations


import torch

from .. import ops
from ..core.layer import ChunkMeta, LossStats, ParamSpec, TensorSpec
from .loss import CrossEntropyLoss, TokenSlice, apply_loss


class LMHead:
    def __init__(self, vocab_size: int, d_model: int, *, dtype=torch.bfloat16, norm_dtype=torch.float32,
                 grad_dtype=None, master_dtype=None, norm_eps: float = 1e-5, head_chunk_size: int = 4096,
                 final_softcap: float = 0.0, frozen: bool = False, tied: bool = False):
        self.vocab_size, self.d_model, self.norm_eps = vocab_size, d_model, norm_eps
        self.head_chunk_size = head_chunk_size
        self.final_softcap = final_softcap
        self.tied = tied
        self.param_spec = ParamSpec([
            TensorSpec("w_final_norm", (d_model,), norm_dtype, master_dtype=norm_dtype, grad_dtype=torch.float32,
                       init="ones", frozen=frozen),
            TensorSpec("w_head_proj", (vocab_size, d_model), dtype, master_dtype=master_dtype, grad_dtype=grad_dtype,
                       frozen=frozen, optimizer="adamw"),
        ])

    def forward_backward(self, x: torch.Tensor, meta: ChunkMeta, params, grads, loss_fn=None,
                         loss_scale: float = 1.0, *, want_dx: bool = True) -> LossStats:
        loss_fn = loss_fn or CrossEntropyLoss()
        T = x.shape[0]
        W = params["w_head_proj"]
        per_tok = torch.empty(T, dtype=torch.float32, device=x.device)
        gW = grads.get("g_head_proj")
        for a in range(0, T, self.head_chunk_size):
            b = min(T, a + self.head_chunk_size)
            xa = x[a:b]
            hn, rstd = ops.rmsnorm_fwd(xa, params["w_final_norm"], self.norm_eps)
            logits = ops.gemm(hn, W, trans_b=True)
            sl = TokenSlice(meta.targets[a:b], meta.loss_mask[a:b] if meta.loss_mask is not None else None,
                            meta.extra.get("advantages")[a:b] if meta.extra.get("advantages") is not None else None,
                            meta.extra.get("ref_logprobs")[a:b] if meta.extra.get("ref_logprobs") is not None else None)
            per_tok[a:b] = apply_loss(loss_fn, logits, sl, loss_scale, self.final_softcap)
            if gW is not None:
                ops.gemm(logits, hn, trans_a=True, beta=1.0, out=gW)
            if want_dx:
                dhn = ops.gemm(logits, W)
                dxa, _ = ops.rmsnorm_bwd(dhn, xa, params["w_final_norm"], rstd, dw_out=grads.get("g_final_norm"))
                x[a:b].copy_(dxa)
        active = (meta.targets != -100)
        if meta.loss_mask is not None:
            active = active & (meta.loss_mask > 0)
        return LossStats(total_loss=per_tok.sum(), active_tokens=active.sum(), per_token_loss=per_tok)

    @torch.no_grad()
    def logits(self, x: torch.Tensor, params) -> torch.Tensor:
        """Inference-only logits (generation / parity checks)."""
        hn, _ = ops.rmsnorm_fwd(x, params["w_final_norm"], self.norm_eps)
        z = ops.gemm(hn, params["w_head_proj"], trans_b=True)
        if self.final_softcap > 0:
            z = (self.final_softcap * torch.tanh(z.to(torch.float32) / self.final_softcap)).to(z.dtype)
        return z
