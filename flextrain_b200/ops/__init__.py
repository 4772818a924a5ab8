"""Op layer: one function per primitive, CUDA kernel on a B200, PyTorch fp32 oracle on CPU.

The layers in ``flextrain_b200.nn`` call only these functions, so the same model code runs the
CPU parity configuration and the sm_100a kernels.  Mirrors the role of the reference project's
``flextrain/ops/__init__.py:77-120`` export list.

Backends (``set_gemm_backend`` / ``set_attention_backend``):
  * GEMM       ``tcgen05`` (hand-written kernel, default on CUDA) | ``library`` (torch.matmul → cuBLAS)
  * attention  ``ftb`` (hand-written kernel) | ``library`` (torch's bundled flash kernels) | ``reference``
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from . import reference as ref

_GEMM_BACKEND = os.environ.get("FTB_GEMM_BACKEND", "tcgen05")
_ATTN_BACKEND = os.environ.get("FTB_ATTN_BACKEND", "auto")
_launches = 0          # number of kernels of this package launched (bench.py reports it)
_backends_used: dict = {}      # op family -> set of back ends that actually ran since the last reset


class LibraryFallback(RuntimeError):
    """Raised in strict mode (``FTB_STRICT=1``) when a hot op on a CUDA tensor would leave the hand-written
    kernels for a library call (cuBLAS through ``torch.matmul``, torch's bundled flash attention, eager PyTorch)."""


def strict() -> bool:
    return os.environ.get("FTB_STRICT", "0") == "1"


def _used(family: str, backend: str) -> None:
    _backends_used.setdefault(family, set()).add(backend)


def _fallback(family: str, why: str) -> None:
    """Record (or, in strict mode, refuse) a library / eager path taken by ``family`` on a CUDA tensor."""
    if strict():
        raise LibraryFallback(f"{family}: {why} -- no hand-written kernel takes this call (FTB_STRICT=1)")
    _used(family, "library")


def backends_used() -> dict:
    """``{family: sorted back ends that ran}`` since :func:`reset_backends_used` — what ran, not what was asked."""
    return {k: sorted(v) for k, v in sorted(_backends_used.items())}


def reset_backends_used() -> None:
    _backends_used.clear()


def set_gemm_backend(name: str) -> None:
    global _GEMM_BACKEND
    assert name in ("tcgen05", "library")
    _GEMM_BACKEND = name


def set_attention_backend(name: str) -> None:
    """``auto`` | ``ftb`` | ``library`` | ``reference`` (flextrain/ops/_kernels/attention.py:133)."""
    global _ATTN_BACKEND
    assert name in ("auto", "ftb", "library", "reference", "eager")
    _ATTN_BACKEND = "reference" if name == "eager" else name


def get_attention_backend() -> str:
    return _ATTN_BACKEND


def launch_count() -> int:
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


def _cuda_bf16(*ts) -> bool:
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts) and ts[0].is_cuda


def _kernels():
    from . import cuda
    return cuda


# ------------------------------------------------------------------------------- GEMM
def gemm(a, b, *, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None, bias=None, out=None, out_dtype=None):
    """``alpha * op(a) @ op(b) + beta * c (+ bias)``; fp32 accumulation; see ``reference.gemm``."""
    if a.is_cuda:
        od = out_dtype or (out.dtype if out is not None else a.dtype)
        k = _kernels()
        M = a.shape[1] if trans_a else a.shape[0]
        N = b.shape[0] if trans_b else b.shape[1]
        K = a.shape[0] if trans_a else a.shape[1]
        # The tensor-core kernel takes any N, K >= 8 (multiples of 8): TMA zero-fills the part of a tile that lies
        # outside the matrix, so the rank-r LoRA products (N = r or K = r) run on it too.
        why = None
        if _GEMM_BACKEND != "tcgen05":
            why = "FTB_GEMM_BACKEND=library"
        elif not k.gemm_supported(a, b, trans_a, trans_b, od):
            why = f"operands not bf16 / 16-byte aligned / N % 8 ({tuple(a.shape)}, {tuple(b.shape)}, {a.dtype})"
        elif N < 8 or K < 8 or M < 1:
            why = f"N={N} or K={K} below 8"
        elif out is not None and not (out.stride(-1) == 1 and out.data_ptr() % 16 == 0):
            why = "output not row-contiguous / 16-byte aligned"
        elif bias is not None and bias.dtype != torch.float32:
            why = "bias not fp32"
        if why is None:
            _count()
            _used("gemm", "tcgen05")
            return k.gemm(a, b, trans_a=trans_a, trans_b=trans_b, alpha=alpha, beta=beta, c=c, bias=bias, out=out,
                          out_dtype=od)
        _fallback("gemm", why)
        # library GEMM for shapes the tensor-core kernel does not take (odd strides, N or K not a multiple of 8)
        A = a.t() if trans_a else a
        B = b.t() if trans_b else b
        if od == a.dtype and b.dtype == a.dtype:
            d = torch.matmul(A, B)
            if alpha != 1.0:
                d = d * alpha
        else:
            d = torch.matmul(A.to(torch.float32), B.to(torch.float32)) * alpha
        if beta != 0.0:
            src = c if c is not None else out
            d = d.to(torch.float32) + beta * src.to(torch.float32)
        if bias is not None:
            d = d + bias
        if out is not None:
            out.copy_(d)
            return out
        return d.to(od)
    return ref.gemm(a, b, trans_a=trans_a, trans_b=trans_b, alpha=alpha, beta=beta, c=c, bias=bias, out=out,
                    out_dtype=out_dtype)


def linear_fwd(x, w, *, bias=None, residual=None, out=None):
    """``y = x @ w.T (+ bias) (+ residual)`` with ``w (out, in)``; residual add fused in the epilogue."""
    if residual is not None:
        return gemm(x, w, trans_b=True, beta=1.0, c=residual, bias=bias, out=out)
    return gemm(x, w, trans_b=True, bias=bias, out=out)


def linear_dgrad(dy, w, *, out=None, accumulate=False):
    """``dx = dy @ w`` (``w (out, in)``), optionally accumulated into ``out``."""
    return gemm(dy, w, beta=1.0 if accumulate else 0.0, out=out)


def linear_wgrad(dy, x, gw, *, alpha=1.0, accumulate=True):
    """``gw (out, in) (+)= alpha * dy.T @ x`` in the gradient's dtype (bf16 or fp32)."""
    return gemm(dy, x, trans_a=True, alpha=alpha, beta=1.0 if accumulate else 0.0, out=gw)


def bias_grad(dy, gb, *, alpha=1.0, accumulate=True):
    s = dy.to(torch.float32).sum(0) * alpha
    if accumulate:
        gb.add_(s.to(gb.dtype))
    else:
        gb.copy_(s)


# --------------------------------------------------------------------------- norms / rope / glu
def rmsnorm_fwd(x, w, eps):
    if _cuda_bf16(x) and (w is None or w.dtype == torch.float32):
        _count()
        return _kernels().rmsnorm_fwd(x.contiguous(), w, eps)
    return ref.rmsnorm_fwd(x, w, eps)


def rmsnorm_bwd(dy, x, w, rstd, *, dx_add=None, emit_y=False, dw_out=None):
    """Returns ``(dx, y)``; ``dw`` is accumulated into ``dw_out`` (fp32 or grad dtype)."""
    if _cuda_bf16(dy, x) and (w is None or w.dtype == torch.float32) and (dw_out is None or dw_out.dtype == torch.float32):
        _count(2)
        dx, _, y = _kernels().rmsnorm_bwd(dy.contiguous(), x.contiguous(), w, rstd.contiguous(), dx_add=dx_add,
                                          emit_y=emit_y, dw_out=dw_out)
        return dx, y
    dx, dw = ref.rmsnorm_bwd(dy, x, w, rstd)
    if dx_add is not None:
        dx = (dx.to(torch.float32) + dx_add.to(torch.float32)).to(dx.dtype)
    if dw_out is not None and dw is not None:
        dw_out.add_(dw.reshape(dw_out.shape).to(dw_out.dtype))
    y = ref.rmsnorm_fwd(x, w, 0.0)[0] if False else None
    if emit_y:
        xf = x.to(torch.float32) * rstd.unsqueeze(-1)
        y = (xf * w.to(torch.float32) if w is not None else xf).to(x.dtype)
    return dx, y


def rope(x, positions, inv_freq, *, out=None, inverse=False, mrope_sections=None):
    """RoPE on ``x (T,H,hd)`` (token-strided views allowed) written to ``out`` (in place when None)."""
    if _cuda_bf16(x) and x.stride(2) == 1 and x.stride(1) == x.shape[2] and \
            (out is None or (out.stride(2) == 1 and out.stride(1) == out.shape[2])):
        _count()
        return _kernels().rope(x, positions.to(torch.int32).contiguous(), inv_freq, out=out, inverse=inverse,
                               mrope_sections=mrope_sections)
    y = ref.rope_apply(x, positions, inv_freq, inverse=inverse, mrope_sections=mrope_sections)
    if out is None:
        x.copy_(y)
        return x
    out.copy_(y)
    return out


def glu_fwd(gate, up, kind="swiglu"):
    if _cuda_bf16(gate, up):
        _count()
        return _kernels().glu_fwd(gate, up, kind)
    return ref.glu_fwd(gate, up, kind)


def glu_bwd(dact, gate, up, kind="swiglu", *, dgate=None, dup=None):
    """Returns ``(dgate, dup, act)``."""
    if _cuda_bf16(dact, gate, up):
        _count()
        return _kernels().glu_bwd(dact, gate, up, kind, dgate=dgate, dup=dup)
    dg, du, act = ref.glu_bwd(dact, gate, up, kind)
    if dgate is not None:
        dgate.copy_(dg); dup.copy_(du)
        return dgate, dup, act
    return dg, du, act


_GLU_FUSED = os.environ.get("FTB_GLU_FUSED", "1") == "1"


def gemm_glu_fwd(x, w13, kind="swiglu", *, x13=None):
    """The fused kernel itself (GPU only); ``linear_glu_fwd`` is the entry that falls back."""
    return _kernels().gemm_glu_fwd(x, w13, kind, x13=x13)


def gemm_glu_bwd(dy, w2, x13, kind="swiglu"):
    return _kernels().gemm_glu_bwd(dy, w2, x13, kind)


def _glu_fused_ok(x, w, F: int) -> bool:
    if not (_GLU_FUSED and _cuda_bf16(x, w)):
        return False
    from . import cuda
    return cuda.have("gemm_tcgen05") and cuda.gemm_glu_supported(x, w, F)


def linear_glu_fwd(x, w13, kind="swiglu", *, x13=None):
    """Gated-FFN up projection and activation: ``x13 = x @ w13^T`` (``w13 = [W_gate ; W_up]``), ``act = act_fn(gate) * up``.
    On the GPU both come out of ONE two-SM tcgen05 GEMM (the activation is computed in the epilogue from the tile
    that is being stored); elsewhere, or for shapes the kernel does not take, a GEMM followed by the activation pass.
    Returns ``(x13, act)``."""
    F = w13.shape[0] // 2
    if _glu_fused_ok(x, w13, F):
        _count()
        _used("linear_glu_fwd", "ftb")
        return gemm_glu_fwd(x, w13, kind, x13=x13)
    x13 = linear_fwd(x, w13, out=x13)
    return x13, glu_fwd(x13[:, :F], x13[:, F:], kind)


def linear_glu_bwd(dy, w2, x13, kind="swiglu"):
    """Backward of ``y = act(x13) @ w2^T`` down to ``x13``: returns ``(dx13 = [dgate | dup], act)``; ``act`` is re-emitted
    for the down projection's weight gradient.  One fused GEMM on the GPU (``dact`` never reaches memory)."""
    F = w2.shape[1]
    if _glu_fused_ok(dy, w2, F) and x13.stride(1) == 1 and x13.stride(0) % 8 == 0 and x13.data_ptr() % 16 == 0:
        _count()
        _used("linear_glu_bwd", "ftb")
        return gemm_glu_bwd(dy, w2, x13, kind)
    dact = linear_dgrad(dy, w2)
    dx13 = torch.empty_like(x13)
    _, _, act = glu_bwd(dact, x13[:, :F], x13[:, F:], kind, dgate=dx13[:, :F], dup=dx13[:, F:])
    return dx13, act


def glu_bwd_weighted(dact_u, gate, up, w_row, kind="swiglu", *, dgate, dup):
    """Expert backward through the gated activation with the router weight folded in (one pass):
    ``dgate, dup`` from ``w_row * dact_u``; returns ``(act_w = w_row * act, dw_row = sum(dact_u * act, -1))``."""
    if _cuda_bf16(dact_u, gate, up) and dact_u.is_contiguous():
        _count()
        return _kernels().glu_bwd_weighted(dact_u, gate, up, w_row.to(torch.float32).contiguous(), kind,
                                           dgate=dgate, dup=dup)
    wcol = w_row.to(torch.float32).unsqueeze(-1)
    dactw = (dact_u.to(torch.float32) * wcol).to(dact_u.dtype)
    _, _, act = glu_bwd(dactw, gate, up, kind, dgate=dgate, dup=dup)
    dw_row = (dact_u.to(torch.float32) * act.to(torch.float32)).sum(-1)
    return (act.to(torch.float32) * wcol).to(act.dtype), dw_row


# -------------------------------------------------------------------------- attention
def _attn_backend_for(q) -> str:
    if not q.is_cuda or q.dtype not in (torch.bfloat16, torch.float16):
        return "reference"
    if _ATTN_BACKEND == "auto":
        from . import cuda
        return "ftb" if cuda.have("attention") and q.shape[-1] in (64, 128) else "library"
    return _ATTN_BACKEND


def attention_fwd(q, k, v, cu_q, cu_k, max_q, max_k, *, scale, causal=True, window=0, softcap=0.0):
    """Varlen GQA attention, bottom-right aligned causal. Returns ``(out (Tq,H,hd), lse (H,Tq) fp32)``."""
    be = _attn_backend_for(q)
    if be == "ftb":
        from . import attention_cuda
        _count()
        _used("attention_fwd", "ftb")
        return attention_cuda.fwd(q, k, v, cu_q, cu_k, max_q, max_k, scale=scale, causal=causal, window=window,
                                  softcap=softcap)
    if q.is_cuda:
        _fallback("attention_fwd", f"backend {be}, head_dim {q.shape[-1]}, dtype {q.dtype}")
    if be in ("library", "ftb") and not softcap:
        wl = (window - 1) if window and window > 0 else None
        o, lse, _, _, _ = torch.ops.aten._flash_attention_forward(
            q, k, v, cu_q.to(torch.int32), cu_k.to(torch.int32), max_q, max_k, 0.0, causal, False, scale=scale,
            window_size_left=wl, window_size_right=0 if (wl is not None) else None)
        return o, lse
    return ref.attention_fwd(q, k, v, cu_q, cu_k, scale=scale, causal=causal, window=window, softcap=softcap)


def attention_bwd(dout, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, *, scale, causal=True, window=0, softcap=0.0):
    """Returns ``(dq, dk, dv)``; dk/dv span all visible keys."""
    be = _attn_backend_for(q)
    if be == "ftb" and hasattr(_kernels().load("attention"), "ftb_attn_bwd"):
        from . import attention_cuda
        _count(3)
        _used("attention_bwd", "ftb")
        return attention_cuda.bwd(dout, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, scale=scale, causal=causal,
                                  window=window, softcap=softcap)
    if q.is_cuda:
        _fallback("attention_bwd", f"backend {be}, head_dim {q.shape[-1]}, dtype {q.dtype}")
    if be in ("library", "ftb") and not softcap:
        wl = (window - 1) if window and window > 0 else None
        rng = torch.zeros(2, dtype=torch.uint64, device=q.device)
        unused = torch.empty(0, device=q.device)
        dq, dk, dv = torch.ops.aten._flash_attention_backward(
            dout, q, k, v, out, lse, cu_q.to(torch.int32), cu_k.to(torch.int32), max_q, max_k, 0.0, causal, rng, unused,
            scale=scale, window_size_left=wl, window_size_right=0 if (wl is not None) else None)
        return dq, dk, dv
    return ref.attention_bwd(dout, q, k, v, out, lse, cu_q, cu_k, scale=scale, causal=causal, window=window,
                             softcap=softcap)


# ---------------------------------------------------------------------- loss / embed
def softmax_ce_(logits, targets, *, grad_scale=1.0, softcap=0.0, loss_mask=None, ignore_index=-100):
    """Fused softmax-CE: returns per-token loss; ``logits`` is overwritten with dlogits."""
    if _cuda_bf16(logits) and logits.stride(1) == 1:
        _count()
        return _kernels().softmax_ce_(logits, targets.to(torch.int64), grad_scale=grad_scale, softcap=softcap,
                                      loss_mask=loss_mask, ignore_index=ignore_index)
    loss, dz = ref.softmax_ce_fwd_bwd(logits, targets, grad_scale=grad_scale, softcap=softcap, loss_mask=loss_mask,
                                      ignore_index=ignore_index)
    logits.copy_(dz)
    return loss


def embedding_fwd(tokens, table, scale=1.0):
    if _cuda_bf16(table) and table.shape[1] % 8 == 0:
        _count()
        return _kernels().embedding_fwd(tokens.to(torch.int64).contiguous(), table, scale)
    return ref.embedding_fwd(tokens, table, scale)


def embedding_bwd(dy, tokens, grad_table, scale=1.0):
    if dy.is_cuda and dy.dtype == torch.bfloat16 and grad_table.dtype in (torch.bfloat16, torch.float32) \
            and grad_table.shape[1] % 8 == 0:
        _count()
        return _kernels().embedding_bwd(dy.contiguous(), tokens.to(torch.int64).contiguous(), grad_table, scale)
    return ref.embedding_bwd(dy, tokens, grad_table, scale)


# ------------------------------------------------------------------------- optimizers
def adamw_multi(params, grads, ms, vs, *, lrs, wds, beta1, beta2, eps, step, grad_scale=1.0):
    """Fused AdamW over a list of tensors (one launch per layer on CUDA)."""
    ok = all(p.is_cuda and p.is_contiguous() and g.is_contiguous() and p.dtype in (torch.bfloat16, torch.float32)
             and g.dtype in (torch.bfloat16, torch.float32) and m.dtype in (torch.bfloat16, torch.float32)
             and m.dtype == v.dtype for p, g, m, v in zip(params, grads, ms, vs))
    if ok and params:
        _count((len(params) + 23) // 24)
        return _kernels().adamw_multi(params, grads, ms, vs, lrs=list(lrs), wds=list(wds), beta1=beta1, beta2=beta2,
                                      eps=eps, step=step, grad_scale=grad_scale)
    for p, g, m, v, lr, wd in zip(params, grads, ms, vs, lrs, wds):
        ref.adamw_step(p, g, m, v, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=wd, step=step,
                       grad_scale=grad_scale)


def newton_schulz_bf16(u: torch.Tensor, iters: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation of one matrix on the tcgen05 GEMM, bf16 iterates with fp32
    accumulation: per iteration ``A = X Xᵀ``, ``B = bA + cA²`` (epilogue ``alpha=c, beta=b``), ``X = aX + BX``
    (epilogue ``beta=a``) — three launches, no elementwise pass (flextrain/ops/_kernels/muon.py:53-61 issues
    mm / addmm through cuBLAS).  A tall matrix is iterated as ``AᵀA`` on the right, so nothing is transposed."""
    a, b, c = ref.NS_COEFFS
    x = (u / (u.norm() + 1e-7)).to(torch.bfloat16).contiguous()
    tall = x.shape[0] > x.shape[1]
    for _ in range(iters):
        if not tall:
            A = gemm(x, x, trans_b=True)                       # (m, m)
            B = gemm(A, A, alpha=c, beta=b, c=A)
            x = gemm(B, x, beta=a, c=x)
        else:
            A = gemm(x, x, trans_a=True)                       # (n, n) = XᵀX
            B = gemm(A, A, alpha=c, beta=b, c=A)
            x = gemm(x, B, beta=a, c=x)
    return x


def muon_step(p, g, mom, *, lr, beta=0.95, weight_decay=0.0, ns_iters=5, nesterov=True, grad_scale=1.0):
    """Muon update (flextrain/ops/_kernels/muon.py:16-75).  On CUDA bf16 the Newton-Schulz GEMMs run on the
    tcgen05 kernel; 3-D tensors (stacked experts) are updated matrix by matrix."""
    if not (_cuda_bf16(p) and _GEMM_BACKEND == "tcgen05" and p.dim() in (2, 3) and min(p.shape[-2:]) >= 64
            and p.shape[-1] % 8 == 0 and p.shape[-2] % 8 == 0):
        return ref.muon_step(p, g, mom, lr=lr, beta=beta, weight_decay=weight_decay, ns_iters=ns_iters,
                             nesterov=nesterov, grad_scale=grad_scale)
    gf = g.to(torch.float32) * grad_scale
    mf = beta * mom.to(torch.float32) + gf
    mom.copy_(mf.to(mom.dtype))
    u = gf + beta * mf if nesterov else mf
    scale = 0.2 * math.sqrt(max(p.shape[-2], p.shape[-1]))
    mats = [(p, u)] if p.dim() == 2 else [(p[i], u[i]) for i in range(p.shape[0])]
    for pm, um in mats:
        x = newton_schulz_bf16(um, ns_iters)
        pm.copy_((pm.to(torch.float32) * (1.0 - lr * weight_decay) - (lr * scale) * x.to(torch.float32)).to(pm.dtype))


# -------------------------------------------------------------------------------- MoE
def topk_route(logits, k, mode="topk_then_softmax"):
    if _cuda_bf16(logits) and logits.shape[1] <= 256 and k <= 16:
        _count()
        return _kernels().topk_route(logits, k, mode)
    return ref.topk_route(logits, k, mode)


def topk_route_bwd(dw, logits, w, experts, mode="topk_then_softmax"):
    """dlogits (T, E) fp32 from the gradient of the selected routing weights."""
    if _cuda_bf16(logits) and logits.shape[1] <= 256 and experts.shape[1] <= 32:
        _count()
        return _kernels().topk_route_bwd(dw, logits, w, experts, mode)
    return ref.topk_route_bwd(dw, logits, w, experts, mode)


moe_sort = ref.moe_sort


def load_balance_bwd_(dlogits, logits, experts, alpha: float, total_tokens_per_step: int, counts=None):
    """Add the load-balance auxiliary gradient into ``dlogits (T, E)`` fp32 in place:
    ``alpha * p * (gvec - sum(p * gvec))`` with ``p = softmax(logits)`` and ``gvec = counts / n_slots * E / total_tokens``
    (flextrain/ops/_kernels/moe.py:601-646); ``counts`` are the per-expert slot counts of this chunk."""
    T, E = logits.shape
    n = experts.numel()
    if _cuda_bf16(logits) and E <= 256 and dlogits.dtype == torch.float32 and dlogits.is_contiguous():
        if counts is None:
            counts = torch.bincount(experts.reshape(-1).long(), minlength=E)
        _count()
        return _kernels().load_balance_bwd_(dlogits, logits.contiguous(), counts.to(torch.int32).contiguous(),
                                            float(alpha), float(E) / max(n, 1) / float(total_tokens_per_step))
    p = torch.softmax(logits.to(torch.float32), -1)
    f = torch.zeros(E, dtype=torch.float32, device=logits.device).index_add_(
        0, experts.reshape(-1).long(), torch.ones(n, dtype=torch.float32, device=logits.device))
    gvec = f / max(n, 1) * E / total_tokens_per_step
    dlogits += alpha * p * (gvec - (p * gvec).sum(-1, keepdim=True))
    return dlogits


def moe_plan(experts, num_experts: int, pad: int = 1):
    """Expert-major row layout of one chunk's routed slots (``reference.MoEPlan``): a stable counting sort by expert
    with every expert's segment padded to ``pad`` rows.  On CUDA three small kernels build it without a host read
    and without the library sort (flextrain/ops/_kernels/moe.py:318-357,461-505 plus the host sync of
    flextrain/ops/full_moe.py:134-148 in the reference)."""
    if experts.is_cuda and num_experts <= 1024:
        T, K = experts.shape
        R = ref.moe_rows_bound(T, K, num_experts, pad)
        _count(3)
        _used("moe_plan", "ftb")
        row_src, inv, offsets, counts = _kernels().moe_plan(experts, num_experts, pad, R)
        return ref.MoEPlan(row_src, inv, offsets, R, counts)
    if experts.is_cuda:
        _fallback("moe_plan", f"{num_experts} experts (the plan kernels take up to 1024)")
    return ref.moe_plan(experts, num_experts, pad)


def gather_rows(x, idx, weights=None, idx_div=1):
    """``out[i] = x[idx[i] // idx_div] * weights[i]``."""
    if _cuda_bf16(x) and x.shape[1] % 8 == 0 and x.is_contiguous():
        _count()
        return _kernels().gather_rows(x, idx.to(torch.int32).contiguous(), weights, idx_div)
    src = idx.long()
    y = x[(src.clamp(min=0) // idx_div)] * (src >= 0).unsqueeze(-1).to(x.dtype)
    if weights is not None:
        y = (y.to(torch.float32) * weights.unsqueeze(-1)).to(x.dtype)
    return y


def moe_combine(y, inv, weights, resid):
    """``out[t] = resid[t] + sum_k weights[t,k] * y[inv[t,k]]`` in fp32."""
    if _cuda_bf16(y) and y.shape[1] % 8 == 0 and y.is_contiguous():
        _count()
        return _kernels().moe_combine(y, inv.to(torch.int32).contiguous(), weights, resid)
    g = y[inv.long()].to(torch.float32)                       # (T,K,D)
    if weights is not None:
        g = g * weights.unsqueeze(-1)
    out = g.sum(1)
    if resid is not None:
        out = out + resid.to(torch.float32)
    return out.to(y.dtype)


def grouped_gemm(x, w, offsets, *, trans_w=True, out=None, alpha=1.0, beta=0.0):
    """``out[rows_e] = alpha * x[rows_e] @ op(w[e]) + beta * out[rows_e]`` for every expert in one launch."""
    if x.is_cuda:
        why = None
        if not (_cuda_bf16(x, w) and _GEMM_BACKEND == "tcgen05"):
            why = "operands not bf16 or FTB_GEMM_BACKEND=library"
        elif x.shape[1] % 8 or x.shape[1] < 8 or not w.is_contiguous() or (w.shape[1] if trans_w else w.shape[2]) % 8:
            why = f"K or N not a multiple of 8 ({tuple(x.shape)}, {tuple(w.shape)})"
        if why is None:
            _count()
            _used("grouped_gemm", "tcgen05")
            return _kernels().grouped_gemm(x if x.stride(1) == 1 else x.contiguous(), w, offsets.to(torch.int32),
                                           trans_w=trans_w, out=out, alpha=alpha, beta=beta)
        _fallback("grouped_gemm", why)
    y = ref.grouped_gemm(x, w, offsets, trans_w=trans_w)
    if alpha != 1.0:
        y = (y.to(torch.float32) * alpha).to(y.dtype)
    if out is not None:
        if beta != 0.0:
            rows = int(offsets[-1])
            out[:rows] = (beta * out[:rows].to(torch.float32) + y[:rows].to(torch.float32)).to(out.dtype)
        else:
            out.copy_(y)
        return out
    return y


def grouped_wgrad(dy, x, offsets, gw, *, alpha=1.0, pad: int = 1):
    """``gw[e] += alpha * dy[rows_e].T @ x[rows_e]``. On CUDA one tcgen05 launch covers all experts; it needs every
    expert's row segment padded to a multiple of 64 with zero rows (``pad``), which the MoE dispatch plan provides."""
    if (_cuda_bf16(dy, x) and _GEMM_BACKEND == "tcgen05" and pad % 64 == 0 and gw.is_contiguous()
            and gw.dtype in (torch.bfloat16, torch.float32) and dy.shape[1] % 8 == 0 and x.shape[1] % 8 == 0
            and dy.stride(1) == 1 and x.stride(1) == 1 and dy.stride(0) % 8 == 0 and x.stride(0) % 8 == 0):
        _count()
        _used("grouped_wgrad", "tcgen05")
        return _kernels().grouped_wgrad(dy, x, offsets.to(torch.int32), gw, alpha=alpha)
    if dy.is_cuda:
        _fallback("grouped_wgrad", f"dtype / stride / padding not supported ({tuple(dy.shape)}, {tuple(x.shape)}, pad {pad})")
    return ref.grouped_wgrad(dy, x, offsets, gw, alpha=alpha)


# ---------------------------------------------------------------------- linear attention
def l2norm_fwd(x, eps=1e-6):
    if _cuda_bf16(x) and x.is_contiguous():
        _count()
        return _kernels().l2norm_fwd(x, eps)
    return ref.l2norm_fwd(x, eps)


l2norm_bwd = ref.l2norm_bwd


def gated_rmsnorm_fwd(o, z, w, eps):
    if _cuda_bf16(o, z) and w.dtype == torch.float32 and o.is_contiguous() and z.is_contiguous():
        _count()
        return _kernels().gated_rmsnorm_fwd(o, z, w, eps)
    return ref.gated_rmsnorm_fwd(o, z, w, eps)


causal_conv1d_fwd = ref.causal_conv1d_fwd
gated_delta_rule = ref.gated_delta_rule
gated_delta_rule_chunked = ref.gated_delta_rule_chunked
def top_p_sample(logits, top_p, temperature, generator=None):
    """Nucleus sampling per row (flextrain/ops/_kernels/sample_top_p.py:7-150)."""
    if _cuda_bf16(logits):
        from . import linattn_cuda
        _count()
        return linattn_cuda.top_p_sample(logits, top_p, temperature, generator=generator)
    return ref.top_p_sample(logits, top_p, temperature, generator=generator)


rope_inv_freq = ref.rope_inv_freq


# ------------------------------------------------------------------ per-op device timing
# ``FTB_OP_TIMING=1`` brackets every leaf op of this module with CUDA events on the current stream and
# ``timing_report()`` aggregates them by (op, shape): the per-kernel time table of a training step without a
# profiler attached.  The events add host work, so a throughput number taken with it on is not a benchmark value.
_TIMED_OPS = ("gemm", "gemm_glu_fwd", "gemm_glu_bwd", "rmsnorm_fwd", "rmsnorm_bwd", "rope", "glu_fwd", "glu_bwd", "glu_bwd_weighted", "attention_fwd",
              "attention_bwd", "softmax_ce_", "embedding_fwd", "embedding_bwd", "adamw_multi", "topk_route",
              "topk_route_bwd", "gather_rows", "moe_combine", "grouped_gemm", "grouped_wgrad", "l2norm_fwd",
              "gated_rmsnorm_fwd", "bias_grad")
_timing_events: list = []


def _timing_key(name, args, kwargs):
    if name == "gemm":
        a, b = args[0], args[1]
        ta, tb = kwargs.get("trans_a", False), kwargs.get("trans_b", False)
        M = a.shape[1] if ta else a.shape[0]
        K = a.shape[0] if ta else a.shape[1]
        N = b.shape[0] if tb else b.shape[1]
        lay = ("T" if ta else "N") + ("T" if tb else "N")
        od = kwargs.get("out_dtype") or (kwargs["out"].dtype if kwargs.get("out") is not None else a.dtype)
        return f"{M}x{N}x{K} {lay}" + (" +C" if kwargs.get("beta", 0.0) else "") + (" f32" if od == torch.float32 else "")
    for v in list(args) + list(kwargs.values()):
        if isinstance(v, torch.Tensor):
            return "x".join(str(s) for s in v.shape)
        if isinstance(v, (list, tuple)) and v and isinstance(v[0], torch.Tensor):
            return f"{len(v)} tensors, {sum(t.numel() for t in v)} elements"
    return ""


def _timed(name, fn):
    def wrapper(*args, **kwargs):
        first = next((v for v in args if isinstance(v, torch.Tensor)), None)
        if first is None and args and isinstance(args[0], (list, tuple)) and args[0]:
            first = args[0][0]
        if first is None or not first.is_cuda:
            return fn(*args, **kwargs)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*args, **kwargs)
        e1.record()
        _timing_events.append((name, _timing_key(name, args, kwargs), e0, e1))
        return out
    wrapper.__name__ = fn.__name__
    wrapper.__doc__ = fn.__doc__
    return wrapper


def enable_op_timing() -> None:
    g = globals()
    for n in _TIMED_OPS:
        if not getattr(g[n], "_ftb_timed", False):
            g[n] = _timed(n, g[n])
            g[n]._ftb_timed = True


def reset_op_timing() -> None:
    _timing_events.clear()


def timing_report() -> list:
    """``[{op, shape, calls, total_ms, mean_us, share}]`` sorted by total time; synchronises the device."""
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    agg: dict = {}
    for name, key, e0, e1 in _timing_events:
        ms = e0.elapsed_time(e1)
        c = agg.setdefault((name, key), [0, 0.0])
        c[0] += 1
        c[1] += ms
    total = sum(v[1] for v in agg.values()) or 1.0
    rows = [{"op": k[0], "shape": k[1], "calls": v[0], "total_ms": v[1], "mean_us": 1e3 * v[1] / v[0],
             "share": v[1] / total} for k, v in agg.items()]
    return sorted(rows, key=lambda r: -r["total_ms"])


if os.environ.get("FTB_OP_TIMING", "0") == "1":
    enable_op_timing()
