"""Pure-PyTorch fp32 oracle for every op in the framework.

These functions are (a) the CPU execution path, (b) the numerical reference that
every CUDA kernel test compares against.  They compute in fp32 internally and
return tensors in the dtype of their inputs.  Conventions:

* Linear weights are stored ``(out_features, in_features)`` (the HuggingFace /
  ``nn.Linear`` convention), so ``y = x @ w.T``.  The reference project stores
  ``(in, out)`` and transposes on load (flextrain/io/hf_weights.py:44-52); keeping
  the on-disk layout removes that transpose and makes the forward GEMM operands
  both K-major for the tensor cores.
* RoPE uses the HuggingFace "rotate-half" channel pairing ``(i, i + rot/2)``.
  The reference permutes Q/K rows to a pair-interleaved layout on load
  (flextrain/io/arch/llama.py:326-366); attention scores are invariant under
  that permutation, so we keep the checkpoint layout and need no permutation.
* Attention is varlen, causal and *bottom-right aligned*: the ``Lq`` queries of
  a sequence are the last ``Lq`` positions of its ``Lk`` keys, which is what a
  chunk of a long sequence sees (prior chunks' K/V precede its own)
  (flextrain/ops/_kernels/attention.py:431-621).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

F32 = torch.float32


# --------------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = False,
         alpha: float = 1.0, beta: float = 0.0, c: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``D = alpha * op(A) @ op(B) + beta * C (+ bias)`` with fp32 accumulation."""
    A = a.to(F32).t() if trans_a else a.to(F32)
    B = b.to(F32).t() if trans_b else b.to(F32)
    d = alpha * (A @ B)
    if beta != 0.0:
        src = c if c is not None else out
        d = d + beta * src.to(F32)
    if bias is not None:
        d = d + bias.to(F32)
    dt = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is not None:
        out.copy_(d.to(out.dtype))
        return out
    return d.to(dt)


# ------------------------------------------------------------------------ RMSNorm
def rmsnorm_fwd(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Row RMSNorm over the last dim. Returns ``(y, rstd)`` with ``rstd`` fp32 of shape ``x.shape[:-1]``."""
    xf = x.to(F32)
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1) + eps)
    y = xf * rstd.unsqueeze(-1)
    if w is not None:
        y = y * w.to(F32)
    return y.to(x.dtype), rstd


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: Optional[torch.Tensor], rstd: torch.Tensor,
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns ``(dx, dw_fp32)``; ``dw`` is summed over all leading dims."""
    xf, dyf = x.to(F32), dy.to(F32)
    n = x.shape[-1]
    xhat = xf * rstd.unsqueeze(-1)
    g = dyf * w.to(F32) if w is not None else dyf
    dot = (g * xhat).sum(dim=-1, keepdim=True)
    dx = (g - xhat * dot / n) * rstd.unsqueeze(-1)
    dw = None
    if w is not None:
        dw = (dyf * xhat).reshape(-1, n).sum(dim=0)
    return dx.to(x.dtype), dw


# --------------------------------------------------------------------------- RoPE
def rope_inv_freq(head_dim: int, theta: float, *, rotary_dim: Optional[int] = None,
                  scaling: Optional[dict] = None) -> torch.Tensor:
    """Inverse frequencies (fp32, length ``rotary_dim // 2``).

    ``scaling`` follows HuggingFace ``rope_scaling``: ``{"rope_type": "linear",
    "factor": f}``, ``{"rope_type": "llama3", factor, low_freq_factor,
    high_freq_factor, original_max_position_embeddings}``, or
    ``{"rope_type": "proportional", "partial_rotary_factor": p}`` where the
    rotation angles are laid out over the full head and the tail is zero-angle
    (flextrain/nn/blocks/rope.py:28-104,141-205).
    """
    rot = rotary_dim or head_dim
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type", "default"))
    if kind == "proportional":
        p = float(scaling.get("partial_rotary_factor", 1.0))
        n_rot = int(head_dim * p) // 2
        inv = torch.zeros(head_dim // 2, dtype=F32)
        idx = torch.arange(0, 2 * n_rot, 2, dtype=F32)
        inv[:n_rot] = 1.0 / (theta ** (idx / head_dim))
        return inv
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=F32) / rot))
    if kind == "linear":
        inv = inv / float(scaling["factor"])
    elif kind == "llama3":
        factor = float(scaling["factor"])
        lo = float(scaling.get("low_freq_factor", 1.0))
        hi = float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        smooth = (old / wavelen - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor, inv)
        mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        inv = torch.where(mid, (1 - smooth) * inv / factor + smooth * inv, scaled)
    return inv


def _rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor,
                 mrope_sections: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Angles ``(T, rot/2)``. ``positions`` is ``(T,)`` or ``(T, 3)`` for MRoPE.

    MRoPE (interleaved variant, flextrain/nn/blocks/rope.py:284-507): frequency
    slot ``j`` takes its position from axis ``j % 3`` while ``j < 3*min_section``
    style interleaving covers the h/w sections; remaining slots use the t axis.
    """
    inv = inv_freq.to(positions.device)
    if positions.dim() == 1:
        return positions.to(F32).unsqueeze(-1) * inv
    assert positions.shape[-1] == 3 and mrope_sections is not None
    ang = positions.to(F32).unsqueeze(-1) * inv  # (T,3,rot/2)
    n = inv.numel()
    axis = torch.zeros(n, dtype=torch.long, device=positions.device)
    for ax in (1, 2):
        sl = torch.arange(ax, 3 * mrope_sections[ax], 3, device=positions.device)
        sl = sl[sl < n]
        axis[sl] = ax
    return ang.gather(1, axis.view(1, 1, n).expand(ang.shape[0], 1, n)).squeeze(1)


def rope_apply(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, *, inverse: bool = False,
               mrope_sections: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Rotate-half RoPE on ``x (T, H, hd)`` over the first ``2*len(inv_freq)`` channels.

    ``inverse=True`` applies the transpose rotation, which is the backward of the op.
    """
    rot = 2 * inv_freq.numel()
    ang = _rope_angles(positions, inv_freq, mrope_sections)
    cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
    if inverse:
        sin = -sin
    xf = x.to(F32)
    x1, x2 = xf[..., : rot // 2], xf[..., rot // 2: rot]
    out = xf.clone()
    out[..., : rot // 2] = x1 * cos - x2 * sin
    out[..., rot // 2: rot] = x2 * cos + x1 * sin
    return out.to(x.dtype)


# ------------------------------------------------------------------- gated activations
def _act(x: torch.Tensor, kind: str) -> torch.Tensor:
    return F.silu(x) if kind == "swiglu" else F.gelu(x, approximate="tanh")


def glu_fwd(gate: torch.Tensor, up: torch.Tensor, kind: str = "swiglu") -> torch.Tensor:
    """``act(gate) * up`` with ``act`` = SiLU (SwiGLU) or tanh-GELU (GeGLU)."""
    return (_act(gate.to(F32), kind) * up.to(F32)).to(gate.dtype)


def glu_bwd(dact: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, kind: str = "swiglu"
            ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns ``(dgate, dup, act)``; the activation is re-emitted for the down-proj wgrad."""
    g, u, d = gate.to(F32), up.to(F32), dact.to(F32)
    if kind == "swiglu":
        s = torch.sigmoid(g)
        a = g * s
        da = s * (1 + g * (1 - s))
    else:
        k0, k1 = 0.7978845608028654, 0.044715
        t = torch.tanh(k0 * (g + k1 * g ** 3))
        a = 0.5 * g * (1 + t)
        da = 0.5 * (1 + t) + 0.5 * g * (1 - t * t) * k0 * (1 + 3 * k1 * g * g)
    return (d * u * da).to(gate.dtype), (d * a).to(gate.dtype), (a * u).to(gate.dtype)


# ---------------------------------------------------------------------- attention
def _attn_mask(lq: int, lk: int, window: int, device) -> torch.Tensor:
    off = lk - lq
    qi = torch.arange(lq, device=device).unsqueeze(1) + off
    kj = torch.arange(lk, device=device).unsqueeze(0)
    m = kj <= qi
    if window and window > 0:
        m = m & (kj > qi - window)
    return m


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_q: torch.Tensor, cu_k: torch.Tensor, *,
                  scale: float, causal: bool = True, window: int = 0, softcap: float = 0.0
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Varlen GQA attention. ``q (Tq,H,hd)``, ``k,v (Tk,KV,hd)``; returns ``(out (Tq,H,hd), lse (H,Tq) fp32)``."""
    Tq, H, hd = q.shape
    KV = k.shape[1]
    rep = H // KV
    out = torch.empty_like(q)
    lse = torch.empty(H, Tq, dtype=F32, device=q.device)
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for s in range(len(cq) - 1):
        q0, q1, k0, k1 = cq[s], cq[s + 1], ck[s], ck[s + 1]
        if q1 == q0:
            continue
        qs = q[q0:q1].to(F32).transpose(0, 1)                       # (H,Lq,hd)
        ks = k[k0:k1].to(F32).transpose(0, 1).repeat_interleave(rep, 0)
        vs = v[k0:k1].to(F32).transpose(0, 1).repeat_interleave(rep, 0)
        sc = torch.einsum("hqd,hkd->hqk", qs, ks) * scale
        if softcap and softcap > 0:
            sc = softcap * torch.tanh(sc / softcap)
        if causal:
            sc = sc.masked_fill(~_attn_mask(q1 - q0, k1 - k0, window, q.device), float("-inf"))
        l = torch.logsumexp(sc, dim=-1)
        p = torch.exp(sc - l.unsqueeze(-1))
        out[q0:q1] = torch.einsum("hqk,hkd->hqd", p, vs).transpose(0, 1).to(q.dtype)
        lse[:, q0:q1] = l
    return out, lse


def attention_bwd(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
                  lse: torch.Tensor, cu_q: torch.Tensor, cu_k: torch.Tensor, *, scale: float, causal: bool = True,
                  window: int = 0, softcap: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns ``(dq, dk, dv)`` — dk/dv cover *all* visible keys (prior-chunk keys included)."""
    Tq, H, hd = q.shape
    KV = k.shape[1]
    rep = H // KV
    dq = torch.zeros_like(q, dtype=F32)
    dk = torch.zeros_like(k, dtype=F32)
    dv = torch.zeros_like(v, dtype=F32)
    cq, ck = cu_q.tolist(), cu_k.tolist()
    for s in range(len(cq) - 1):
        q0, q1, k0, k1 = cq[s], cq[s + 1], ck[s], ck[s + 1]
        if q1 == q0:
            continue
        qs = q[q0:q1].to(F32).transpose(0, 1)
        ks = k[k0:k1].to(F32).transpose(0, 1).repeat_interleave(rep, 0)
        vs = v[k0:k1].to(F32).transpose(0, 1).repeat_interleave(rep, 0)
        do = dout[q0:q1].to(F32).transpose(0, 1)
        o = out[q0:q1].to(F32).transpose(0, 1)
        raw = torch.einsum("hqd,hkd->hqk", qs, ks) * scale
        sc = softcap * torch.tanh(raw / softcap) if softcap and softcap > 0 else raw
        if causal:
            sc = sc.masked_fill(~_attn_mask(q1 - q0, k1 - k0, window, q.device), float("-inf"))
        p = torch.exp(sc - lse[:, q0:q1].unsqueeze(-1))
        dvs = torch.einsum("hqk,hqd->hkd", p, do)
        dp = torch.einsum("hqd,hkd->hqk", do, vs)
        delta = (do * o).sum(-1, keepdim=True)
        ds = p * (dp - delta)
        if softcap and softcap > 0:
            ds = ds * (1 - torch.tanh(raw / softcap) ** 2)
        ds = ds * scale
        dq[q0:q1] = torch.einsum("hqk,hkd->hqd", ds, ks).transpose(0, 1)
        dks = torch.einsum("hqk,hqd->hkd", ds, qs)
        dk[k0:k1] += dks.reshape(KV, rep, k1 - k0, hd).sum(1).transpose(0, 1)
        dv[k0:k1] += dvs.reshape(KV, rep, k1 - k0, hd).sum(1).transpose(0, 1)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


# ------------------------------------------------------------------ loss / embedding
def softmax_ce_fwd_bwd(logits: torch.Tensor, targets: torch.Tensor, *, grad_scale: float = 1.0,
                       softcap: float = 0.0, loss_mask: Optional[torch.Tensor] = None,
                       ignore_index: int = -100) -> Tuple[torch.Tensor, torch.Tensor]:
    """Fused softmax cross-entropy. Returns ``(per_token_loss fp32 (T,), dlogits)``.

    ``dlogits = grad_scale * (softmax - onehot)`` (zero on ignored rows), already chained
    through the optional final-logit tanh softcap.  The reference does this as a softmax
    pass plus an in-place ``P[label] -= 1`` pass (flextrain/ops/_kernels/softmax.py:13-108,
    cross_entropy.py:14-58).
    """
    z = logits.to(F32)
    if softcap and softcap > 0:
        t = torch.tanh(z / softcap)
        zc = softcap * t
    else:
        zc = z
    valid = targets != ignore_index
    if loss_mask is not None:
        valid = valid & (loss_mask > 0)
    tgt = torch.where(valid, targets, torch.zeros_like(targets)).long()
    lse = torch.logsumexp(zc, dim=-1)
    loss = (lse - zc.gather(1, tgt.unsqueeze(1)).squeeze(1)) * valid
    p = torch.exp(zc - lse.unsqueeze(-1))
    p.scatter_add_(1, tgt.unsqueeze(1), -torch.ones_like(lse).unsqueeze(1))
    dz = p * (valid.to(F32) * grad_scale).unsqueeze(-1)
    if softcap and softcap > 0:
        dz = dz * (1 - t * t)
    return loss, dz.to(logits.dtype)


def embedding_fwd(tokens: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    y = table[tokens.long()]
    return (y.to(F32) * scale).to(table.dtype) if scale != 1.0 else y


def embedding_bwd(dy: torch.Tensor, tokens: torch.Tensor, grad_table: torch.Tensor, scale: float = 1.0) -> None:
    """``grad_table[tokens] += scale * dy`` (fp32 accumulation, duplicate-safe)."""
    acc = torch.zeros(grad_table.shape, dtype=F32, device=grad_table.device)
    acc.index_add_(0, tokens.long(), dy.to(F32) * scale)
    grad_table.add_(acc.to(grad_table.dtype))


# ---------------------------------------------------------------------- optimizers
def adamw_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float, beta1: float,
               beta2: float, eps: float, weight_decay: float, step: int, grad_scale: float = 1.0) -> None:
    """Decoupled-weight-decay AdamW in fp32 registers, any storage dtype
    (flextrain/ops/_kernels/adamw.py:36-60): ``p -= lr*wd*p``; EMA; host bias correction;
    ``p -= lr * mhat / (sqrt(vhat) + eps)``."""
    pf, gf, mf, vf = p.to(F32), g.to(F32) * grad_scale, m.to(F32), v.to(F32)
    pf = pf - lr * weight_decay * pf
    mf = beta1 * mf + (1 - beta1) * gf
    vf = beta2 * vf + (1 - beta2) * gf * gf
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    pf = pf - lr * (mf / bc1) / ((vf / bc2).sqrt() + eps)
    p.copy_(pf.to(p.dtype)); m.copy_(mf.to(m.dtype)); v.copy_(vf.to(v.dtype))


NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(g: torch.Tensor, iters: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation (flextrain/ops/_kernels/muon.py:53-61)."""
    a, b, c = NS_COEFFS
    x = g.to(F32)
    tall = x.shape[-2] > x.shape[-1]
    if tall:
        x = x.transpose(-1, -2)
    x = x / (x.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(iters):
        A = x @ x.transpose(-1, -2)
        B = b * A + c * (A @ A)
        x = a * x + B @ x
    if tall:
        x = x.transpose(-1, -2)
    return x


def muon_step(p: torch.Tensor, g: torch.Tensor, mom: torch.Tensor, *, lr: float, beta: float = 0.95,
              weight_decay: float = 0.0, ns_iters: int = 5, nesterov: bool = True, grad_scale: float = 1.0) -> None:
    """Muon: momentum, Nesterov, NS orthogonalise, ``p -= lr * 0.2*sqrt(max(m,n)) * X``
    (flextrain/ops/_kernels/muon.py:16-75). 3-D tensors are treated as a batch of matrices."""
    gf = g.to(F32) * grad_scale
    mf = beta * mom.to(F32) + gf
    mom.copy_(mf.to(mom.dtype))
    u = gf + beta * mf if nesterov else mf
    x = newton_schulz(u, ns_iters)
    scale = 0.2 * math.sqrt(max(p.shape[-2], p.shape[-1]))
    pf = p.to(F32)
    pf = pf - lr * weight_decay * pf - lr * scale * x
    p.copy_(pf.to(p.dtype))


# ------------------------------------------------------------------------------ MoE
def topk_route(logits: torch.Tensor, k: int, mode: str = "topk_then_softmax") -> Tuple[torch.Tensor, torch.Tensor]:
    """Router. Returns ``(weights (T,k) fp32, experts (T,k) int32)``; ties → lowest index.

    ``topk_then_softmax``: softmax over the k selected logits (Qwen3-MoE / OLMoE norm_topk);
    ``softmax_then_topk``: full softmax, take top-k probabilities, not renormalised
    (flextrain/ops/_kernels/moe.py:218-314).
    """
    z = logits.to(F32)
    if mode == "softmax_then_topk":
        z = torch.softmax(z, dim=-1)
    # stable sort on (-value) gives lowest index on ties
    vals, idx = torch.sort(z, dim=-1, descending=True, stable=True)
    vals, idx = vals[:, :k], idx[:, :k]
    w = torch.softmax(vals, dim=-1) if mode == "topk_then_softmax" else vals
    return w, idx.to(torch.int32)


def topk_route_bwd(dw: torch.Tensor, logits: torch.Tensor, w: torch.Tensor, experts: torch.Tensor,
                   mode: str = "topk_then_softmax") -> torch.Tensor:
    """dlogits (T,E) fp32 from the gradient of the selected routing weights."""
    T, E = logits.shape
    dl = torch.zeros(T, E, dtype=F32, device=logits.device)
    idx = experts.long()
    dwf = dw.to(F32)
    if mode == "topk_then_softmax":
        dsel = w * (dwf - (dwf * w).sum(-1, keepdim=True))
        dl.scatter_(1, idx, dsel)
    else:
        p = torch.softmax(logits.to(F32), dim=-1)
        dp = torch.zeros_like(p).scatter_(1, idx, dwf)
        dl = p * (dp - (dp * p).sum(-1, keepdim=True))
    return dl


def moe_sort(experts: torch.Tensor, num_experts: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Counting sort of the ``T*K`` assignments by expert (stable in slot order).

    Returns ``(perm (T*K,) int32: sorted position -> flat slot id, counts (E,) int32,
    offsets (E+1,) int32)``.
    """
    flat = experts.reshape(-1).long()
    perm = torch.sort(flat, stable=True).indices.to(torch.int32)
    counts = torch.bincount(flat, minlength=num_experts).to(torch.int32)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32, device=experts.device)
    offsets[1:] = torch.cumsum(counts, 0)
    return perm, counts, offsets


def grouped_gemm(x: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, *, trans_w: bool = True) -> torch.Tensor:
    """Expert-major grouped GEMM: rows ``offsets[e]:offsets[e+1]`` of ``x`` times ``w[e]``.

    ``w (E, N, K)`` with ``trans_w`` (``y = x @ w[e].T``) or ``w (E, K, N)`` without.
    """
    E = w.shape[0]
    n_out = w.shape[1] if trans_w else w.shape[2]
    y = torch.zeros(x.shape[0], n_out, dtype=x.dtype, device=x.device)
    off = offsets.tolist()
    for e in range(E):
        a, b = off[e], off[e + 1]
        if b > a:
            we = w[e].to(F32)
            y[a:b] = (x[a:b].to(F32) @ (we.t() if trans_w else we)).to(x.dtype)
    return y


def grouped_wgrad(dy: torch.Tensor, x: torch.Tensor, offsets: torch.Tensor, gw: torch.Tensor, *,
                  alpha: float = 1.0) -> None:
    """``gw[e] += alpha * dy[rows_e].T @ x[rows_e]`` for ``gw (E, N, K)``."""
    off = offsets.tolist()
    for e in range(gw.shape[0]):
        a, b = off[e], off[e + 1]
        if b > a:
            gw[e] += (alpha * (dy[a:b].to(F32).t() @ x[a:b].to(F32))).to(gw.dtype)


# ------------------------------------------------------- Gated DeltaNet and friends
def l2norm_fwd(x: torch.Tensor, eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    xf = x.to(F32)
    r = torch.rsqrt(xf.pow(2).sum(-1) + eps)
    return (xf * r.unsqueeze(-1)).to(x.dtype), r


def l2norm_bwd(dy: torch.Tensor, x: torch.Tensor, r: torch.Tensor) -> torch.Tensor:
    xf, dyf = x.to(F32), dy.to(F32)
    y = xf * r.unsqueeze(-1)
    return ((dyf - y * (dyf * y).sum(-1, keepdim=True)) * r.unsqueeze(-1)).to(x.dtype)


def gated_rmsnorm_fwd(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``rmsnorm(o) * w * silu(z)`` (flextrain/ops/_kernels/gated_rmsnorm.py:65-140)."""
    of = o.to(F32)
    r = torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps)
    return (of * r * w.to(F32) * F.silu(z.to(F32))).to(o.dtype)


def causal_conv1d_fwd(x: torch.Tensor, w: torch.Tensor, cu: torch.Tensor, init_state: Optional[torch.Tensor] = None,
                      activation: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Depthwise causal conv over packed sequences. ``x (T, D)``, ``w (D, W)``.

    ``init_state (S, D, W-1)`` holds the last ``W-1`` inputs of each sequence's prior
    chunk (zeros when absent). Returns ``(y, final_state (S, D, W-1))``.
    """
    T, D = x.shape
    W = w.shape[1]
    cs = cu.tolist()
    S = len(cs) - 1
    y = torch.empty_like(x)
    fin = torch.zeros(S, D, W - 1, dtype=x.dtype, device=x.device)
    for s in range(S):
        a, b = cs[s], cs[s + 1]
        if b == a:
            if init_state is not None:
                fin[s] = init_state[s]
            continue
        pre = init_state[s].to(F32).t() if init_state is not None else torch.zeros(W - 1, D, device=x.device)
        xx = torch.cat([pre, x[a:b].to(F32)], 0)                  # (L+W-1, D)
        win = xx.unfold(0, W, 1)                                  # (L, D, W)
        out = (win * w.to(F32).unsqueeze(0)).sum(-1)
        y[a:b] = (F.silu(out) if activation else out).to(x.dtype)
        fin[s] = xx[-(W - 1):].t().to(x.dtype)
    return y, fin


def gated_delta_rule(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
                     cu: torch.Tensor, init_state: Optional[torch.Tensor] = None, scale: Optional[float] = None
                     ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gated delta rule, token-recurrent definition (autograd-friendly fp32).

    ``q,k (T,HK,dk)``, ``v (T,HV,dv)``, ``g (T,HV)`` log-decay (≤0), ``beta (T,HV)``.
    State ``S (HV,dk,dv)``:  ``S = exp(g_t) S``;  ``S += k_t ⊗ beta_t (v_t − S^T k_t)``;
    ``o_t = S^T (q_t * scale)``.  HK heads are repeated to HV (GVA).  Returns
    ``(o (T,HV,dv), final_state (Nseq,HV,dk,dv) fp32)``; semantics match the FLA call the
    reference makes (flextrain/nn/blocks/linear_attn.py:1090-1145).
    """
    T, HK, dk = q.shape
    HV, dv = v.shape[1], v.shape[2]
    rep = HV // HK
    scale = scale if scale is not None else dk ** -0.5
    cs = cu.tolist()
    outs, finals = [], []
    for s in range(len(cs) - 1):
        a, b = cs[s], cs[s + 1]
        S = init_state[s].to(F32) if init_state is not None else torch.zeros(HV, dk, dv, dtype=F32, device=q.device)
        qs = q[a:b].to(F32).repeat_interleave(rep, 1) * scale
        ks = k[a:b].to(F32).repeat_interleave(rep, 1)
        vs, gs, bs = v[a:b].to(F32), g[a:b].to(F32), beta[a:b].to(F32)
        o_s = []
        for t in range(b - a):
            S = S * gs[t].exp().view(HV, 1, 1)
            pred = torch.einsum("hkv,hk->hv", S, ks[t])
            upd = bs[t].view(HV, 1) * (vs[t] - pred)
            S = S + torch.einsum("hk,hv->hkv", ks[t], upd)
            o_s.append(torch.einsum("hkv,hk->hv", S, qs[t]))
        outs.append(torch.stack(o_s, 0) if o_s else torch.zeros(0, HV, dv, dtype=F32, device=q.device))
        finals.append(S)
    return torch.cat(outs, 0).to(v.dtype), torch.stack(finals, 0)


def gated_delta_rule_chunked(q, k, v, g, beta, cu, init_state=None, scale=None, chunk: int = 64):
    """Chunk-parallel (WY representation) form of :func:`gated_delta_rule`; same results,
    O(T/chunk) sequential steps.  Differentiable; used on GPU when no fused kernel applies."""
    T, HK, dk = q.shape
    HV, dv = v.shape[1], v.shape[2]
    rep = HV // HK
    scale = scale if scale is not None else dk ** -0.5
    cs = cu.tolist()
    outs, finals = [], []
    for s in range(len(cs) - 1):
        a, b = cs[s], cs[s + 1]
        L = b - a
        S = init_state[s].to(F32) if init_state is not None else torch.zeros(HV, dk, dv, dtype=F32, device=q.device)
        if L == 0:
            finals.append(S); continue
        pad = (-L) % chunk
        def prep(x):
            x = x[a:b].to(F32)
            if pad:
                x = torch.cat([x, torch.zeros(pad, *x.shape[1:], dtype=F32, device=x.device)], 0)
            return x
        qs = prep(q).repeat_interleave(rep, 1) * scale
        ks = prep(k).repeat_interleave(rep, 1)
        vs, gs, bs = prep(v), prep(g), prep(beta)
        n = (L + pad) // chunk
        # (H, n, C, d)
        rs = lambda x: x.reshape(n, chunk, HV, -1).permute(2, 0, 1, 3)
        qs, ks, vs = rs(qs), rs(ks), rs(vs)
        gs = gs.reshape(n, chunk, HV).permute(2, 0, 1)
        bs = bs.reshape(n, chunk, HV).permute(2, 0, 1)
        gc = gs.cumsum(-1)                                                    # (H,n,C)
        decay = (gc.unsqueeze(-1) - gc.unsqueeze(-2))                         # g_i - g_j
        tril = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device))
        strict = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool, device=q.device), -1)
        dm = torch.where(tril, decay, torch.zeros_like(decay)).exp() * tril
        kb = ks * bs.unsqueeze(-1)
        A = -(kb @ ks.transpose(-1, -2)) * dm * strict                        # strictly lower
        # (I - A)^-1 via forward substitution rows
        rows = [A[..., 0, :]]
        for i in range(1, chunk):                                             # out-of-place: autograd-safe
            prev = torch.stack(rows, -2)                                      # (H,n,i,C)
            rows.append(A[..., i, :] + (A[..., i, :i].unsqueeze(-1) * prev).sum(-2))
        Tm = torch.stack(rows, -2) + torch.eye(chunk, device=q.device)
        w_ = Tm @ (kb * gc.exp().unsqueeze(-1))                               # (H,n,C,dk)
        u_ = Tm @ (vs * bs.unsqueeze(-1))                                     # (H,n,C,dv)
        o_chunks = []
        for c in range(n):
            qc, kc, gcc = qs[:, c], ks[:, c], gc[:, c]
            v_new = u_[:, c] - w_[:, c] @ S                                   # (H,C,dv)
            attn = (qc @ kc.transpose(-1, -2)) * dm[:, c]
            o = (qc * gcc.exp().unsqueeze(-1)) @ S + attn @ v_new
            o_chunks.append(o)
            glast = gcc[:, -1]
            S = S * glast.exp().view(HV, 1, 1) + (kc * (glast.unsqueeze(-1) - gcc).exp().unsqueeze(-1)).transpose(-1, -2) @ v_new
        o = torch.stack(o_chunks, 1).permute(1, 2, 0, 3).reshape(n * chunk, HV, dv)[:L]
        outs.append(o); finals.append(S)
    return torch.cat(outs, 0).to(v.dtype), torch.stack(finals, 0)


def top_p_sample(logits: torch.Tensor, top_p: float, temperature: float, generator=None) -> torch.Tensor:
    """Nucleus sampling per row (flextrain/ops/_kernels/sample_top_p.py:7-150)."""
    z = logits.to(F32) / max(temperature, 1e-6)
    p = torch.softmax(z, -1)
    sp, si = torch.sort(p, dim=-1, descending=True)
    keep = (sp.cumsum(-1) - sp) < top_p
    sp = sp * keep
    sp = sp / sp.sum(-1, keepdim=True)
    pick = torch.multinomial(sp, 1, generator=generator)
    return si.gather(1, pick).squeeze(1)


# ------------------------------------------------------------------- MoE dispatch plan
class MoEPlan:
    """Expert-major row layout of one chunk's ``T*K`` routed slots, built without a host sync.

    ``row_src (R,)``: flat slot id ``t*K + k`` held by each row, ``-1`` for padding rows;
    ``inv (T,K)``: row of each slot; ``offsets (E+1,)``: start row of each expert (each expert's
    segment is padded to a multiple of ``pad`` so GEMM tiles never straddle two experts).
    """
    __slots__ = ("row_src", "inv", "offsets", "rows", "counts")

    def __init__(self, row_src, inv, offsets, rows, counts=None):
        self.row_src, self.inv, self.offsets, self.rows, self.counts = row_src, inv, offsets, rows, counts


def moe_rows_bound(T: int, K: int, E: int, pad: int) -> int:
    """Static upper bound of rows: every expert can waste at most ``pad - 1`` rows."""
    return (T * K + E * (pad - 1) + pad - 1) // pad * pad


def moe_plan(experts: torch.Tensor, num_experts: int, pad: int = 1) -> MoEPlan:
    T, K = experts.shape
    dev = experts.device
    flat = experts.reshape(-1).long()
    n = flat.numel()
    R = moe_rows_bound(T, K, num_experts, pad)
    counts = torch.zeros(num_experts, dtype=torch.long, device=dev).index_add_(
        0, flat, torch.ones(n, dtype=torch.long, device=dev))
    padded = (counts + pad - 1) // pad * pad
    offsets = torch.zeros(num_experts + 1, dtype=torch.long, device=dev)
    offsets[1:] = torch.cumsum(padded, 0)
    starts = torch.zeros(num_experts, dtype=torch.long, device=dev)
    starts[1:] = torch.cumsum(counts, 0)[:-1]
    order = torch.sort(flat, stable=True).indices                    # sorted position -> slot
    e_sorted = flat[order]
    rank = torch.arange(n, device=dev) - starts[e_sorted]
    rows = offsets[e_sorted] + rank
    row_src = torch.full((R,), -1, dtype=torch.int32, device=dev)
    row_src[rows] = order.to(torch.int32)
    inv = torch.empty(n, dtype=torch.int32, device=dev)
    inv[order] = rows.to(torch.int32)
    return MoEPlan(row_src, inv.view(T, K), offsets.to(torch.int32), R, counts.to(torch.int32))


def moe_row_weights(w: torch.Tensor, plan: MoEPlan) -> torch.Tensor:
    """Router weight of the slot held by each row (0 for padding rows), fp32 ``(R,)``."""
    src = plan.row_src.long()
    out = w.reshape(-1).to(F32)[src.clamp(min=0)]
    return out * (src >= 0)


def moe_rows_to_slots(v: torch.Tensor, plan: MoEPlan, shape) -> torch.Tensor:
    """Inverse of the row layout for a per-row scalar: returns ``(T,K)``."""
    return v[plan.inv.reshape(-1).long()].view(shape)
