"""ctypes bindings of the Gated DeltaNet kernels (``csrc/gdn.cu``) and the small kernels around them
(``csrc/seqmix.cu``): causal conv1d, strided L2 norm, gated RMSNorm backward, top-p sampling.

All tensors are bf16 unless noted; ``cu`` is the int32 cumulative sequence-length vector of the chunk.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long
from typing import Optional, Tuple

import torch

from .cuda import _check, _ptr, _stream, load

BF, F32 = torch.bfloat16, torch.float32


def _rows_ld(x: torch.Tensor) -> int:
    """Leading dimension (elements) of a 2-D view whose rows are contiguous."""
    assert x.dim() == 2 and x.stride(1) == 1
    return x.stride(0)


# ------------------------------------------------------------------------------------------------ conv1d
def conv1d_fwd(x: torch.Tensor, w: torch.Tensor, cu: torch.Tensor, init: Optional[torch.Tensor], activation=True
               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x (T, D)`` (row-strided view allowed), ``w (D, W)``, ``init (S, D, W-1)`` or None → ``(y (T,D), final)``."""
    lib = load("seqmix")
    T, D = x.shape
    W = w.shape[1]
    S = cu.numel() - 1
    y = torch.empty(T, D, dtype=BF, device=x.device)
    fin = torch.empty(S, D, W - 1, dtype=BF, device=x.device)
    init_c = init.to(BF).contiguous() if init is not None else None
    rc = lib.ftb_conv1d_fwd(_ptr(x), c_long(_rows_ld(x)), _ptr(w.contiguous()), _ptr(init_c), _ptr(cu), c_int(S), _ptr(y),
                            _ptr(fin), c_int(T), c_int(D), c_int(W), c_int(1 if activation else 0), _stream())
    _check(rc, "ftb_conv1d_fwd")
    return y, fin


def conv1d_bwd(x, w, cu, init, dy, dfin, dx_out: torch.Tensor, dw: Optional[torch.Tensor], want_dinit: bool,
               activation=True) -> Optional[torch.Tensor]:
    """Writes ``dx`` into ``dx_out (T, D)`` (row-strided view allowed), accumulates ``dw (D, W)`` fp32, returns the
    gradient of ``init`` (or None)."""
    lib = load("seqmix")
    T, D = x.shape
    W = w.shape[1]
    S = cu.numel() - 1
    dpre = torch.empty(T, D, dtype=F32, device=x.device)
    init_c = init.to(BF).contiguous() if init is not None else None
    dfin_c = dfin.to(BF).contiguous() if dfin is not None else None
    dinit = torch.empty(S, D, W - 1, dtype=BF, device=x.device) if want_dinit else None
    assert dw is None or (dw.dtype == F32 and dw.is_contiguous())
    rc = lib.ftb_conv1d_bwd(_ptr(x), c_long(_rows_ld(x)), _ptr(w.contiguous()), _ptr(init_c), _ptr(cu), c_int(S),
                            _ptr(dy.contiguous()), _ptr(dfin_c), _ptr(dpre), _ptr(dx_out), c_long(_rows_ld(dx_out)),
                            _ptr(dw), _ptr(dinit), c_int(T), c_int(D), c_int(W), c_int(1 if activation else 0), _stream())
    _check(rc, "ftb_conv1d_bwd")
    return dinit


# ----------------------------------------------------------------------------------------------- L2 norm
def l2norm_heads_fwd(x2d: torch.Tensor, H: int, D: int, eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-head L2 normalisation of the ``H*D`` leading columns of each row of ``x2d (T, >=H*D)``.
    Returns ``(y (T,H,D) contiguous, rnorm (T,H) fp32)``."""
    lib = load("seqmix")
    T = x2d.shape[0]
    y = torch.empty(T, H, D, dtype=BF, device=x2d.device)
    rn = torch.empty(T, H, dtype=F32, device=x2d.device)
    rc = lib.ftb_l2norm_strided_fwd(_ptr(x2d), c_long(_rows_ld(x2d)), _ptr(y), c_long(H * D), _ptr(rn), c_long(T), c_int(H),
                                    c_int(D), c_float(eps), _stream())
    _check(rc, "ftb_l2norm_strided_fwd")
    return y, rn


def l2norm_heads_bwd(dy: torch.Tensor, x2d: torch.Tensor, rnorm: torch.Tensor, dx_out2d: torch.Tensor, H: int, D: int
                     ) -> None:
    """``dy (T,H,D)`` fp32 → gradient of the pre-norm values written into ``dx_out2d (T, >=H*D)``."""
    lib = load("seqmix")
    T = x2d.shape[0]
    assert dy.dtype == F32 and dy.is_contiguous()
    rc = lib.ftb_l2norm_strided_bwd(_ptr(dy), _ptr(x2d), c_long(_rows_ld(x2d)), _ptr(rnorm), _ptr(dx_out2d),
                                    c_long(_rows_ld(dx_out2d)), c_long(T), c_int(H), c_int(D), _stream())
    _check(rc, "ftb_l2norm_strided_bwd")


# ------------------------------------------------------------------------------------- gated RMSNorm backward
def gated_rmsnorm_bwd(dy: torch.Tensor, o: torch.Tensor, z2d: torch.Tensor, w: torch.Tensor, dz_out2d: torch.Tensor,
                      dw: Optional[torch.Tensor], H: int, D: int, eps: float) -> torch.Tensor:
    """``dy, o (T,H,D)`` contiguous; ``z2d`` / ``dz_out2d`` are row-strided ``(T, H*D)`` views.  Returns ``d_o``."""
    lib = load("seqmix")
    T = o.shape[0]
    d_o = torch.empty_like(o)
    assert w.dtype == F32 and (dw is None or (dw.dtype == F32 and dw.is_contiguous()))
    rc = lib.ftb_gated_rmsnorm_bwd(_ptr(dy.contiguous()), _ptr(o.contiguous()), _ptr(z2d), c_long(_rows_ld(z2d)), c_int(H),
                                   _ptr(w), _ptr(d_o), _ptr(dz_out2d), c_long(_rows_ld(dz_out2d)), _ptr(dw), c_long(T),
                                   c_int(D), c_float(eps), _stream())
    _check(rc, "ftb_gated_rmsnorm_bwd")
    return d_o


# ------------------------------------------------------------------------------------------ gated delta rule
def gate_prep_fwd(ba: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``beta = sigmoid(b)``, ``g = -exp(A_log) * softplus(a + dt_bias)`` from the bf16 ``[b | a]`` projection
    ``(T, 2*HV)`` in one launch; both fp32 ``(T, HV)``."""
    lib = load("seqmix")
    T, two_hv = ba.shape
    HV = two_hv // 2
    assert ba.dtype == torch.bfloat16 and ba.is_contiguous() and dt_bias.dtype == torch.float32 and a_log.dtype == torch.float32
    beta = torch.empty(T, HV, dtype=torch.float32, device=ba.device)
    g = torch.empty(T, HV, dtype=torch.float32, device=ba.device)
    _check(lib.ftb_gate_prep_fwd(_ptr(ba), _ptr(dt_bias), _ptr(a_log), _ptr(beta), _ptr(g), c_long(T), c_int(HV),
                                 _stream()), "ftb_gate_prep_fwd")
    return beta, g


def gate_prep_bwd(ba, dt_bias, a_log, g, dbeta, dg, d_a_log: Optional[torch.Tensor], d_dt_bias: Optional[torch.Tensor]
                  ) -> torch.Tensor:
    """Backward of :func:`gate_prep_fwd`: returns ``dba (T, 2*HV)`` bf16 and accumulates the two parameter gradients
    (fp32 ``(HV,)`` buffers) in the same launch."""
    lib = load("seqmix")
    T, two_hv = ba.shape
    HV = two_hv // 2
    dba = torch.empty_like(ba)
    for t in (d_a_log, d_dt_bias):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    _check(lib.ftb_gate_prep_bwd(_ptr(ba), _ptr(dt_bias), _ptr(a_log), _ptr(g.contiguous()), _ptr(dbeta.contiguous()),
                                 _ptr(dg.contiguous()), _ptr(dba), _ptr(d_a_log), _ptr(d_dt_bias), c_long(T),
                                 c_int(HV), _stream()), "ftb_gate_prep_bwd")
    return dba


def gdn_supported(dk: int, dv: int) -> bool:
    return dk in (16, 32, 64, 128) and dv % 8 == 0


def _gdn(pass_, q, k, v, g, beta, cu, state_in, state_out, o, r, d_o, de, dv, dbeta, dq, dk, sacc, scale):
    lib = load("gdn")
    T, HK, DK = q.shape
    HV, DV = v.shape[1], v.shape[2]
    rc = lib.ftb_gdn(c_int(pass_), _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(cu), c_int(cu.numel() - 1),
                     _ptr(state_in), _ptr(state_out), _ptr(o), _ptr(r), _ptr(d_o), _ptr(de), _ptr(dv), _ptr(dbeta),
                     _ptr(dq), _ptr(dk), _ptr(sacc), c_int(HK), c_int(HV), c_int(DK), c_int(DV), c_float(scale), _stream())
    _check(rc, f"ftb_gdn(pass {pass_})")


def gdn_fwd(q, k, v, g, beta, cu, state_in=None, scale=None, want_r=False):
    """``q,k (T,HK,dk)``, ``v (T,HV,dv)`` bf16 contiguous; ``g, beta (T,HV)`` fp32; ``state_in (S,HV,dk,dv)`` fp32.
    Returns ``(o (T,HV,dv) bf16, final_state fp32, r or None)``."""
    T, HK, DK = q.shape
    HV, DV = v.shape[1], v.shape[2]
    S = cu.numel() - 1
    scale = scale if scale is not None else DK ** -0.5
    o = torch.empty(T, HV, DV, dtype=BF, device=q.device)
    fin = torch.empty(S, HV, DK, DV, dtype=F32, device=q.device)
    r = torch.empty(T, HV, DV, dtype=F32, device=q.device) if want_r else None
    sin = state_in.to(F32).contiguous() if state_in is not None else None
    _gdn(0, q, k, v, g, beta, cu, sin, fin, o, r, None, None, None, None, None, None, None, scale)
    return o, fin, r


def gdn_bwd(q, k, v, g, beta, cu, state_in, final_state, r, d_o, dstate_final=None, scale=None):
    """Backward of :func:`gdn_fwd`.  Returns ``(dq (T,HK,dk) fp32, dk (T,HK,dk) fp32, dv (T,HV,dv) bf16,
    dg (T,HV) fp32, dbeta (T,HV) fp32, dstate_in (S,HV,dk,dv) fp32)``."""
    T, HK, DK = q.shape
    HV, DV = v.shape[1], v.shape[2]
    S = cu.numel() - 1
    rep = HV // HK
    scale = scale if scale is not None else DK ** -0.5
    dev = q.device
    de = torch.empty(T, HV, DV, dtype=F32, device=dev)
    dv = torch.empty(T, HV, DV, dtype=BF, device=dev)
    dbeta = torch.zeros(T, HV, dtype=F32, device=dev)
    dk_hv = torch.zeros(T, HV, DK, dtype=F32, device=dev)
    s = torch.zeros(T, HV, dtype=F32, device=dev)
    dstate_in = torch.empty(S, HV, DK, DV, dtype=F32, device=dev)
    dsf = dstate_final.to(F32).contiguous() if dstate_final is not None else None
    d_o = d_o.contiguous()
    _gdn(1, q, k, v, g, beta, cu, dsf, dstate_in, None, r, d_o, de, dv, dbeta, None, dk_hv, s, scale)
    dq_hv = torch.zeros(T, HV, DK, dtype=F32, device=dev)
    sin = state_in.to(F32).contiguous() if state_in is not None else None
    _gdn(2, q, k, v, g, beta, cu, sin, None, None, None, d_o, de, None, None, dq_hv, dk_hv, s, scale)
    # dg_t = sum_{u >= t, same sequence} s_u  (+ <dS_final, S_final>), with the per-token scalar
    # s_u = q_u.dq_u - k_u.(dS'_u e_u) + k_u.(S^_u dr_u) accumulated by the two passes
    csum = torch.flip(torch.cumsum(torch.flip(s, [0]), 0), [0])            # suffix sums over the whole chunk
    ends = cu[1:].long()                                                    # first token AFTER each sequence
    tail = torch.cat([csum, torch.zeros(1, HV, dtype=F32, device=dev)], 0)[ends]       # (S, HV) mass past the end
    if dstate_final is not None:
        tail = tail - (dsf * final_state.to(F32)).sum((-1, -2))
    lens = (cu[1:] - cu[:-1]).long()
    dg = csum - torch.repeat_interleave(tail, lens, dim=0)
    if rep > 1:
        dq = dq_hv.view(T, HK, rep, DK).sum(2)
        dk = dk_hv.view(T, HK, rep, DK).sum(2)
    else:
        dq, dk = dq_hv, dk_hv
    return dq, dk, dv, dg, dbeta, dstate_in


def top_p_sample(logits: torch.Tensor, top_p: float, temperature: float, generator=None) -> torch.Tensor:
    lib = load("seqmix")
    rows, V = logits.shape
    u = torch.rand(rows, device=logits.device, generator=generator, dtype=F32)
    out = torch.empty(rows, dtype=torch.long, device=logits.device)
    rc = lib.ftb_top_p(_ptr(logits.contiguous()), _ptr(u), _ptr(out), c_int(rows), c_int(V), c_float(top_p),
                       c_float(temperature), _stream())
    _check(rc, "ftb_top_p")
    return out
