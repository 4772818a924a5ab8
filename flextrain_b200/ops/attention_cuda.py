"""Bindings to the tcgen05 flash-attention kernels (``csrc/attention.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_long

import torch

from .cuda import _check, _ptr, _stream, load


def _strided_ok(t: torch.Tensor) -> bool:
    return t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def fwd(q, k, v, cu_q, cu_k, max_q, max_k, *, scale, causal=True, window=0, softcap=0.0):
    """``q (Tq,H,hd)``, ``k,v (Tk,KV,hd)`` bf16 (token-strided views allowed). Returns ``(out, lse (H,Tq) fp32)``."""
    lib = load("attention")
    if not _strided_ok(q):
        q = q.contiguous()
    if not _strided_ok(k):
        k = k.contiguous()
    if not _strided_ok(v):
        v = v.contiguous()
    Tq, H, hd = q.shape
    Tk, KV = k.shape[0], k.shape[1]
    nseq = cu_q.numel() - 1
    out = torch.empty(Tq, H, hd, dtype=q.dtype, device=q.device)
    lse = torch.empty(H, Tq, dtype=torch.float32, device=q.device)
    cu_q = cu_q.to(torch.int32)
    cu_k = cu_k.to(torch.int32)
    rc = lib.ftb_attn_fwd(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), _ptr(cu_q), _ptr(cu_k), c_int(nseq),
                          c_int(Tq), c_int(Tk), c_int(H), c_int(KV), c_int(hd), c_long(q.stride(0)),
                          c_long(k.stride(0)), c_long(v.stride(0)), c_float(scale), c_float(float(softcap or 0.0)),
                          c_int(1 if causal else 0), c_int(int(window or 0)), c_int(Tq // 128 + nseq), _stream())
    _check(rc, "ftb_attn_fwd")
    return out, lse


def deterministic_default() -> bool:
    """``FTB_ATTN_DETERMINISTIC`` (default 1): fixed dQ summation order, as the reference asks of its flash back ends
    (``deterministic=True``, flextrain/ops/_kernels/attention.py:227,302,378)."""
    import os
    return os.environ.get("FTB_ATTN_DETERMINISTIC", "1") != "0"


def bwd(dout, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, *, scale, causal=True, window=0, softcap=0.0,
        deterministic=None):
    """Returns ``(dq, dk, dv)``; dk / dv cover all keys.  ``deterministic`` (default: :func:`deterministic_default`)
    orders the key tiles' additions to every query tile, so two runs give bit-identical dQ (dK / dV always are)."""
    lib = load("attention")
    if not hasattr(lib, "ftb_attn_bwd"):
        raise NotImplementedError
    q = q if _strided_ok(q) else q.contiguous()
    k = k if _strided_ok(k) else k.contiguous()
    v = v if _strided_ok(v) else v.contiguous()
    dout = dout if _strided_ok(dout) else dout.contiguous()
    out = out if _strided_ok(out) else out.contiguous()
    Tq, H, hd = q.shape
    Tk, KV = k.shape[0], k.shape[1]
    nseq = cu_q.numel() - 1
    dq_acc = torch.zeros(Tq, H, hd, dtype=torch.float32, device=q.device)
    dq = torch.empty(Tq, H, hd, dtype=q.dtype, device=q.device)
    dk = torch.empty(Tk, KV, hd, dtype=q.dtype, device=q.device)
    dv = torch.empty(Tk, KV, hd, dtype=q.dtype, device=q.device)
    delta = torch.empty(H, Tq, dtype=torch.float32, device=q.device)
    cu_q = cu_q.to(torch.int32)
    cu_k = cu_k.to(torch.int32)
    det = deterministic_default() if deterministic is None else bool(deterministic)
    sem = torch.zeros(1 + (Tq // 128 + nseq) * H, dtype=torch.int32, device=q.device) if det else None
    rc = lib.ftb_attn_bwd(_ptr(dout), _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), _ptr(delta), _ptr(dq_acc),
                          _ptr(sem), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(cu_q), _ptr(cu_k), c_int(nseq), c_int(Tq), c_int(Tk),
                          c_int(H), c_int(KV), c_int(hd), c_long(q.stride(0)), c_long(k.stride(0)),
                          c_long(v.stride(0)), c_long(dout.stride(0)), c_long(out.stride(0)), c_float(scale),
                          c_float(float(softcap or 0.0)), c_int(1 if causal else 0), c_int(int(window or 0)),
                          c_int(Tk // 128 + nseq), _stream())
    _check(rc, "ftb_attn_bwd")
    dq.copy_(dq_acc)
    return dq, dk, dv
