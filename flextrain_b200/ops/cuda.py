"""ctypes bindings to the in-tree sm_100a libraries (``flextrain_b200/_lib/libftb_*.so``).

Every wrapper takes torch CUDA tensors, passes raw pointers plus the current stream, and
raises on a non-zero return code.  A missing library on a machine with a GPU is an error,
never a silent fallback: the CUDA path is the product, the torch path is the CPU oracle.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from ..build import lib_path

_libs: dict = {}


class NativeLibraryMissing(RuntimeError):
    pass


def load(name: str) -> ctypes.CDLL:
    """dlopen ``_lib/libftb_<name>.so`` once; build it first if the source is newer or it is absent."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    path = lib_path(name)
    if not path.exists():
        try:
            from ..build import build_all
            build_all()
        except Exception as exc:  # pragma: no cover - only on a box without nvcc
            raise NativeLibraryMissing(f"{path} is missing and could not be built: {exc}") from exc
    if not path.exists():
        raise NativeLibraryMissing(f"native library {path} is missing; run `python -m flextrain_b200.build`")
    lib = ctypes.CDLL(str(path))
    _libs[name] = lib
    if name == "gemm_tcgen05" and os.environ.get("FTB_GEMM_TWO_SM", "1") == "0":
        lib.ftb_gemm_set_two_sm(c_int(0))   # one-SM tiles for every shape (A/B comparisons)
    if name == "attention" and os.environ.get("FTB_ATTN_DQ_BULK", "1") == "0":
        lib.ftb_attn_set_dq_bulk(c_int(0))      # backward: dQ by per-thread vector reductions (A/B comparisons)
    if name == "gemm_tcgen05" and os.environ.get("FTB_TMAP_CACHE", "1") == "0":
        lib.ftb_gemm_set_tmap_cache(c_int(0))   # encode the tensor maps on every call
    if name == "gemm_tcgen05" and os.environ.get("FTB_TP_PULL", "bulk") == "threads":
        lib.ftb_gemm_set_tp_pull_threads(c_int(1))   # all-gather GEMM: pull remote panels with per-thread loads
    return lib


_fast = None


def fastcall():
    """The CPython fast-call module for GEMM launches (``csrc/fastcall.cpp``), bound to the kernel library; ``None``
    if it was not built.  ``FTB_FASTCALL=0`` keeps the ctypes path."""
    global _fast
    if _fast is None:
        _fast = False
        if os.environ.get("FTB_FASTCALL", "1") != "0":
            import importlib.util
            import sysconfig
            path = lib_path("x").parent / f"_ftb_fastcall{sysconfig.get_config_var('EXT_SUFFIX')}"
            if path.exists():
                load("gemm_tcgen05")
                spec = importlib.util.spec_from_file_location("_ftb_fastcall", str(path))
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                mod.bind(str(lib_path("gemm_tcgen05")))
                _fast = mod
    return _fast or None


def have(name: str) -> bool:
    return lib_path(name).exists()


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def device_error_words() -> dict:
    """Read (and clear) the error word of each loaded kernel library: ``{lib: code*1000 + where}``."""
    out = {}
    for name, fn in (("gemm_tcgen05", "ftb_gemm_error"), ("attention", "ftb_attn_error"), ("comm", "ftb_comm_error"),
                     ("moe", "ftb_moe_error")):
        lib = _libs.get(name)
        if lib is not None and hasattr(lib, fn):
            f = getattr(lib, fn)
            f.restype = c_int
            out[name] = int(f())
    return out


# ------------------------------------------------------------------------------- GEMM
GEMM_MAX_CTAS = int(os.environ.get("FTB_GEMM_MAX_CTAS", "0"))


def tmap_cache_stats() -> dict:
    """``{"hits": n, "misses": n}`` of the GEMM library's tensor-map cache since it was loaded."""
    lib = load("gemm_tcgen05")
    h, m = ctypes.c_ulonglong(0), ctypes.c_ulonglong(0)
    lib.ftb_gemm_tmap_cache_stats(ctypes.byref(h), ctypes.byref(m))
    return {"hits": int(h.value), "misses": int(m.value)}


def gemm_supported(a: torch.Tensor, b: torch.Tensor, trans_a: bool, trans_b: bool, out_dtype) -> bool:
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or out_dtype not in (torch.bfloat16, torch.float32):
        return False
    if a.dim() != 2 or b.dim() != 2 or a.stride(1) != 1 or b.stride(1) != 1:
        return False
    n = b.shape[0] if trans_b else b.shape[1]
    return n % 8 == 0 and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 \
        and b.data_ptr() % 16 == 0


def gemm(a, b, *, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None, bias=None, out=None, out_dtype=None,
         bn: int = 0):
    """``out = alpha * op(a) @ op(b) + beta * c + bias`` on the tcgen05 kernel.

    ``a``: (M,K), or (K,M) with ``trans_a``;  ``b``: (K,N), or (N,K) with ``trans_b``.  Rows may be strided.
    """
    lib = load("gemm_tcgen05")
    M = a.shape[1] if trans_a else a.shape[0]
    K = a.shape[0] if trans_a else a.shape[1]
    N = b.shape[0] if trans_b else b.shape[1]
    kb = b.shape[1] if trans_b else b.shape[0]
    assert K == kb, f"inner dims differ: {tuple(a.shape)} ta={trans_a} x {tuple(b.shape)} tb={trans_b}"
    out_dtype = out_dtype or (out.dtype if out is not None else torch.bfloat16)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, N)
    if beta != 0.0 and c is None:
        c = out
    if c is not None:
        assert c.dtype == out.dtype and c.stride(1) == 1
    if bias is not None:
        assert bias.dtype == torch.float32
    # small output, long reduction (rank-r LoRA gradients: M or N = r, K = tokens): a handful of tiles would each walk
    # the whole K on a handful of SMs; split K so that tiles x slices fill the GPU (fp32 slabs + ordered reduce)
    tiles = ((M + 127) // 128) * ((N + (127 if N <= 128 else 255)) // (128 if N <= 128 else 256))
    if bn == 0 and tiles <= 40 and K >= 4096 and (N <= 128 or M < 512):
        splits = max(2, min(148 // tiles, K // 512, 64))
        ws = torch.empty(splits * M * N, dtype=torch.float32, device=a.device)
        rc = lib.ftb_gemm_bf16_splitk(_ptr(a), _ptr(b), _ptr(out), _ptr(c), _ptr(bias), c_int(M), c_int(N), c_int(K),
                                      c_int(1 if trans_a else 0), c_int(0 if trans_b else 1), c_int(a.stride(0)),
                                      c_int(b.stride(0)), c_int(out.stride(0)), c_int(c.stride(0) if c is not None else 0),
                                      c_float(alpha), c_float(beta), c_int(1 if out.dtype == torch.float32 else 0),
                                      c_int(splits), _ptr(ws), _stream())
        _check(rc, "ftb_gemm_bf16_splitk")
        return out
    fast = fastcall()
    if fast is not None:
        rc = fast.gemm(a.data_ptr(), b.data_ptr(), out.data_ptr(), None if c is None else c.data_ptr(),
                       None if bias is None else bias.data_ptr(), M, N, K, 1 if trans_a else 0, 0 if trans_b else 1,
                       a.stride(0), b.stride(0), out.stride(0), c.stride(0) if c is not None else 0, float(alpha),
                       float(beta), 1 if out.dtype == torch.float32 else 0, bn, GEMM_MAX_CTAS,
                       torch.cuda.current_stream().cuda_stream)
        _check(rc, "ftb_gemm_bf16")
        return out
    rc = lib.ftb_gemm_bf16(_ptr(a), _ptr(b), _ptr(out), _ptr(c), _ptr(bias), c_int(M), c_int(N), c_int(K),
                           c_int(1 if trans_a else 0), c_int(0 if trans_b else 1), c_int(a.stride(0)),
                           c_int(b.stride(0)), c_int(out.stride(0)), c_int(c.stride(0) if c is not None else 0),
                           c_float(alpha), c_float(beta), c_int(1 if out.dtype == torch.float32 else 0), c_int(bn),
                           c_int(GEMM_MAX_CTAS), _stream())
    _check(rc, "ftb_gemm_bf16")
    return out


def grouped_gemm(x, w, offsets, *, trans_w=True, out=None, alpha=1.0, beta=0.0):
    """Expert-major grouped GEMM in one launch. ``x (R,K)``, ``w (E,N,K)`` (``trans_w``) or ``(E,K,N)``."""
    lib = load("gemm_tcgen05")
    E = w.shape[0]
    N = w.shape[1] if trans_w else w.shape[2]
    K = x.shape[1]
    assert w.is_contiguous() and x.stride(1) == 1 and offsets.dtype == torch.int32
    if out is None:
        out = torch.empty(x.shape[0], N, dtype=torch.bfloat16, device=x.device)
    rc = lib.ftb_grouped_gemm_bf16(_ptr(x), _ptr(w), _ptr(out), _ptr(out if beta != 0 else None), _ptr(offsets),
                                   c_int(E), c_int(x.shape[0]), c_int(N), c_int(K), c_int(0 if trans_w else 1),
                                   c_int(x.stride(0)), c_int(out.stride(0)), c_float(alpha), c_float(beta),
                                   c_int(1 if out.dtype == torch.float32 else 0), c_int(GEMM_MAX_CTAS), _stream())
    _check(rc, "ftb_grouped_gemm_bf16")
    return out


def grouped_wgrad(dy, x, offsets, gw, *, alpha=1.0, accumulate=True):
    """``gw[e] (N, Kd) (+)= alpha * dy[rows_e].T @ x[rows_e]`` for all experts in one launch (rows padded to 64)."""
    lib = load("gemm_tcgen05")
    E, N, Kd = gw.shape
    assert gw.is_contiguous() and dy.stride(1) == 1 and x.stride(1) == 1 and offsets.dtype == torch.int32
    rc = lib.ftb_grouped_wgrad_bf16(_ptr(dy), _ptr(x), _ptr(gw), _ptr(offsets), c_int(E), c_int(dy.shape[0]), c_int(N),
                                    c_int(Kd), c_int(dy.stride(0)), c_int(x.stride(0)), c_float(alpha),
                                    c_float(1.0 if accumulate else 0.0), c_int(1 if gw.dtype == torch.float32 else 0),
                                    c_int(GEMM_MAX_CTAS), _stream())
    _check(rc, "ftb_grouped_wgrad_bf16")
    return gw


# ------------------------------------------------------------------------ elementwise
def rmsnorm_fwd(x, w, eps):
    lib = load("elementwise")
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    T = x2.shape[0]
    y = torch.empty_like(x2)
    rstd = torch.empty(T, dtype=torch.float32, device=x.device)
    if D <= 512 and (w is None or w.dim() <= 2):
        heads_w = w.shape[0] if (w is not None and w.dim() == 2) else 1
        rc = lib.ftb_rmsnorm_small_fwd(_ptr(x2), _ptr(w), _ptr(y), _ptr(rstd), c_long(T), c_int(D), c_int(heads_w),
                                       c_float(eps), _stream())
    else:
        rc = lib.ftb_rmsnorm_fwd(_ptr(x2), _ptr(w), _ptr(y), _ptr(rstd), c_int(T), c_int(D), c_float(eps), _stream())
    _check(rc, "ftb_rmsnorm_fwd")
    return y.view(x.shape), rstd.view(x.shape[:-1])


def rmsnorm_bwd(dy, x, w, rstd, *, dx_add=None, emit_y=False, dw_out=None, dw_accumulate=True):
    """Returns ``(dx, dw, y)``. ``dw`` goes (accumulated) into ``dw_out`` when given, else a fresh fp32 vector."""
    lib = load("elementwise")
    D = x.shape[-1]
    x2, dy2 = x.reshape(-1, D), dy.reshape(-1, D)
    T = x2.shape[0]
    dx = torch.empty_like(x2)
    y = torch.empty_like(x2) if emit_y else None
    dw = None
    if D <= 512 and dx_add is None and not emit_y:
        if w is not None:
            dw = dw_out if dw_out is not None else torch.zeros(D, dtype=torch.float32, device=x.device)
            if dw_out is not None and not dw_accumulate:
                dw.zero_()
        rc = lib.ftb_rmsnorm_small_bwd(_ptr(dy2), _ptr(x2), _ptr(w), _ptr(rstd), _ptr(dx), _ptr(dw), c_long(T),
                                       c_int(D), _stream())
    else:
        lib.ftb_rmsnorm_bwd_blocks.restype = c_int
        part = None
        if w is not None:
            blocks = lib.ftb_rmsnorm_bwd_blocks(c_int(T))
            part = torch.empty(max(blocks, 1) * D, dtype=torch.float32, device=x.device)
            if dw_out is not None:
                dw, acc = dw_out, dw_accumulate
            else:
                dw, acc = torch.empty(D, dtype=torch.float32, device=x.device), False
        else:
            acc = False
        rc = lib.ftb_rmsnorm_bwd(_ptr(dy2), _ptr(x2), _ptr(w), _ptr(rstd),
                                 _ptr(dx_add.reshape(-1, D) if dx_add is not None else None), _ptr(dx), _ptr(y),
                                 _ptr(part), _ptr(dw), c_int(1 if acc else 0), c_int(T), c_int(D), _stream())
    _check(rc, "ftb_rmsnorm_bwd")
    return dx.view(x.shape), dw, (y.view(x.shape) if y is not None else None)


def rope(x, positions, inv_freq, *, out=None, inverse=False, mrope_sections=None):
    """Rotate-half RoPE on ``x (T,H,hd)`` (any token stride) into ``out`` (``x`` itself when None)."""
    lib = load("elementwise")
    out = x if out is None else out
    assert positions.dtype == torch.int32 and inv_freq.dtype == torch.float32
    T, H, hd = x.shape
    assert x.stride(2) == 1 and x.stride(1) == hd and out.stride(2) == 1 and out.stride(1) == hd
    half = inv_freq.numel()
    ps = 3 if positions.dim() == 2 else 1
    sh, sw = (mrope_sections[1], mrope_sections[2]) if mrope_sections is not None else (0, 0)
    rc = lib.ftb_rope(_ptr(x), c_long(x.stride(0)), _ptr(out), c_long(out.stride(0)), _ptr(positions),
                      _ptr(inv_freq), c_int(T), c_int(H), c_int(hd), c_int(half), c_int(1 if inverse else 0),
                      c_int(ps), c_int(sh), c_int(sw), _stream())
    _check(rc, "ftb_rope")
    return out


_KIND = {"swiglu": 0, "geglu": 1}


def glu_fwd(gate, up, kind="swiglu", out=None):
    lib = load("elementwise")
    T, F = gate.shape
    assert gate.stride(1) == 1 and up.stride(1) == 1 and gate.stride(0) == up.stride(0)
    if out is None:
        out = torch.empty(T, F, dtype=gate.dtype, device=gate.device)
    rc = lib.ftb_glu_fwd(_ptr(gate), _ptr(up), _ptr(out), c_long(T), c_int(F), c_int(gate.stride(0)),
                         c_int(out.stride(0)), c_int(_KIND[kind]), _stream())
    _check(rc, "ftb_glu_fwd")
    return out


def gemm_glu_supported(x, w, F: int, M_min: int = 512) -> bool:
    """Shapes the two-SM gated-FFN kernels take: bf16, contiguous rows, F a multiple of 128, enough rows for 256-row
    tiles to fill the GPU."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.stride(1) == 1 and F % 128 == 0 and x.shape[0] >= M_min
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.shape[1] % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_glu_fwd(x, w13, kind="swiglu", *, x13=None, act=None):
    """``x13 = x @ w13^T`` (``w13`` = stacked ``[W_gate ; W_up]``, (2F, K)) and ``act = act_fn(gate) * up`` from the
    same accumulator tile.  Returns ``(x13 (M, 2F), act (M, F))``."""
    lib = load("gemm_tcgen05")
    M, K = x.shape
    F = w13.shape[0] // 2
    assert w13.shape == (2 * F, K)
    if x13 is None:
        x13 = torch.empty(M, 2 * F, dtype=x.dtype, device=x.device)
    if act is None:
        act = torch.empty(M, F, dtype=x.dtype, device=x.device)
    assert x13.shape == (M, 2 * F) and x13.stride(1) == 1 and act.shape == (M, F) and act.stride(1) == 1
    rc = lib.ftb_gemm_glu_fwd(_ptr(x), _ptr(w13), _ptr(x13), _ptr(act), c_int(M), c_int(F), c_int(K),
                              c_int(x.stride(0)), c_int(w13.stride(0)), c_int(x13.stride(0)), c_int(act.stride(0)),
                              c_int(_KIND[kind]), c_int(GEMM_MAX_CTAS), _stream())
    _check(rc, "ftb_gemm_glu_fwd")
    return x13, act


def gemm_glu_bwd(dy, w2, x13, kind="swiglu", *, dx13=None, act=None):
    """Backward through the down projection's input and the gated activation in one kernel:
    ``dact = dy @ w2`` (``w2`` (d, F)) stays in tensor memory; returns ``(dx13 = [dgate | dup] (M, 2F), act (M, F))``."""
    lib = load("gemm_tcgen05")
    M, K = dy.shape
    F = w2.shape[1]
    assert w2.shape[0] == K and x13.shape == (M, 2 * F) and x13.stride(1) == 1
    if dx13 is None:
        dx13 = torch.empty(M, 2 * F, dtype=dy.dtype, device=dy.device)
    if act is None:
        act = torch.empty(M, F, dtype=dy.dtype, device=dy.device)
    rc = lib.ftb_gemm_glu_bwd(_ptr(dy), _ptr(w2), _ptr(x13), _ptr(dx13), _ptr(act), c_int(M), c_int(F), c_int(K),
                              c_int(dy.stride(0)), c_int(w2.stride(0)), c_int(x13.stride(0)), c_int(dx13.stride(0)),
                              c_int(act.stride(0)), c_int(_KIND[kind]), c_int(GEMM_MAX_CTAS), _stream())
    _check(rc, "ftb_gemm_glu_bwd")
    return dx13, act


def glu_bwd(dact, gate, up, kind="swiglu", *, dgate=None, dup=None, emit_act=True):
    lib = load("elementwise")
    T, F = gate.shape
    if dgate is None:
        buf = torch.empty(T, 2 * F, dtype=gate.dtype, device=gate.device)
        dgate, dup = buf[:, :F], buf[:, F:]
    act = torch.empty(T, F, dtype=gate.dtype, device=gate.device) if emit_act else None
    assert dact.stride(0) == F or not emit_act or dact.stride(0) == act.stride(0)
    rc = lib.ftb_glu_bwd(_ptr(dact), _ptr(gate), _ptr(up), _ptr(dgate), _ptr(dup), _ptr(act), c_long(T), c_int(F),
                         c_int(gate.stride(0)), c_int(dgate.stride(0)), c_int(dact.stride(0)), c_int(_KIND[kind]),
                         _stream())
    _check(rc, "ftb_glu_bwd")
    return dgate, dup, act


def topk_route_bwd(dw, logits, w, experts, mode="topk_then_softmax"):
    lib = load("elementwise")
    T, E = logits.shape
    K = experts.shape[1]
    dl = torch.empty(T, E, dtype=torch.float32, device=logits.device)
    rc = lib.ftb_topk_route_bwd(_ptr(dw.to(torch.float32).contiguous()), _ptr(logits.contiguous()),
                                _ptr(w.to(torch.float32).contiguous()), _ptr(experts.to(torch.int32).contiguous()),
                                _ptr(dl), c_int(T), c_int(E), c_int(K), c_int(0 if mode == "topk_then_softmax" else 1),
                                _stream())
    _check(rc, "ftb_topk_route_bwd")
    return dl


def load_balance_bwd_(dl, logits, counts, alpha: float, gscale: float):
    lib = load("elementwise")
    T, E = logits.shape
    rc = lib.ftb_load_balance_bwd(_ptr(logits), _ptr(counts), _ptr(dl), c_int(T), c_int(E), c_float(alpha),
                                  c_float(gscale), _stream())
    _check(rc, "ftb_load_balance_bwd")
    return dl


def glu_bwd_weighted(dact_u, gate, up, w_row, kind="swiglu", *, dgate, dup):
    """MoE expert backward through the gated activation with the per-row router weight folded in.
    Returns ``(act_w (T,F) = w_row * act, dw_row (T,) = sum(dact_u * act))``; writes ``dgate / dup``."""
    lib = load("elementwise")
    T, F = gate.shape
    assert dact_u.is_contiguous() and w_row.dtype == torch.float32 and dgate.stride(0) == dup.stride(0)
    act_w = torch.empty(T, F, dtype=gate.dtype, device=gate.device)
    dw_row = torch.empty(T, dtype=torch.float32, device=gate.device)
    rc = lib.ftb_glu_bwd_weighted(_ptr(dact_u), _ptr(gate), _ptr(up), _ptr(w_row), _ptr(dgate), _ptr(dup), _ptr(act_w),
                                  _ptr(dw_row), c_long(T), c_int(F), c_int(gate.stride(0)), c_int(dgate.stride(0)),
                                  c_int(_KIND[kind]), _stream())
    _check(rc, "ftb_glu_bwd_weighted")
    return act_w, dw_row


def softmax_ce_(logits, targets, *, grad_scale=1.0, softcap=0.0, loss_mask=None, ignore_index=-100):
    """In place: ``logits`` becomes dlogits. Returns per-token loss (fp32)."""
    lib = load("elementwise")
    T, V = logits.shape
    assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1 and targets.dtype == torch.int64
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    rc = lib.ftb_softmax_ce(_ptr(logits), _ptr(targets), _ptr(loss_mask), _ptr(loss), c_int(T), c_int(V),
                            c_long(logits.stride(0)), c_float(grad_scale), c_float(softcap), c_long(ignore_index),
                            _stream())
    _check(rc, "ftb_softmax_ce")
    return loss


def embedding_fwd(tokens, table, scale=1.0):
    lib = load("elementwise")
    T, D = tokens.numel(), table.shape[1]
    out = torch.empty(T, D, dtype=table.dtype, device=table.device)
    rc = lib.ftb_embedding_fwd(_ptr(tokens), _ptr(table), _ptr(out), c_int(T), c_int(D), c_float(scale), _stream())
    _check(rc, "ftb_embedding_fwd")
    return out


def embedding_bwd(dy, tokens, grad_table, scale=1.0):
    lib = load("elementwise")
    T, D = tokens.numel(), grad_table.shape[1]
    st, order = torch.sort(tokens.reshape(-1), stable=True)
    rc = lib.ftb_embedding_bwd(_ptr(st), _ptr(order), _ptr(dy), _ptr(grad_table), c_int(T), c_int(D), c_float(scale),
                               c_int(1 if grad_table.dtype == torch.float32 else 0), _stream())
    _check(rc, "ftb_embedding_bwd")


_DT = {torch.bfloat16: 0, torch.float32: 1}


def adamw_multi(params, grads, ms, vs, *, lrs, wds, beta1, beta2, eps, step, grad_scale=1.0):
    """One launch per <=24 tensors. All of ``params/grads/ms/vs`` are lists of contiguous CUDA tensors."""
    lib = load("elementwise")
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    for i0 in range(0, len(params), 24):
        sl = slice(i0, i0 + 24)
        P, G, M, V = params[sl], grads[sl], ms[sl], vs[sl]
        n = len(P)
        arr = lambda ts: (c_void_p * n)(*[t.data_ptr() for t in ts])
        rc = lib.ftb_adamw_multi(c_int(n), arr(P), arr(G), arr(M), arr(V), (c_long * n)(*[t.numel() for t in P]),
                                 (c_float * n)(*lrs[sl]), (c_float * n)(*wds[sl]),
                                 (c_int * n)(*[_DT[t.dtype] for t in P]), (c_int * n)(*[_DT[t.dtype] for t in G]),
                                 (c_int * n)(*[_DT[t.dtype] for t in M]), c_float(beta1), c_float(beta2),
                                 c_float(eps), c_float(bc1), c_float(bc2), c_float(grad_scale), _stream())
        _check(rc, "ftb_adamw_multi")


def topk_route(logits, k, mode):
    lib = load("elementwise")
    T, E = logits.shape
    w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    idx = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    rc = lib.ftb_topk_route(_ptr(logits.contiguous()), _ptr(w), _ptr(idx), c_int(T), c_int(E), c_int(k),
                            c_int(0 if mode == "topk_then_softmax" else 1), _stream())
    _check(rc, "ftb_topk_route")
    return w, idx


PLAN_CHUNK = 2048          # slots per block of the routing-plan kernels (csrc/moe.cu)


def moe_plan(experts: torch.Tensor, num_experts: int, pad: int, rows: int):
    """Routing plan of one chunk on the device (three launches, no host read): returns
    ``(row_src (rows,), inv (T,K), offsets (E+1,), counts (E,))``, all int32 (csrc/moe.cu ``ftb_moe_plan``)."""
    lib = load("moe")
    T, K = experts.shape
    n = T * K
    dev = experts.device
    ex = experts if (experts.dtype == torch.int32 and experts.is_contiguous()) else experts.to(torch.int32).contiguous()
    nb = max((n + PLAN_CHUNK - 1) // PLAN_CHUNK, 1)
    work = torch.empty(nb * num_experts, dtype=torch.int32, device=dev)
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=dev)
    inv = torch.empty(T, K, dtype=torch.int32, device=dev)
    row_src = torch.empty(rows, dtype=torch.int32, device=dev)
    rc = lib.ftb_moe_plan(_ptr(ex), c_long(n), c_int(num_experts), c_int(pad), c_long(rows), _ptr(work), _ptr(counts),
                          _ptr(offsets), _ptr(inv), _ptr(row_src), _stream())
    _check(rc, "ftb_moe_plan")
    return row_src, inv, offsets, counts


def ep_plan_count(experts: torch.Tensor, num_experts: int):
    """First half of the expert-parallel plan: ``(counts (E,) int32, work)`` of this rank's slots."""
    lib = load("moe")
    n = experts.numel()
    ex = experts if (experts.dtype == torch.int32 and experts.is_contiguous()) else experts.to(torch.int32).contiguous()
    nb = max((n + PLAN_CHUNK - 1) // PLAN_CHUNK, 1)
    work = torch.empty(nb * num_experts, dtype=torch.int32, device=experts.device)
    counts = torch.empty(num_experts, dtype=torch.int32, device=experts.device)
    rc = lib.ftb_ep_plan_count(_ptr(ex), c_long(n), c_int(num_experts), _ptr(work), _ptr(counts), _stream())
    _check(rc, "ftb_ep_plan_count")
    return counts, work, ex


def ep_plan_map(ex: torch.Tensor, shape, num_experts: int, table: torch.Tensor, world: int, rank: int, pad: int,
                capacity: int, work: torch.Tensor, overflow: torch.Tensor):
    """Second half: ``(slot_rank (T,K), slot_row (T,K), my_offsets (E/W+1,))`` from the all-gathered ``(W, E)`` int32
    count table; sets ``overflow`` (int32 scalar tensor) when a destination row exceeds ``capacity``."""
    lib = load("moe")
    T, K = shape
    dev = ex.device
    assert table.dtype == torch.int32 and table.is_contiguous() and overflow.dtype == torch.int32
    start = torch.empty(num_experts, dtype=torch.int32, device=dev)
    offs = torch.empty(num_experts // world + 1, dtype=torch.int32, device=dev)
    slot_rank = torch.empty(T, K, dtype=torch.int32, device=dev)
    slot_row = torch.empty(T, K, dtype=torch.int32, device=dev)
    rc = lib.ftb_ep_plan_map(_ptr(ex), c_long(T * K), c_int(num_experts), _ptr(table), c_int(world), c_int(rank),
                             c_int(pad), c_long(capacity), _ptr(work), _ptr(start), _ptr(offs), _ptr(slot_rank),
                             _ptr(slot_row), _ptr(overflow), _stream())
    _check(rc, "ftb_ep_plan_map")
    return slot_rank, slot_row, offs


def gather_rows(x, idx, weights=None, idx_div=1):
    lib = load("elementwise")
    R, D = idx.numel(), x.shape[1]
    out = torch.empty(R, D, dtype=x.dtype, device=x.device)
    rc = lib.ftb_gather_rows(_ptr(x), _ptr(idx), _ptr(weights), _ptr(out), c_long(R), c_int(D), c_int(idx_div),
                             _stream())
    _check(rc, "ftb_gather_rows")
    return out


def moe_combine(y, inv, weights, resid, out=None):
    lib = load("elementwise")
    T, K = inv.shape
    D = y.shape[1]
    if out is None:
        out = torch.empty(T, D, dtype=y.dtype, device=y.device)
    rc = lib.ftb_moe_combine(_ptr(y), _ptr(inv), _ptr(weights), _ptr(resid), _ptr(out), c_int(T), c_int(K), c_int(D),
                             _stream())
    _check(rc, "ftb_moe_combine")
    return out


def gated_rmsnorm_fwd(o, z, w, eps):
    lib = load("elementwise")
    D = o.shape[-1]
    y = torch.empty_like(o)
    rc = lib.ftb_gated_rmsnorm_fwd(_ptr(o), _ptr(z), _ptr(w), _ptr(y), c_long(o.numel() // D), c_int(D), c_float(eps),
                                   _stream())
    _check(rc, "ftb_gated_rmsnorm_fwd")
    return y


def l2norm_fwd(x, eps=1e-6):
    lib = load("elementwise")
    D = x.shape[-1]
    y = torch.empty_like(x)
    r = torch.empty(x.shape[:-1], dtype=torch.float32, device=x.device)
    rc = lib.ftb_l2norm_fwd(_ptr(x), _ptr(y), _ptr(r), c_long(x.numel() // D), c_int(D), c_float(eps), _stream())
    _check(rc, "ftb_l2norm_fwd")
    return y, r
