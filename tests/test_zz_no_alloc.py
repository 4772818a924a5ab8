"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of the library run where device allocation is not available at call time (a pre-partitioned memory
budget, a host application that owns the allocator, a loop that must not risk an allocator-induced sync).  For
them ``ftb_rmsnorm_bwd_noalloc`` keeps its reduction workspace in a static device array.  This test calls it
twice in a row (the workspace is shared and keeps the previous call's contents) and compares every output with
the regular entry point, ``ftb_rmsnorm_bwd``, which takes a caller-allocated workspace.

The file name sorts last so that a run that stops at the first failure has already run every other test.
"""
import ctypes
from ctypes import c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _call_noalloc(lib, dy, x, w, rstd, dx_add, emit_y, dw, accumulate):
    T, D = x.shape
    dx = torch.empty_like(x)
    y = torch.empty_like(x) if emit_y else None
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.ftb_rmsnorm_bwd_noalloc(_ptr(dy), _ptr(x), _ptr(w), _ptr(rstd), _ptr(dx_add), _ptr(dx), _ptr(y), _ptr(dw),
                                     c_int(1 if accumulate else 0), c_int(T), c_int(D), stream)
    return rc, dx, y


def test_noalloc_matches_regular_entry_point_twice():
    from flextrain_b200.ops import cuda as k
    lib = k.load("noalloc")
    lib.ftb_noalloc_strerror.restype = ctypes.c_char_p
    dev = "cuda"
    torch.manual_seed(0)
    # two different shapes back to back: the second call meets the first call's leftovers in the workspace
    for call, (T, D) in enumerate([(777, 4096), (129, 2048)]):
        x = torch.randn(T, D, device=dev).to(torch.bfloat16)
        dy = torch.randn(T, D, device=dev).to(torch.bfloat16)
        res = torch.randn(T, D, device=dev).to(torch.bfloat16)
        w = torch.rand(D, device=dev) + 0.5
        _, rstd = k.rmsnorm_fwd(x, w, 1e-5)
        base = torch.randn(D, device=dev)
        dw_ref, dw_new = base.clone(), base.clone()
        dx_ref, _, y_ref = k.rmsnorm_bwd(dy, x, w, rstd, dx_add=res, emit_y=True, dw_out=dw_ref, dw_accumulate=True)
        rc, dx_new, y_new = _call_noalloc(lib, dy, x, w, rstd, res, True, dw_new, True)
        assert rc == 0, lib.ftb_noalloc_strerror(rc)
        torch.cuda.synchronize()
        assert _rel(dx_new, dx_ref) < 6e-3, (call, _rel(dx_new, dx_ref))
        assert _rel(y_new, y_ref) < 5e-3
        assert _rel(dw_new, dw_ref) < 5e-3, (call, _rel(dw_new, dw_ref))


def test_noalloc_rejects_oversized_rows():
    from flextrain_b200.ops import cuda as k
    lib = k.load("noalloc")
    lib.ftb_noalloc_strerror.restype = ctypes.c_char_p
    T, D = 4, 16384
    x = torch.zeros(T, D, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(T, device="cuda")
    rc, _, _ = _call_noalloc(lib, x, x, None, rstd, None, False, None, False)
    assert rc == -3
    assert b"8192" in lib.ftb_noalloc_strerror(rc)
    rc, _, _ = _call_noalloc(lib, x[:, :12], x[:, :12], None, rstd, None, False, None, False)
    assert rc == -2


@pytest.mark.parametrize("T,D,with_w,with_dw", [(3, 8192, True, True), (200, 1024, False, False), (65, 4096, True, False)])
def test_noalloc_matches_fp32_reference(T, D, with_w, with_dw):
    """Against the plain PyTorch fp32 statement of the op (``ops.reference.rmsnorm_bwd``), at the widest row the
    built-in workspace takes (every per-thread vector live), without a gain vector, and without a weight gradient."""
    from flextrain_b200.ops import cuda as k
    from flextrain_b200.ops import reference as ref
    lib = k.load("noalloc")
    lib.ftb_noalloc_strerror.restype = ctypes.c_char_p
    torch.manual_seed(1)
    x = torch.randn(T, D, device="cuda").to(torch.bfloat16)
    dy = torch.randn(T, D, device="cuda").to(torch.bfloat16)
    w = (torch.rand(D, device="cuda") + 0.5) if with_w else None
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
    dw = torch.zeros(D, device="cuda") if with_dw else None
    rc, dx, y = _call_noalloc(lib, dy, x, w, rstd, None, True, dw, False)
    assert rc == 0, lib.ftb_noalloc_strerror(rc)
    torch.cuda.synchronize()
    dx_ref, dw_ref = ref.rmsnorm_bwd(dy.float(), x.float(), w, rstd)
    y_ref = x.float() * rstd.unsqueeze(-1) * (w if with_w else 1.0)
    assert _rel(dx, dx_ref) < 6e-3, _rel(dx, dx_ref)
    assert _rel(y, y_ref) < 5e-3
    if with_dw:
        assert _rel(dw, dw_ref) < 5e-3, _rel(dw, dw_ref)


def test_noalloc_rejects_bad_pointers_before_any_launch():
    """An unaligned view, a missing required tensor, or a weight gradient without weights come back as an error code
    from the host-side checks; nothing runs on the GPU."""
    from flextrain_b200.ops import cuda as k
    lib = k.load("noalloc")
    lib.ftb_noalloc_strerror.restype = ctypes.c_char_p
    T, D = 4, 1024
    flat = torch.zeros(T * D + 8, device="cuda", dtype=torch.bfloat16)
    x = flat[: T * D].view(T, D)
    odd = flat[1: T * D + 1].view(T, D)                     # 2-byte offset: not 16-byte aligned
    rstd = torch.ones(T, device="cuda")
    dw = torch.zeros(D, device="cuda")
    rc, _, _ = _call_noalloc(lib, odd, x, None, rstd, None, False, None, False)
    assert rc == -5 and b"16-byte" in lib.ftb_noalloc_strerror(rc)
    rc, _, _ = _call_noalloc(lib, x, x, None, rstd, None, False, dw, False)        # dw without w
    assert rc == -5
    rc, _, _ = _call_noalloc(lib, x, x, None, None, None, False, None, False)      # rstd missing
    assert rc == -5
    torch.cuda.synchronize()
