"""sm_100a kernels against the plain PyTorch fp32 reference of the same op."""

import pytest
import torch

from flextrain_b200 import ops
from flextrain_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV) * scale).to(dtype)


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (384, 1024, 320), (200, 264, 136), (1000, 72, 4096)])
def test_gemm_layouts(ta, tb, M, N, K):
    from flextrain_b200.ops import cuda as k
    if (ta and M % 8) or ((not tb) and N % 8):
        pytest.skip("leading dimension must be a multiple of 8")
    a = _rand(K, M) if ta else _rand(M, K)
    b = _rand(N, K) if tb else _rand(K, N)
    out = k.gemm(a, b, trans_a=ta, trans_b=tb)
    want = ref.gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32)
    assert _rel(out, want) < 5e-3, (ta, tb, M, N, K, _rel(out, want))
    assert k.device_error_words().get("gemm_tcgen05", 0) == 0


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_epilogue_alpha_beta_bias(out_dtype):
    from flextrain_b200.ops import cuda as k
    M, N, K = 512, 768, 1024
    a, b = _rand(M, K), _rand(N, K)
    c = _rand(M, N, dtype=out_dtype)
    bias = torch.randn(N, device=DEV)
    out = k.gemm(a, b, trans_b=True, alpha=0.5, beta=2.0, c=c, bias=bias, out_dtype=out_dtype)
    want = 0.5 * (a.float() @ b.float().t()) + 2.0 * c.float() + bias
    assert _rel(out, want) < 6e-3
    # in-place accumulate (wgrad pattern)
    acc = c.clone()
    k.gemm(a, b, trans_b=True, beta=1.0, out=acc)
    assert _rel(acc, a.float() @ b.float().t() + c.float()) < 6e-3


def test_gemm_large_matches_cublas():
    from flextrain_b200.ops import cuda as k
    M, N, K = 4096, 4096, 4096
    a, b = _rand(M, K), _rand(N, K)
    out = k.gemm(a, b, trans_b=True)
    want = a @ b.t()
    assert _rel(out, want) < 3e-3
    # strided A (a column slice of a wider buffer, as produced by a fused QKV projection)
    wide = _rand(M, 2 * K)
    out2 = k.gemm(wide[:, K:], b, trans_b=True)
    assert _rel(out2, wide[:, K:].float() @ b.float().t()) < 5e-3


@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 512), (1000, 520, 320), (4096, 4096, 1024)])
def test_gemm_two_sm_layouts(ta, tb, M, N, K):
    """The cta_group::2 kernel (a CTA pair per 256 x 256 tile), forced with bn=512, against the fp32 reference."""
    from flextrain_b200.ops import cuda as k
    a = _rand(K, M) if ta else _rand(M, K)
    b = _rand(N, K) if tb else _rand(K, N)
    out = k.gemm(a, b, trans_a=ta, trans_b=tb, bn=512)
    want = ref.gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32)
    assert _rel(out, want) < 5e-3, (ta, tb, M, N, K, _rel(out, want))
    assert k.device_error_words().get("gemm_tcgen05", 0) == 0


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_two_sm_epilogue(out_dtype):
    from flextrain_b200.ops import cuda as k
    M, N, K = 768, 1024, 512
    a, b = _rand(M, K), _rand(N, K)
    c = _rand(M, N, dtype=out_dtype)
    bias = torch.randn(N, device=DEV)
    out = k.gemm(a, b, trans_b=True, alpha=0.5, beta=2.0, c=c, bias=bias, out_dtype=out_dtype, bn=512)
    want = 0.5 * (a.float() @ b.float().t()) + 2.0 * c.float() + bias
    assert _rel(out, want) < 6e-3
    acc = c.clone()
    k.gemm(a, b, trans_b=True, beta=1.0, out=acc, bn=512)
    assert _rel(acc, a.float() @ b.float().t() + c.float()) < 6e-3


def test_grouped_gemm():
    from flextrain_b200.ops import cuda as k
    E, K, N = 8, 256, 384
    counts = [0, 128, 256, 0, 384, 128, 128, 256]
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    R = int(off[-1])
    x = _rand(R, K)
    w = _rand(E, N, K, scale=0.1)
    y = k.grouped_gemm(x, w, off, trans_w=True)
    want = ref.grouped_gemm(x, w, off, trans_w=True)
    assert _rel(y, want) < 6e-3
    w2 = _rand(E, K, N, scale=0.1)
    y2 = k.grouped_gemm(x, w2, off, trans_w=False)
    assert _rel(y2, ref.grouped_gemm(x, w2, off, trans_w=False)) < 6e-3


@pytest.mark.parametrize("T,D", [(7, 256), (300, 4096), (64, 5120)])
def test_rmsnorm(T, D):
    x, w = _rand(T, D), torch.rand(D, device=DEV) + 0.5
    y, r = ops.rmsnorm_fwd(x, w, 1e-5)
    yw, rw = ref.rmsnorm_fwd(x, w, 1e-5)
    assert _rel(y, yw) < 5e-3 and _rel(r, rw) < 1e-4
    dy, res = _rand(T, D), _rand(T, D)
    dw = torch.zeros(D, device=DEV)
    dx, yy = ops.rmsnorm_bwd(dy, x, w, r, dx_add=res, emit_y=True, dw_out=dw)
    dxw, dww = ref.rmsnorm_bwd(dy, x, w, rw)
    assert _rel(dx, dxw.float() + res.float()) < 6e-3
    assert _rel(dw, dww) < 5e-3 and _rel(yy, yw) < 5e-3


def test_rmsnorm_per_head():
    x, w = _rand(50, 8, 128), torch.rand(128, device=DEV) + 0.5
    y, r = ops.rmsnorm_fwd(x, w, 1e-6)
    yw, rw = ref.rmsnorm_fwd(x, w, 1e-6)
    assert _rel(y, yw) < 5e-3 and r.shape == (50, 8)
    dy = _rand(50, 8, 128)
    dw = torch.zeros(128, device=DEV)
    dx, _ = ops.rmsnorm_bwd(dy, x, w, r, dw_out=dw)
    dxw, dww = ref.rmsnorm_bwd(dy, x, w, rw)
    assert _rel(dx, dxw) < 6e-3 and _rel(dw, dww) < 5e-3


@pytest.mark.parametrize("partial", [1.0, 0.25])
def test_rope_strided_and_inverse(partial):
    T, H, hd = 77, 8, 128
    inv = ref.rope_inv_freq(hd, 5e5, rotary_dim=int(hd * partial)).to(DEV)
    pos = torch.randint(0, 100000, (T,), device=DEV, dtype=torch.int32)
    wide = _rand(T, 3 * H * hd)
    x = wide[:, H * hd: 2 * H * hd].unflatten(1, (H, hd))
    out = torch.empty(T, H, hd, device=DEV, dtype=torch.bfloat16)
    ops.rope(x, pos, inv, out=out)
    want = ref.rope_apply(x, pos, inv)
    assert _rel(out, want) < 6e-3
    back = ops.rope(out.clone(), pos, inv, inverse=True)
    assert _rel(back, x) < 1.5e-2


def test_rope_mrope():
    T, H, hd = 40, 4, 128
    inv = ref.rope_inv_freq(hd, 1e6).to(DEV)
    pos = torch.randint(0, 500, (T, 3), device=DEV, dtype=torch.int32)
    x = _rand(T, H, hd)
    out = ops.rope(x.clone(), pos, inv, mrope_sections=(24, 20, 20))
    want = ref.rope_apply(x, pos, inv, mrope_sections=(24, 20, 20))
    assert _rel(out, want) < 6e-3


@pytest.mark.parametrize("kind", ["swiglu", "geglu"])
def test_glu(kind):
    T, F = 333, 1024
    x13 = _rand(T, 2 * F)
    g, u = x13[:, :F], x13[:, F:]
    act = ops.glu_fwd(g, u, kind)
    assert _rel(act, ref.glu_fwd(g, u, kind)) < 5e-3
    d = _rand(T, F)
    dg, du, a2 = ops.glu_bwd(d, g, u, kind)
    wg, wu, wa = ref.glu_bwd(d, g, u, kind)
    assert _rel(dg, wg) < 6e-3 and _rel(du, wu) < 6e-3 and _rel(a2, wa) < 5e-3


@pytest.mark.parametrize("softcap", [0.0, 30.0])
def test_softmax_ce(softcap):
    T, V = 65, 32008
    z = _rand(T, V, scale=3.0)
    tgt = torch.randint(0, V, (T,), device=DEV)
    tgt[3] = -100
    mask = torch.ones(T, device=DEV)
    mask[5] = 0
    lw, dzw = ref.softmax_ce_fwd_bwd(z, tgt, grad_scale=0.01, softcap=softcap, loss_mask=mask)
    zz = z.clone()
    loss = ops.softmax_ce_(zz, tgt, grad_scale=0.01, softcap=softcap, loss_mask=mask)
    assert _rel(loss, lw) < 2e-3
    assert _rel(zz, dzw) < 1e-2
    assert float(loss[3]) == 0.0 and float(zz[5].abs().max()) == 0.0


def test_embedding():
    V, D, T = 1000, 512, 4096
    table = _rand(V, D)
    tok = torch.randint(0, 50, (T,), device=DEV)       # heavy duplication
    y = ops.embedding_fwd(tok, table, 2.0)
    assert _rel(y, ref.embedding_fwd(tok, table, 2.0)) < 5e-3
    dy = _rand(T, D)
    g = torch.zeros(V, D, device=DEV, dtype=torch.float32)
    ops.embedding_bwd(dy, tok, g, 2.0)
    gw = torch.zeros(V, D, dtype=torch.float32, device=DEV)
    ref.embedding_bwd(dy, tok, gw, 2.0)
    assert _rel(g, gw) < 1e-4


def test_adamw_multi():
    shapes = [(300, 40), (4096,), (128, 128), (7,)]
    P = [_rand(*s) for s in shapes]
    G = [_rand(*s, scale=0.1) for s in shapes]
    M = [torch.zeros(*s, device=DEV) for s in shapes]
    V = [torch.zeros(*s, device=DEV) for s in shapes]
    P2, M2, V2 = [p.clone() for p in P], [m.clone() for m in M], [v.clone() for v in V]
    for step in (1, 2):
        ops.adamw_multi(P, G, M, V, lrs=[1e-2] * 4, wds=[0.1, 0.0, 0.1, 0.0], beta1=0.9, beta2=0.95, eps=1e-8, step=step)
        for p, g, m, v, wd in zip(P2, G, M2, V2, [0.1, 0.0, 0.1, 0.0]):
            ref.adamw_step(p, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=wd, step=step)
    for p, q, m, n in zip(P, P2, M, M2):
        assert _rel(p, q) < 5e-3 and _rel(m, n) < 1e-5


@pytest.mark.parametrize("mode", ["topk_then_softmax", "softmax_then_topk"])
def test_topk_route(mode):
    T, E, K = 500, 128, 8
    z = _rand(T, E, scale=2.0)
    w, idx = ops.topk_route(z, K, mode)
    ww, wi = ref.topk_route(z, K, mode)
    assert torch.equal(idx.long(), wi.long())
    assert _rel(w, ww) < 1e-3
    # backward: dlogits from the gradient of the routing weights, against autograd through the fp32 reference
    dw = torch.randn(T, K, device=DEV)
    zr = z.float().clone().requires_grad_(True)
    wr, _ = ref.topk_route(zr, K, mode)
    (want,) = torch.autograd.grad(wr, zr, dw)
    got = ops.topk_route_bwd(dw, z, w, idx, mode)
    assert _rel(got, want) < 2e-3, _rel(got, want)


def test_moe_gather_combine():
    T, K, D, E = 300, 4, 256, 16
    idx = torch.randint(0, E, (T, K), device=DEV, dtype=torch.int32)
    plan = ref.moe_plan(idx, E, 128)
    x = _rand(T, D)
    xs = ops.gather_rows(x, plan.row_src, idx_div=K)
    src = plan.row_src.long()
    want = x[src.clamp(min=0) // K] * (src >= 0).unsqueeze(1)
    assert torch.equal(xs, want)
    w = torch.rand(T, K, device=DEV)
    y = _rand(plan.rows, D)
    out = ops.moe_combine(y, plan.inv, w, x)
    ref_out = (y[plan.inv.long()].float() * w.unsqueeze(-1)).sum(1) + x.float()
    assert _rel(out, ref_out) < 5e-3


def test_attention_library_matches_reference():
    H, KV, hd = 8, 2, 128
    lens_q, lens_k = [100, 64, 37], [100, 200, 37]
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device=DEV)
    q, k, v = _rand(sum(lens_q), H, hd), _rand(sum(lens_k), KV, hd), _rand(sum(lens_k), KV, hd)
    o, lse = ops.attention_fwd(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), scale=hd ** -0.5)
    ow, lw = ref.attention_fwd(q, k, v, cu_q, cu_k, scale=hd ** -0.5)
    assert _rel(o, ow) < 1e-2
    do = _rand(sum(lens_q), H, hd)
    dq, dk, dv = ops.attention_bwd(do, q, k, v, o, lse, cu_q, cu_k, max(lens_q), max(lens_k), scale=hd ** -0.5)
    wq, wk, wv = ref.attention_bwd(do, q, k, v, ow, lw, cu_q, cu_k, scale=hd ** -0.5)
    assert _rel(dq, wq) < 2e-2 and _rel(dk, wk) < 2e-2 and _rel(dv, wv) < 2e-2


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("case", ["equal", "prior_ctx", "ragged", "window", "softcap"])
def test_attention_tcgen05_fwd(hd, case):
    from flextrain_b200.ops import attention_cuda as fa
    H, KV = 8, 2
    window, softcap = 0, 0.0
    if case == "equal":
        lens_q, lens_k = [256, 256, 256], [256, 256, 256]
    elif case == "prior_ctx":
        lens_q, lens_k = [128], [640]
    elif case == "ragged":
        lens_q, lens_k = [100, 37, 300, 1], [100, 200, 300, 129]
    elif case == "softcap":                                # Gemma-2 logit soft-cap, deep in the tanh's curved range
        lens_q, lens_k, window, softcap = [100, 37, 300], [100, 200, 300], 160, 2.0
    else:
        lens_q, lens_k, window = [384, 200], [384, 456], 96
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device=DEV)
    Tq, Tk = sum(lens_q), sum(lens_k)
    wide = _rand(Tq, (H + 2 * KV) * hd)
    q = wide[:, : H * hd].unflatten(1, (H, hd))            # strided view, as in the fused QKV buffer
    k, v = _rand(Tk, KV, hd), _rand(Tk, KV, hd)
    o, lse = fa.fwd(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), scale=hd ** -0.5, window=window, softcap=softcap)
    ow, lw = ref.attention_fwd(q, k, v, cu_q, cu_k, scale=hd ** -0.5, window=window, softcap=softcap)
    from flextrain_b200.ops import cuda as kk
    assert kk.device_error_words().get("attention", 0) == 0
    assert _rel(o, ow) < 1e-2, (case, hd, _rel(o, ow))
    assert float((lse - lw).abs().max()) < 2e-2


@pytest.mark.parametrize("two_tiles", [1, 0])
@pytest.mark.parametrize("hd", [128, 64])
def test_attention_fwd_growing_row_maximum(hd, two_tiles):
    """Scores that jump by far more than 2^8 from one key tile to the next (later keys are scaled up), so the
    two-tile kernel has to rescale the output rows it keeps in tensor memory, next to rows whose maximum does not
    move (their keys are scaled down); also a jump of less than 2^8, which must NOT be rescaled yet give the same
    result.  The one-tile kernel (``ftb_attn_set_two_tiles(0)``) is checked on the same data."""
    from flextrain_b200.ops import attention_cuda as fa
    from flextrain_b200.ops import cuda as kk
    lib = kk.load("attention")
    H, KV, S = 4, 2, 640
    cu = torch.tensor([0, S, 2 * S + 70], dtype=torch.int32, device=DEV)
    T = 2 * S + 70
    q, k, v = _rand(T, H, hd), _rand(T, KV, hd), _rand(T, KV, hd)
    k = k.float()
    k[128:256] *= 1.5          # small growth: stays under the rescale threshold for most rows
    k[256:384] *= 8.0          # large growth
    k[384:512] *= 0.2          # maximum does not move
    k[512:S] *= 20.0           # large growth again
    k = k.to(torch.bfloat16)
    lib.ftb_attn_set_two_tiles(two_tiles)
    try:
        o, lse = fa.fwd(q, k, v, cu, cu, S + 70, S + 70, scale=hd ** -0.5)
    finally:
        lib.ftb_attn_set_two_tiles(1)
    ow, lw = ref.attention_fwd(q, k, v, cu, cu, scale=hd ** -0.5)
    assert kk.device_error_words().get("attention", 0) == 0
    assert _rel(o, ow) < 1e-2, (hd, two_tiles, _rel(o, ow))
    assert float((lse - lw).abs().max()) < 3e-2


def test_attention_fwd_one_tile_kernel_still_matches():
    """The one-query-tile-per-CTA forward kernel stays selectable; same ragged case as the default kernel's test."""
    from flextrain_b200.ops import attention_cuda as fa
    from flextrain_b200.ops import cuda as kk
    lib = kk.load("attention")
    H, KV, hd = 8, 2, 128
    lens_q, lens_k = [100, 37, 300, 1], [100, 200, 300, 129]
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device=DEV)
    q, k, v = _rand(sum(lens_q), H, hd), _rand(sum(lens_k), KV, hd), _rand(sum(lens_k), KV, hd)
    lib.ftb_attn_set_two_tiles(0)
    try:
        o, lse = fa.fwd(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), scale=hd ** -0.5)
    finally:
        lib.ftb_attn_set_two_tiles(1)
    ow, lw = ref.attention_fwd(q, k, v, cu_q, cu_k, scale=hd ** -0.5)
    assert _rel(o, ow) < 1e-2 and float((lse - lw).abs().max()) < 2e-2


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("case", ["equal", "prior_ctx", "ragged", "window", "softcap"])
def test_attention_tcgen05_bwd(hd, case):
    from flextrain_b200.ops import attention_cuda as fa
    from flextrain_b200.ops import cuda as kk
    H, KV = 8, 2
    window, softcap = 0, 0.0
    if case == "equal":
        lens_q, lens_k = [256, 256], [256, 256]
    elif case == "prior_ctx":
        lens_q, lens_k = [128], [640]
    elif case == "ragged":
        lens_q, lens_k = [100, 37, 300, 1], [100, 200, 300, 129]
    elif case == "softcap":
        lens_q, lens_k, window, softcap = [100, 37, 300], [100, 200, 300], 160, 2.0
    else:
        lens_q, lens_k, window = [384, 200], [384, 456], 96
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device=DEV)
    Tq, Tk = sum(lens_q), sum(lens_k)
    q, k, v = _rand(Tq, H, hd), _rand(Tk, KV, hd), _rand(Tk, KV, hd)
    do = _rand(Tq, H, hd)
    kw = dict(scale=hd ** -0.5, window=window, softcap=softcap)
    ow, lw = ref.attention_fwd(q, k, v, cu_q, cu_k, **kw)
    wq, wk, wv = ref.attention_bwd(do, q, k, v, ow, lw, cu_q, cu_k, **kw)
    o, lse = fa.fwd(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), **kw)
    dq, dk, dv = fa.bwd(do, q, k, v, o, lse, cu_q, cu_k, max(lens_q), max(lens_k), **kw)
    assert kk.device_error_words().get("attention", 0) == 0
    assert _rel(dq, wq) < 2e-2, (case, hd, "dq", _rel(dq, wq))
    assert _rel(dk, wk) < 2e-2, (case, hd, "dk", _rel(dk, wk))
    assert _rel(dv, wv) < 2e-2, (case, hd, "dv", _rel(dv, wv))


@pytest.mark.parametrize("shape", [(256, 512), (768, 256), (3, 128, 256)])
def test_muon_newton_schulz_on_tcgen05(shape):
    """Muon step whose Newton-Schulz GEMMs run on the tcgen05 kernel (bf16 iterates) against the fp32 reference."""
    from flextrain_b200 import ops
    torch.manual_seed(0)
    p = (torch.randn(*shape, device=DEV) * 0.05).to(torch.bfloat16)
    g = (torch.randn(*shape, device=DEV) * 0.01).to(torch.bfloat16)
    mom = torch.zeros(*shape, device=DEV, dtype=torch.bfloat16)
    p_ref, mom_ref = p.float().clone(), mom.float().clone()
    ref.muon_step(p_ref, g.float(), mom_ref, lr=0.02, beta=0.95, weight_decay=0.01)
    ops.muon_step(p, g, mom, lr=0.02, beta=0.95, weight_decay=0.01)
    assert _rel(mom, mom_ref) < 1e-2
    torch.manual_seed(0)
    start = (torch.randn(*shape, device=DEV) * 0.05).to(torch.bfloat16).float()
    step, step_ref = p.float() - start, p_ref - start
    cos = torch.nn.functional.cosine_similarity(step.flatten(), step_ref.flatten(), dim=0)
    assert float(cos) > 0.98, float(cos)
    assert _rel(p, p_ref) < 2e-2, _rel(p, p_ref)


@pytest.mark.parametrize("case", ["merge", "dy_b", "x_at", "ga", "gb"])
def test_gemm_rank16_lora_shapes(case):
    """The five products of a rank-16 LoRA linear (N = r or K = r or M = r): tiles mostly outside the matrix,
    filled with zeros by TMA.  All of them must run on the tensor-core kernel (strict mode raises otherwise)."""
    import os
    T, d_in, d_out, r = 1000, 512, 768, 16
    x, dy = _rand(T, d_in), _rand(T, d_out)
    A, B = _rand(r, d_in, scale=0.1), _rand(d_out, r, scale=0.1)
    os.environ["FTB_STRICT"] = "1"
    try:
        if case == "merge":       # W' = W + s * B @ A   (K = r, beta = 1, MN-major B operand)
            W = _rand(d_out, d_in)
            got = ops.gemm(B, A, alpha=2.0, beta=1.0, out=W.clone())
            want = W.float() + 2.0 * (B.float() @ A.float())
        elif case == "dy_b":      # (T, out) @ (out, r): N = r
            got, want = ops.gemm(dy, B), dy.float() @ B.float()
        elif case == "x_at":      # (T, in) @ (r, in)^T: N = r
            got, want = ops.gemm(x, A, trans_b=True), x.float() @ A.float().t()
        elif case == "ga":        # (T, r)^T @ (T, in): M = r, accumulated
            dyb = _rand(T, r)
            g0 = _rand(r, d_in)
            got = ops.gemm(dyb, x, trans_a=True, alpha=0.5, beta=1.0, out=g0.clone())
            want = g0.float() + 0.5 * (dyb.float().t() @ x.float())
        else:                     # (T, out)^T @ (T, r): N = r, accumulated
            xa = _rand(T, r)
            g0 = _rand(d_out, r)
            got = ops.gemm(dy, xa, trans_a=True, alpha=0.5, beta=1.0, out=g0.clone())
            want = g0.float() + 0.5 * (dy.float().t() @ xa.float())
    finally:
        os.environ["FTB_STRICT"] = "0"
    assert _rel(got, want) < 6e-3, (case, _rel(got, want))
    from flextrain_b200.ops import cuda as k
    assert k.device_error_words().get("gemm_tcgen05", 0) == 0


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_beta_on_mn_major_layouts(ta, tb, out_dtype):
    """alpha / beta accumulate with MN-major operands (the dgrad and wgrad layouts), one-SM and two-SM kernels."""
    from flextrain_b200.ops import cuda as k
    M, N, K = 640, 768, 520
    a = _rand(K, M) if ta else _rand(M, K)
    b = _rand(N, K) if tb else _rand(K, N)
    c = _rand(M, N, dtype=out_dtype)
    want = 0.25 * ref.gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32) + 1.5 * c.float()
    for bn in (0, 256, 512):
        out = k.gemm(a, b, trans_a=ta, trans_b=tb, alpha=0.25, beta=1.5, c=c, out_dtype=out_dtype, bn=bn)
        assert _rel(out, want) < 6e-3, (ta, tb, bn, _rel(out, want))


def test_grouped_gemm_ragged_experts():
    """Expert row segments that are not multiples of the 128-row tile (the rows past a segment's end belong to the
    next expert and must not be overwritten), including empty and one-row experts."""
    from flextrain_b200.ops import cuda as k
    E, K, N = 6, 192, 264
    counts = [5, 0, 130, 1, 257, 64]
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    R = int(off[-1])
    x = _rand(R, K)
    w = _rand(E, N, K, scale=0.1)
    y = k.grouped_gemm(x, w, off, trans_w=True)
    want = ref.grouped_gemm(x, w, off, trans_w=True)
    assert _rel(y, want) < 6e-3, _rel(y, want)
    for e in range(E):                       # per expert, so a small expert's error cannot hide in the total
        a, b = int(off[e]), int(off[e + 1])
        if b > a:
            assert _rel(y[a:b], want[a:b]) < 1e-2, (e, _rel(y[a:b], want[a:b]))


def test_strict_mode_refuses_library_paths():
    import os
    os.environ["FTB_STRICT"] = "1"
    try:
        a, b = _rand(64, 64), _rand(64, 60)             # N = 60 is not a multiple of 8
        with pytest.raises(ops.LibraryFallback):
            ops.gemm(a, b)
        ops.reset_backends_used()
        ops.gemm(_rand(64, 64), _rand(64, 64))
        assert ops.backends_used() == {"gemm": ["tcgen05"]}
    finally:
        os.environ["FTB_STRICT"] = "0"
    ops.gemm(a, b)                                       # outside strict mode the library path still works
    assert "library" in ops.backends_used()["gemm"]


@pytest.mark.parametrize("M,N,K,ta,tb", [(16, 4096, 16384, True, False), (4096, 16, 16384, True, False),
                                         (16, 1024, 5000, True, False), (256, 264, 8192, False, True),
                                         (1000, 16, 4096, False, False)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_split_k_small_outputs(M, N, K, ta, tb, out_dtype):
    """Small outputs with a long reduction take the split-K path (K cut into slices, fp32 slabs, ordered reduce with
    alpha / beta): same result as the fp32 reference, bit-identical between two runs."""
    from flextrain_b200.ops import cuda as k
    a = _rand(K, M, scale=0.3) if ta else _rand(M, K, scale=0.3)
    b = _rand(N, K, scale=0.3) if tb else _rand(K, N, scale=0.3)
    c = _rand(M, N, dtype=out_dtype)
    want = 0.5 * ref.gemm(a, b, trans_a=ta, trans_b=tb, out_dtype=torch.float32) + c.float()
    got = k.gemm(a, b, trans_a=ta, trans_b=tb, alpha=0.5, beta=1.0, c=c, out_dtype=out_dtype)
    again = k.gemm(a, b, trans_a=ta, trans_b=tb, alpha=0.5, beta=1.0, c=c, out_dtype=out_dtype)
    assert _rel(got, want) < 6e-3, _rel(got, want)
    assert torch.equal(got, again)
    assert k.device_error_words().get("gemm_tcgen05", 0) == 0


@pytest.mark.parametrize("case", ["causal_ragged", "prior_ctx_window"])
def test_attention_bwd_deterministic_dq(case):
    """With the key tiles' additions to each query tile ordered by the semaphore chain, two backward runs on the same
    inputs give bit-identical dQ (dK / dV accumulate in tensor memory and always are); the unordered mode agrees with
    it to fp32 round-off."""
    from flextrain_b200.ops import attention_cuda as fa
    from flextrain_b200.ops import cuda as kk
    H, KV, hd = 8, 2, 128
    if case == "causal_ragged":
        lens_q, lens_k, window = [1024, 700, 333, 1], [1024, 700, 333, 129], 0
    else:
        lens_q, lens_k, window = [512, 384], [1152, 456], 300
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device=DEV)
    q, k, v = _rand(sum(lens_q), H, hd), _rand(sum(lens_k), KV, hd), _rand(sum(lens_k), KV, hd)
    do = _rand(sum(lens_q), H, hd)
    kw = dict(scale=hd ** -0.5, window=window)
    o, lse = fa.fwd(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), **kw)
    runs = [fa.bwd(do, q, k, v, o, lse, cu_q, cu_k, max(lens_q), max(lens_k), deterministic=True, **kw) for _ in range(3)]
    for r in runs[1:]:
        assert torch.equal(r[0], runs[0][0]) and torch.equal(r[1], runs[0][1]) and torch.equal(r[2], runs[0][2])
    loose = fa.bwd(do, q, k, v, o, lse, cu_q, cu_k, max(lens_q), max(lens_k), deterministic=False, **kw)
    assert _rel(loose[0], runs[0][0]) < 1e-3
    ow, lw = ref.attention_fwd(q, k, v, cu_q, cu_k, **kw)
    wq, wk, wv = ref.attention_bwd(do, q, k, v, ow, lw, cu_q, cu_k, **kw)
    assert _rel(runs[0][0], wq) < 2e-2 and _rel(runs[0][1], wk) < 2e-2 and _rel(runs[0][2], wv) < 2e-2
    assert kk.device_error_words().get("attention", 0) == 0


def test_attention_bwd_deterministic_more_key_tiles_than_sms():
    """One 24,576-token sequence: 192 key-tile CTAs per KV head, more than fit on the GPU at once.  The ordered mode
    hands key tiles out from the last to the first, so a CTA only waits for CTAs that started before it: the run
    finishes at the unordered kernel's pace, keeps its order (error word stays zero) and repeats bit for bit."""
    from flextrain_b200.ops import attention_cuda as fa
    from flextrain_b200.ops import cuda as kk
    S, H, KV, hd = 24576, 2, 1, 128
    cu = torch.tensor([0, S], dtype=torch.int32, device=DEV)
    q, k, v, do = _rand(S, H, hd), _rand(S, KV, hd), _rand(S, KV, hd), _rand(S, H, hd)
    o, lse = fa.fwd(q, k, v, cu, cu, S, S, scale=hd ** -0.5)
    a = fa.bwd(do, q, k, v, o, lse, cu, cu, S, S, scale=hd ** -0.5, deterministic=True)
    b = fa.bwd(do, q, k, v, o, lse, cu, cu, S, S, scale=hd ** -0.5, deterministic=True)
    loose = fa.bwd(do, q, k, v, o, lse, cu, cu, S, S, scale=hd ** -0.5, deterministic=False)
    torch.cuda.synchronize()
    assert kk.device_error_words().get("attention", 0) == 0
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    assert _rel(loose[0], a[0]) < 1e-3 and _rel(loose[1], a[1]) < 1e-3


@pytest.mark.parametrize("kind", ["swiglu", "geglu"])
@pytest.mark.parametrize("M,K,F", [(512, 256, 128), (1000, 512, 640), (4096, 1024, 1792)])
def test_gemm_glu_fused_forward_and_backward(kind, M, K, F):
    """Gated-FFN GEMMs with the activation in the epilogue against the fp32 composition of GEMM and activation."""
    from flextrain_b200.ops import cuda as k
    x, w13, w2 = _rand(M, K, scale=0.5), _rand(2 * F, K, scale=K ** -0.5), _rand(K, F, scale=F ** -0.5)
    x13, act = ops.linear_glu_fwd(x, w13, kind)
    assert "ftb" in ops.backends_used().get("linear_glu_fwd", [])
    want13 = x.float() @ w13.float().t()
    assert _rel(x13, want13) < 5e-3
    # the activation is defined on the stored (bf16) projection, which is what the backward reads back
    want_act = ref.glu_fwd(x13[:, :F].float(), x13[:, F:].float(), kind)
    assert _rel(act, want_act) < 5e-3
    dy = _rand(M, K, scale=0.3)
    dx13, act2 = ops.linear_glu_bwd(dy, w2, x13, kind)
    assert "ftb" in ops.backends_used().get("linear_glu_bwd", [])
    dact = dy.float() @ w2.float()
    dg, du, a = ref.glu_bwd(dact, x13[:, :F].float(), x13[:, F:].float(), kind)
    assert _rel(dx13[:, :F], dg) < 6e-3 and _rel(dx13[:, F:], du) < 6e-3 and _rel(act2, a) < 5e-3
    assert k.device_error_words().get("gemm_tcgen05", 0) == 0


def test_tensor_map_cache_reuses_encodings_and_keeps_results():
    """Repeated GEMMs on the same buffers hit the tensor-map cache; a new shape at a cached address re-encodes."""
    from flextrain_b200.ops import cuda as k
    a, b = _rand(512, 256), _rand(384, 256)
    out = torch.empty(512, 384, dtype=torch.bfloat16, device=DEV)
    k.gemm(a, b, trans_b=True, out=out)
    s0 = k.tmap_cache_stats()
    for _ in range(5):
        k.gemm(a, b, trans_b=True, out=out)
    s1 = k.tmap_cache_stats()
    assert s1["hits"] - s0["hits"] >= 10 and s1["misses"] == s0["misses"], (s0, s1)
    assert _rel(out, a.float() @ b.float().t()) < 5e-3
    a2 = a.view(-1)[: 256 * 256].view(256, 256)                 # same base address, different extent
    out2 = k.gemm(a2, b, trans_b=True)
    assert k.tmap_cache_stats()["misses"] > s1["misses"]
    assert _rel(out2, a2.float() @ b.float().t()) < 5e-3


@pytest.mark.parametrize("hd", [128, 64])
def test_attention_bwd_dq_drains_agree(hd):
    """dQ leaves the SM either as tiled reduce-adds from shared memory (default) or as per-thread vector reductions;
    with the ordered mode on, both add the same fp32 partial tiles in the same order, so dQ agrees bit for bit."""
    from flextrain_b200.ops import attention_cuda as fa
    from flextrain_b200.ops import cuda as kk
    H, KV = 4, 2
    lens_q, lens_k = [640, 300, 1], [640, 428, 129]
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device=DEV)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device=DEV)
    q, k, v = _rand(sum(lens_q), H, hd), _rand(sum(lens_k), KV, hd), _rand(sum(lens_k), KV, hd)
    do = _rand(sum(lens_q), H, hd)
    kw = dict(scale=hd ** -0.5)
    o, lse = fa.fwd(q, k, v, cu_q, cu_k, max(lens_q), max(lens_k), **kw)
    lib = kk.load("attention")
    try:
        a = fa.bwd(do, q, k, v, o, lse, cu_q, cu_k, max(lens_q), max(lens_k), deterministic=True, **kw)
        lib.ftb_attn_set_dq_bulk(0)
        b = fa.bwd(do, q, k, v, o, lse, cu_q, cu_k, max(lens_q), max(lens_k), deterministic=True, **kw)
    finally:
        lib.ftb_attn_set_dq_bulk(1)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    ow, lw = ref.attention_fwd(q, k, v, cu_q, cu_k, **kw)
    wq, _, _ = ref.attention_bwd(do, q, k, v, ow, lw, cu_q, cu_k, **kw)
    assert _rel(a[0], wq) < 2e-2
    assert kk.device_error_words().get("attention", 0) == 0
