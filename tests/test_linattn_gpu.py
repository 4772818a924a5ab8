"""Gated DeltaNet kernels (csrc/gdn.cu, csrc/seqmix.cu) against plain PyTorch fp32 references (autograd for the
backward passes)."""

import pytest
import torch
import torch.nn.functional as F

from flextrain_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF, F32 = torch.bfloat16, torch.float32


def _rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / (b.norm() + 1e-12))


def _cu(lens):
    return torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("lens,with_init", [([37, 64, 5], True), ([200], False), ([1, 2, 3], True)])
def test_conv1d_fwd_bwd(lens, with_init):
    from flextrain_b200.ops import linattn_cuda as la
    torch.manual_seed(0)
    T, D, W, S = sum(lens), 192, 4, len(lens)
    wide = (torch.randn(T, D + 64, device=DEV) * 0.7).to(BF)
    x = wide[:, :D]                                              # row-strided view, as the block passes it
    w = (torch.randn(D, W, device=DEV) * 0.5).to(BF)
    init = (torch.randn(S, D, W - 1, device=DEV) * 0.7).to(BF) if with_init else None
    cu = _cu(lens)
    y, fin = la.conv1d_fwd(x, w, cu, init)
    xr = x.float().clone().requires_grad_(True)
    wr = w.float().clone().requires_grad_(True)
    ir = init.float().clone().requires_grad_(True) if with_init else None
    y_ref, fin_ref = ref.causal_conv1d_fwd(xr, wr, cu.cpu(), ir, activation=True)
    assert _rel(y, y_ref) < 1e-2 and _rel(fin, fin_ref) < 1e-2
    dy = (torch.randn(T, D, device=DEV) * 0.3).to(BF)
    dfin = (torch.randn(S, D, W - 1, device=DEV) * 0.3).to(BF)
    outs = torch.autograd.grad([y_ref, fin_ref], [xr, wr] + ([ir] if with_init else []), [dy.float(), dfin.float()])
    dx_wide = torch.zeros(T, D + 64, dtype=BF, device=DEV)
    dw = torch.zeros(D, W, dtype=F32, device=DEV)
    dinit = la.conv1d_bwd(x, w, cu, init, dy, dfin, dx_wide[:, :D], dw, want_dinit=with_init)
    assert _rel(dx_wide[:, :D], outs[0]) < 1.5e-2, _rel(dx_wide[:, :D], outs[0])
    assert float(dx_wide[:, D:].abs().max()) == 0.0
    assert _rel(dw, outs[1]) < 1.5e-2
    if with_init:
        assert _rel(dinit, outs[2]) < 1.5e-2


def test_l2norm_heads_fwd_bwd():
    from flextrain_b200.ops import linattn_cuda as la
    torch.manual_seed(1)
    T, H, D = 300, 4, 128
    wide = torch.randn(T, H * D + 96, device=DEV).to(BF)
    x2d = wide[:, : H * D]
    y, rn = la.l2norm_heads_fwd(x2d, H, D)
    xr = x2d.float().reshape(T, H, D).clone().requires_grad_(True)
    y_ref = xr * torch.rsqrt(xr.pow(2).sum(-1, keepdim=True) + 1e-6)
    assert _rel(y, y_ref) < 6e-3
    dy = torch.randn(T, H, D, device=DEV)
    (dx_ref,) = torch.autograd.grad(y_ref, xr, dy)
    dx = torch.zeros_like(wide)
    la.l2norm_heads_bwd(dy, x2d, rn, dx[:, : H * D], H, D)
    assert _rel(dx[:, : H * D].reshape(T, H, D), dx_ref) < 8e-3


def test_gated_rmsnorm_bwd():
    from flextrain_b200.ops import linattn_cuda as la
    torch.manual_seed(2)
    T, H, D, eps = 257, 4, 64, 1e-6
    o = torch.randn(T, H, D, device=DEV).to(BF)
    zwide = torch.randn(T, H * D + 32, device=DEV).to(BF)
    z2d = zwide[:, 32:]
    w = torch.rand(D, device=DEV) + 0.5
    dy = (torch.randn(T, H, D, device=DEV) * 0.5).to(BF)
    orr = o.float().clone().requires_grad_(True)
    zr = z2d.float().reshape(T, H, D).clone().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    y_ref = orr * torch.rsqrt(orr.pow(2).mean(-1, keepdim=True) + eps) * wr * F.silu(zr)
    do_ref, dz_ref, dw_ref = torch.autograd.grad(y_ref, [orr, zr, wr], dy.float())
    dz_wide = torch.zeros_like(zwide)
    dw = torch.zeros(D, dtype=F32, device=DEV)
    d_o = la.gated_rmsnorm_bwd(dy, o, z2d, w, dz_wide[:, 32:], dw, H, D, eps)
    assert _rel(d_o, do_ref) < 1e-2 and _rel(dz_wide[:, 32:].reshape(T, H, D), dz_ref) < 1e-2
    assert _rel(dw, dw_ref) < 1e-2


def _gdn_inputs(lens, HK, HV, dk, dv, seed=0):
    torch.manual_seed(seed)
    T = sum(lens)
    q = F.normalize(torch.randn(T, HK, dk, device=DEV), dim=-1).to(BF)
    k = F.normalize(torch.randn(T, HK, dk, device=DEV), dim=-1).to(BF)
    v = (torch.randn(T, HV, dv, device=DEV) * 0.5).to(BF)
    g = -torch.rand(T, HV, device=DEV) * 0.3
    beta = torch.rand(T, HV, device=DEV) * 0.9 + 0.05
    return q, k, v, g.contiguous(), beta.contiguous(), _cu(lens)


@pytest.mark.parametrize("lens,HK,HV,dk,dv,with_state", [
    ([50, 13, 64], 2, 4, 16, 16, True),
    ([130], 2, 2, 32, 48, False),
    ([33, 70], 1, 2, 64, 64, True),
    ([96], 2, 4, 128, 128, True),
])
def test_gdn_forward_backward(lens, HK, HV, dk, dv, with_state):
    from flextrain_b200.ops import linattn_cuda as la
    q, k, v, g, beta, cu = _gdn_inputs(lens, HK, HV, dk, dv)
    S = len(lens)
    s0 = (torch.randn(S, HV, dk, dv, device=DEV) * 0.2) if with_state else None
    o, fin, r = la.gdn_fwd(q, k, v, g, beta, cu, s0, want_r=True)
    leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v, g, beta)]
    s0r = s0.clone().requires_grad_(True) if with_state else None
    o_ref, fin_ref = ref.gated_delta_rule(*leaves, cu.cpu(), s0r)
    assert _rel(o, o_ref) < 1.5e-2, _rel(o, o_ref)
    assert _rel(fin, fin_ref) < 1e-3
    d_o = (torch.randn_like(o_ref) * 0.5).to(BF)
    dfin = torch.randn_like(fin_ref) * 0.1
    want = torch.autograd.grad([o_ref, fin_ref], leaves + ([s0r] if with_state else []), [d_o.float(), dfin])
    dq, dk_, dv_, dg, dbeta, ds0 = la.gdn_bwd(q, k, v, g, beta, cu, s0, fin, r, d_o, dstate_final=dfin)
    names = ["dq", "dk", "dv", "dg", "dbeta"]
    for name, got, ref_g in zip(names, (dq, dk_, dv_, dg, dbeta), want):
        assert _rel(got, ref_g) < 2e-2, (name, _rel(got, ref_g))
    if with_state:
        assert _rel(ds0, want[5]) < 1e-3


def test_gdn_block_cuda_matches_reference_path(monkeypatch):
    """The block's hand-written CUDA forward / backward against its own fp32 autograd formulation."""
    from flextrain_b200.core.activation_schema import ActivationSchema, ActivationSlot
    from flextrain_b200.core.layer import ChunkMeta, LayerContext
    from flextrain_b200.nn.blocks.linear_attn import GatedDeltaNetBlock, GDNConfig
    torch.manual_seed(3)
    cfg = GDNConfig(d_model=256, n_k_heads=2, n_v_heads=4, head_k_dim=64, head_v_dim=64)
    blk = GatedDeltaNetBlock(cfg, dtype=BF)
    P = {}
    for s in blk.tensor_specs():
        if s.name == "w_lin_norm" or s.name == "w_lin_dt_bias":
            P[s.name] = torch.ones(s.shape, device=DEV) + 0.1 * torch.randn(s.shape, device=DEV)
        elif s.name == "w_lin_A_log":
            P[s.name] = torch.randn(s.shape, device=DEV) * 0.3
        else:
            P[s.name] = (torch.randn(s.shape, device=DEV) * (0.3 if s.name == "w_lin_conv" else 0.06)).to(BF)
    lens = [100, 156]
    T = sum(lens)
    meta = ChunkMeta.build(0, [0, 1], lens, [0, 0], [False, False], DEV)
    h = (torch.randn(T, cfg.d_model, device=DEV)).to(BF)
    x = (torch.randn(T, cfg.d_model, device=DEV) * 0.1).to(BF)
    dx = (torch.randn(T, cfg.d_model, device=DEV) * 0.1).to(BF)
    sch = ActivationSchema(blk.activation_fields())
    res = {}
    for mode in ("cuda", "reference"):
        monkeypatch.setenv("FTB_GDN_BACKEND", mode)
        G = {"g_" + n[2:]: torch.zeros_like(p, dtype=F32) for n, p in P.items()}
        slot, ctx = ActivationSlot(sch, T), LayerContext()
        out = blk.fwd(h, x, meta, P, slot, ctx)
        dh = blk.bwd(dx, h, meta, P, G, slot, LayerContext())
        res[mode] = (out, dh, G)
    assert _rel(res["cuda"][0], res["reference"][0]) < 2e-2
    assert _rel(res["cuda"][1], res["reference"][1]) < 4e-2, _rel(res["cuda"][1], res["reference"][1])
    for name in res["cuda"][2]:
        a, b = res["cuda"][2][name], res["reference"][2][name]
        assert _rel(a, b) < 5e-2, (name, _rel(a, b))


def test_top_p_sampler_stays_in_nucleus():
    from flextrain_b200.ops import linattn_cuda as la
    torch.manual_seed(4)
    rows, V = 64, 5000
    logits = (torch.randn(rows, V, device=DEV) * 3).to(BF)
    g = torch.Generator(device=DEV).manual_seed(11)
    pick = la.top_p_sample(logits, 0.8, 1.0, generator=g)
    p = torch.softmax(logits.float(), -1)
    sp, si = torch.sort(p, dim=-1, descending=True)
    keep = (sp.cumsum(-1) - sp) < 0.8
    smallest = torch.where(keep, sp, torch.ones_like(sp)).min(-1).values       # smallest probability in the nucleus
    chosen_p = p.gather(1, pick.view(-1, 1)).squeeze(1)
    assert bool((chosen_p >= smallest * 0.98).all())
    # top_p -> 0 degenerates to the arg-max
    assert torch.equal(la.top_p_sample(logits, 1e-6, 1.0, generator=g), p.argmax(-1))


@pytest.mark.parametrize("T,HV", [(1000, 32), (77, 4), (4096, 48)])
def test_gate_prep_fwd_bwd(T, HV):
    """``beta = sigmoid(b)``, ``g = -exp(A_log) softplus(a + dt_bias)`` and their backward (incl. the two parameter
    gradients, reduced inside the kernel) against autograd on the same bf16 projection output."""
    import torch.nn.functional as F
    from flextrain_b200.ops import linattn_cuda as la
    torch.manual_seed(T)
    ba = (torch.randn(T, 2 * HV, device="cuda") * 2).to(torch.bfloat16)
    dtb = torch.randn(HV, device="cuda")
    alog = torch.randn(HV, device="cuda") * 0.5
    beta, g = la.gate_prep_fwd(ba, dtb, alog)
    baf = ba.float().requires_grad_(True)
    dtb_r, alog_r = dtb.clone().requires_grad_(True), alog.clone().requires_grad_(True)
    beta_w = torch.sigmoid(baf[:, :HV])
    g_w = -torch.exp(alog_r) * F.softplus(baf[:, HV:] + dtb_r)
    assert _rel(beta, beta_w) < 1e-5 and _rel(g, g_w) < 1e-5
    dbeta, dg = torch.randn(T, HV, device="cuda"), torch.randn(T, HV, device="cuda")
    (beta_w * dbeta + g_w * dg).sum().backward()
    d_alog, d_dtb = torch.zeros(HV, device="cuda"), torch.zeros(HV, device="cuda")
    dba = la.gate_prep_bwd(ba, dtb, alog, g, dbeta, dg, d_alog, d_dtb)
    assert _rel(dba, baf.grad) < 6e-3
    assert _rel(d_alog, alog_r.grad) < 1e-4 and _rel(d_dtb, dtb_r.grad) < 1e-4
