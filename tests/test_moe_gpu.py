"""MoE on a B200: the grouped weight-gradient kernel and a small Qwen3-MoE / OLMoE model against the CPU oracle."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.ops import reference as ref
from conftest import build_tiny

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_grouped_wgrad(gdtype):
    from flextrain_b200.ops import cuda as k
    E, N, Kd = 6, 384, 256
    counts = [128, 0, 256, 128, 384, 0]
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    R = int(off[-1])
    dy = (torch.randn(R, N, device="cuda") * 0.1).to(torch.bfloat16)
    x = (torch.randn(R, Kd, device="cuda") * 0.1).to(torch.bfloat16)
    g0 = (torch.randn(E, N, Kd, device="cuda") * 0.01).to(gdtype)
    want = g0.clone().float()
    ref.grouped_wgrad(dy, x, off, want, alpha=0.5)
    got = g0.clone()
    k.grouped_wgrad(dy, x, off, got, alpha=0.5)
    assert k.device_error_words().get("gemm_tcgen05", 0) == 0
    assert _rel(got, want) < 8e-3
    assert torch.equal(got[1], g0[1]) and torch.equal(got[5], g0[5])       # empty experts untouched


@pytest.mark.parametrize("arch", ["qwen3_moe", "olmoe"])
def test_moe_model_bf16_tracks_fp32(arch):
    dims = dict(vocab_size=512, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=128,
                num_routed_experts=8, top_k=2, num_shared_experts=0, is_causal=True)
    cpu = build_tiny(arch=arch, dims=dims, max_seq_len=128, batch_tokens=512)
    gpu = build_tiny(arch=arch, dims=dims, max_seq_len=128, batch_tokens=512, device="cuda:0", dtype=torch.bfloat16)
    src = {(s, l, n): t for s, l, n, t in cpu.named_master_params()}
    for s, l, n, t in gpu.named_master_params():
        t.copy_(src[(s, l, n)].to(t.dtype))
    for (s, l, n, t), (_, _, _, g) in zip(cpu.named_master_params(), gpu.named_master_params()):
        t.copy_(g.float().cpu())
    data = ft.SyntheticTokenSource(512, 128, seed=3)
    for step in range(2):
        seqs = data.get_sequences(512)
        a = cpu.fwd_bwd(seqs)
        b = gpu.fwd_bwd(seqs)
        assert abs(a.loss - b.loss) < 0.05, (step, a.loss, b.loss)
        if step == 0:
            for l in range(2):
                ga, gb = cpu.buffers.grads(l), gpu.buffers.grads(l)
                for name in ("g_up", "g_down", "g_q"):
                    cos = torch.nn.functional.cosine_similarity(ga[name].flatten().float(),
                                                                gb[name].flatten().float().cpu(), dim=0)
                    assert cos > 0.98, (arch, l, name, float(cos))
        cpu.step(); gpu.step()
