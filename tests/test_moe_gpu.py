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


@pytest.mark.parametrize("T,K,E,pad,skew", [(300, 2, 8, 128, False), (4096, 8, 128, 128, False), (5000, 8, 64, 128, True),
                                            (16384, 8, 128, 128, True), (77, 4, 256, 64, False), (2049, 1, 60, 1, False)])
def test_device_routing_plan_equals_stable_sort(T, K, E, pad, skew):
    """The three plan kernels against the plain tensor-op statement (library stable sort + cumsum): identical row
    layout, inverse map and padded offsets, also when a few experts take most slots or some take none."""
    from flextrain_b200 import ops
    from flextrain_b200.ops import reference as ref
    g = torch.Generator(device="cuda").manual_seed(T + E)
    if skew:
        p = torch.ones(E, device="cuda"); p[:3] = 200.0; p[5] = 0.0
        idx = torch.multinomial(p.expand(T, E), K, generator=g).to(torch.int32)
    else:
        idx = torch.randint(0, E, (T, K), device="cuda", generator=g, dtype=torch.int32)
    got = ops.moe_plan(idx, E, pad)
    want = ref.moe_plan(idx, E, pad)
    assert got.rows == want.rows
    assert torch.equal(got.offsets.long(), want.offsets.long())
    assert torch.equal(got.inv.long(), want.inv.long())
    assert torch.equal(got.row_src.long(), want.row_src.long())
    assert ops.backends_used().get("moe_plan") == ["ftb"]


@pytest.mark.parametrize("W,rank", [(2, 0), (4, 3), (8, 5)])
def test_expert_parallel_plan_kernels_against_tensor_ops(W, rank):
    """Expert-parallel destination rows on one GPU: the count table of the other ranks is made up, this rank's row is
    the real count of its slots; the scan + map kernels must give the rows of ``ExpertParallel.plan_from_table``."""
    from flextrain_b200.ops import cuda as k
    from flextrain_b200.parallel.ep import PAD, ExpertParallel
    T, K, E = 3000, 8, 64
    g = torch.Generator(device="cuda").manual_seed(W * 10 + rank)
    idx = torch.randint(0, E, (T, K), device="cuda", generator=g, dtype=torch.int32)
    w = torch.rand(T, K, device="cuda", generator=g)
    counts, work, ex = k.ep_plan_count(idx, E)
    assert torch.equal(counts.long(), torch.bincount(idx.reshape(-1).long(), minlength=E))
    table = torch.randint(0, 700, (W, E), device="cuda", generator=g, dtype=torch.int32)
    table[rank] = counts
    ep = ExpertParallel(rank, W, "cuda", None, backend="collective", capacity_factor=float(W))
    want = ep.plan_from_table(idx, w, E, table.long())
    cap = ep.capacity(T, K, E)
    over = torch.zeros((), dtype=torch.int32, device="cuda")
    slot_rank, slot_row, offs = k.ep_plan_map(ex, (T, K), E, table.contiguous(), W, rank, PAD, cap, work, over)
    assert torch.equal(slot_rank, want.slot_rank) and torch.equal(slot_row, want.slot_row)
    assert torch.equal(offs, want.offsets) and int(over) == 0
    # a capacity that is too small is flagged, never silently accepted
    small = int(want.slot_row.max()) - 5
    k.ep_plan_map(ex, (T, K), E, table.contiguous(), W, rank, PAD, small, work, over)
    assert int(over) == 1


@pytest.mark.parametrize("T,E,K", [(300, 8, 2), (2048, 128, 8), (77, 60, 4)])
def test_load_balance_gradient_kernel(T, E, K):
    """The auxiliary load-balance gradient added into dlogits by one kernel, against the tensor-op statement."""
    from flextrain_b200 import ops
    torch.manual_seed(E)
    logits = (torch.randn(T, E, device="cuda") * 2).to(torch.bfloat16)
    idx = torch.topk(logits.float(), K, dim=-1).indices.to(torch.int32)
    dl0 = torch.randn(T, E, device="cuda")
    alpha, total = 0.05, 4 * T
    got = ops.load_balance_bwd_(dl0.clone(), logits, idx, alpha, total)
    p = torch.softmax(logits.float(), -1)
    f = torch.bincount(idx.reshape(-1).long(), minlength=E).float()
    gvec = f / idx.numel() * E / total
    want = dl0 + alpha * p * (gvec - (p * gvec).sum(-1, keepdim=True))
    assert _rel(got, want) < 1e-5
    assert _rel(got - dl0, want - dl0) < 2e-3
