"""Every architecture family on CPU in fp32: hand-written forward/backward against autograd on the naive model."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.bench.naive import clone_params, naive_loss
from conftest import build_tiny

BASE = dict(vocab_size=512, n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, expert_dim=256, ffn_dim=256,
            num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
MOE = dict(BASE, expert_dim=64, num_routed_experts=8, top_k=2)

CASES = {
    "llama": ("llama", BASE, {}),
    "llama3_rope_scaling": ("llama", BASE, {"rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                             "high_freq_factor": 4.0,
                                                             "original_max_position_embeddings": 64}}),
    "mistral_sliding": ("mistral", BASE, {"sliding_window": 16, "layer_pattern": "S"}),
    "qwen2_bias": ("qwen2", BASE, {}),
    "qwen3_qknorm": ("qwen3", BASE, {}),
    "qwen3_moe": ("qwen3_moe", MOE, {}),
    "olmoe": ("olmoe", MOE, {}),
    "gemma2": ("gemma2", BASE, {"sliding_window": 16, "layer_pattern": "SF", "attn_softcap": 50.0, "final_softcap": 30.0}),
    "gemma3": ("gemma3", BASE, {"sliding_window": 16, "layer_pattern": "SF"}),
    "gemma4": ("gemma4", BASE, {"sliding_window": 16, "layer_pattern": "SF"}),
    "qwen3_5_moe": ("qwen3_5_moe", dict(MOE, num_shared_experts=1, shared_dim=64),
                    {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 4, "head_k_dim": 16, "head_v_dim": 16}}),
    "qwen3_next": ("qwen3_next", dict(MOE, num_shared_experts=1, shared_dim=64),
                   {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 4, "head_k_dim": 16, "head_v_dim": 16}}),
    "qwen3_5_dense": ("qwen3_5", BASE,
                      {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 2, "head_k_dim": 16, "head_v_dim": 32}}),
}


def _check(am, seqs, rtol=3e-4, atol=3e-6):
    P = clone_params(am)
    loss = naive_loss(am, P, seqs)
    loss.backward()
    st = am.fwd_bwd(seqs)
    assert abs(st.loss - float(loss.detach())) < 2e-4, (st.loss, float(loss))
    bm = am.buffers
    n = 0
    for (scope, l, name), p in P.items():
        g = {"embed": bm.embed_grads(), "head": bm.head_grads()}.get(scope) or bm.grads(l)
        gname = "g_" + name[2:] if name.startswith("w_") else "g_" + name
        if gname not in g:
            continue
        want = p.grad if p.grad is not None else torch.zeros_like(p)
        if am.head.tied and name in ("w_tok_embeddings", "w_head_proj"):
            # one tied parameter: the engine folds the head's share into the embedding's gradient
            both = P[("embed", -1, "w_tok_embeddings")].grad + P[("head", -1, "w_head_proj")].grad
            want = both if name == "w_tok_embeddings" else torch.zeros_like(p)
        torch.testing.assert_close(g[gname].float(), want, rtol=rtol, atol=atol, msg=f"{scope}/{l}/{name}")
        n += 1
    assert n > 5


@pytest.mark.parametrize("case", sorted(CASES))
def test_family_gradients(case):
    arch, dims, hyper = CASES[case]
    am = build_tiny(arch=arch, dims=dims, hyper=hyper, max_seq_len=48, batch_tokens=96)
    torch.manual_seed(0)
    # perturb norm weights and biases so their gradients are exercised away from the init point
    for scope, l, name, t in am.named_master_params():
        if "norm" in name or name.startswith("b_") or "dt_bias" in name or "A_log" in name or "scalar" in name:
            t.add_(torch.randn_like(t) * 0.1)
    seqs = ft.SyntheticTokenSource(dims["vocab_size"], [48, 40], seed=2).get_sequences(96)
    _check(am, seqs)


def test_lora_gradients():
    am = build_tiny(dims=BASE, max_seq_len=48, batch_tokens=96, lora_targets="all", lora_rank=4, lora_alpha=8.0,
                    lora_adapter_compute_dtype=torch.float32, lora_adapter_master_dtype=torch.float32,
                    lora_adapter_grad_dtype=torch.float32, lora_adapter_opt_state_dtype=torch.float32)
    torch.manual_seed(0)
    for scope, l, name, t in am.named_master_params():
        if name.endswith("_lora_b"):
            t.copy_(torch.randn_like(t) * 0.05)
    seqs = ft.SyntheticTokenSource(512, 48, seed=3).get_sequences(96)
    P = clone_params(am)
    naive_loss(am, P, seqs).backward()
    am.fwd_bwd(seqs)
    checked = 0
    for l in range(2):
        g = am.buffers.grads(l)
        assert "g_q" not in g, "base weights must be frozen under LoRA"
        for name in ("w_q", "w_v", "w_o", "w_1", "w_2", "w_3", "w_k"):
            for ab in ("_lora_a", "_lora_b"):
                torch.testing.assert_close(g["g_" + name[2:] + ab].float(), P[("layer", l, name + ab)].grad,
                                           rtol=3e-4, atol=3e-6, msg=f"{l}/{name}{ab}")
                checked += 1
    assert checked == 28
    assert am.step() == 0


@pytest.mark.parametrize("arch", ["qwen3_moe", "olmoe"])
def test_moe_load_balance_gradient(arch):
    """The auxiliary load-balance loss ``alpha * E * sum_e f_e * mean_t p_te`` (routed fractions ``f`` held constant,
    flextrain/nn/blocks/ffn_moe.py:95-110) only exists as a gradient in the engine; with one sequence per chunk it must
    equal autograd's gradient of cross-entropy + that term on the naive model."""
    am = build_tiny(arch=arch, dims=MOE, hyper={"aux_loss_alpha": 0.05}, max_seq_len=48, batch_tokens=96,
                    ws=ft.WorkingSetConfig.simple(max_seq_len=48, max_global_batch_tokens=96, chunk=48))
    assert am.layers[0].moe.cfg.aux_loss_alpha == 0.05
    torch.manual_seed(0)
    for scope, l, name, t in am.named_master_params():
        if "norm" in name or "router" in name:
            t.add_(torch.randn_like(t) * 0.1)
    seqs = ft.SyntheticTokenSource(512, 48, seed=2).get_sequences(96)
    P = clone_params(am)
    total, active, aux = 0.0, 0, []
    from flextrain_b200.bench.naive import naive_forward
    for s in seqs:
        z = naive_forward(am, P, s.tokens, aux=aux)
        total = total + torch.nn.functional.cross_entropy(z, s.targets, ignore_index=-100, reduction="sum")
        active += int((s.targets != -100).sum())
    n_tokens = sum(len(s) for s in seqs)
    assert len(aux) == 2 * len(seqs)
    loss = total / active + sum(aux) / n_tokens
    loss.backward()
    st = am.fwd_bwd(seqs)
    assert abs(st.loss - float(total.detach()) / active) < 2e-4          # the reported loss is the cross-entropy
    bm = am.buffers
    for l in range(2):
        for gname, pname in (("g_router", "w_router"), ("g_up", "w_up"), ("g_q", "w_q")):
            want = P[("layer", l, pname)].grad
            torch.testing.assert_close(bm.grads(l)[gname].float(), want, rtol=3e-4, atol=3e-6, msg=f"{l}/{pname}")
    # and the term matters: without it the router gradient differs
    P2 = clone_params(am)
    tot2 = 0.0
    for s in seqs:
        tot2 = tot2 + torch.nn.functional.cross_entropy(naive_forward(am, P2, s.tokens), s.targets, ignore_index=-100,
                                                        reduction="sum")
    (tot2 / active).backward()
    d = (P2[("layer", 0, "w_router")].grad - P[("layer", 0, "w_router")].grad).norm()
    assert float(d) > 1e-5


def test_moe_dump_and_diff(tmp_path, monkeypatch):
    """``FTB_MOE_DUMP_DIR`` diagnostics: every MoE forward is written out; two identical runs diff to zero, a run with
    a perturbed router shows which calls and tensors moved."""
    from flextrain_b200.ops import moe_dump

    def run(d, perturb):
        monkeypatch.setattr(moe_dump, "DUMP_DIR", str(d))
        monkeypatch.setattr(moe_dump, "_calls", 0)
        am = build_tiny(arch="qwen3_moe", dims=MOE, max_seq_len=48, batch_tokens=96)
        if perturb:
            am.buffers.params(1)["w_router"].add_(0.5)
        am.fwd_bwd(ft.SyntheticTokenSource(512, 48, seed=2).get_sequences(96))

    run(tmp_path / "a", False)
    run(tmp_path / "b", False)
    run(tmp_path / "c", True)
    monkeypatch.setattr(moe_dump, "DUMP_DIR", None)
    same = moe_dump.diff_dumps(str(tmp_path / "a"), str(tmp_path / "b"))
    assert len(same) == 2 * 2 * 4 and all(          # 2 layers x 2 chunks, 4 tensors each
        r.get("max_abs", 0.0) == 0.0 and r.get("rows_with_other_experts", 0.0) == 0.0 for r in same)
    moved = moe_dump.diff_dumps(str(tmp_path / "a"), str(tmp_path / "c"))
    first = [r for r in moved if r["call"] == "call000000.pt"]
    assert all(r.get("max_abs", 0.0) == 0.0 for r in first if "max_abs" in r)          # layer 0 is untouched
    logits = [r["max_abs"] for r in moved if r["tensor"] == "router_logits"]
    assert sum(v > 0.1 for v in logits) == 2 and sum(v == 0.0 for v in logits) == 2     # layer 1's router moved, both chunks


@pytest.mark.parametrize("arch", ["qwen3_moe", "olmoe"])
def test_moe_per_expert_lora_gradients(arch):
    """LoRA on the routed-expert stacks: one rank-r pair per expert (``w_up_lora_a (E, r, d)``, ``w_up_lora_b
    (E, 2F, r)``, likewise for ``w_down``).  The engine merges the adapters into the expert weights with one grouped
    GEMM and gets the rank-r gradients from the expert-major ``(x, dy)`` rows with grouped launches; autograd on the
    naive model (``W[e] + s B[e] A[e]`` per token) is the oracle.  Base weights, router included, stay frozen."""
    am = build_tiny(arch=arch, dims=MOE, max_seq_len=48, batch_tokens=96, lora_targets="all", lora_rank=4,
                    lora_alpha=8.0, lora_adapter_compute_dtype=torch.float32, lora_adapter_master_dtype=torch.float32,
                    lora_adapter_grad_dtype=torch.float32, lora_adapter_opt_state_dtype=torch.float32)
    torch.manual_seed(0)
    names = {n for _, _, n, _ in am.named_master_params()}
    assert {"w_up_lora_a", "w_up_lora_b", "w_down_lora_a", "w_down_lora_b", "w_q_lora_a"} <= names
    for scope, l, name, t in am.named_master_params():
        if name.endswith("_lora_b"):
            t.copy_(torch.randn_like(t) * 0.05)
    E, F, d = MOE["num_routed_experts"], MOE["expert_dim"], MOE["d_model"]
    assert am.buffers.params(0)["w_up_lora_a"].shape == (E, 4, d)
    assert am.buffers.params(0)["w_down_lora_b"].shape == (E, d, 4)
    seqs = ft.SyntheticTokenSource(512, 48, seed=3).get_sequences(96)
    P = clone_params(am)
    naive_loss(am, P, seqs).backward()
    am.fwd_bwd(seqs)
    for l in range(2):
        g = am.buffers.grads(l)
        assert "g_up" not in g and "g_down" not in g and "g_router" not in g, "base weights must be frozen under LoRA"
        for name in ("w_up", "w_down", "w_q", "w_o"):
            for ab in ("_lora_a", "_lora_b"):
                want = P[("layer", l, name + ab)].grad
                assert float(want.abs().max()) > 0
                torch.testing.assert_close(g["g_" + name[2:] + ab].float(), want, rtol=3e-4, atol=3e-6,
                                           msg=f"{l}/{name}{ab}")
    before = {n: t.clone() for _, l, n, t in am.named_master_params() if l == 0}
    assert am.step() == 0
    after = {n: t for _, l, n, t in am.named_master_params() if l == 0}
    assert not torch.equal(before["w_up_lora_a"], after["w_up_lora_a"])
    assert torch.equal(before["w_up"], after["w_up"])
    st = am.fwd_bwd(seqs)                       # the merged weights were rebuilt from the updated adapters
    assert st.loss == st.loss
