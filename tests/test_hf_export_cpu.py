"""The other direction of the HuggingFace parity check: a model built and exported by the engine (``save_hf_full``)
must load in ``transformers`` with no missing tensor and give the engine's loss on the same tokens.  This pins the
exported ``config.json`` and the export side of every family's name map to the upstream definition
(the reference's analogue: tests/io/test_export_roundtrip_loss.py, which reloads into the reference itself)."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.export import save_hf_full
from conftest import build_tiny
from test_arch_parity_cpu import CASES

transformers = pytest.importorskip("transformers")


@pytest.mark.parametrize("case", sorted(CASES))
def test_export_loads_in_transformers(case, tmp_path):
    arch, dims, hyper = CASES[case]
    am = build_tiny(arch=arch, dims=dims, hyper=hyper, max_seq_len=64, batch_tokens=128)
    torch.manual_seed(1)
    for _, _, name, t in am.named_master_params():
        if "norm" in name or "scalar" in name or name.startswith("b_"):
            t.add_(torch.randn_like(t) * 0.1)
    out = str(tmp_path / case)
    save_hf_full(am, out)
    model, info = transformers.AutoModelForCausalLM.from_pretrained(out, dtype=torch.float32,
                                                                    attn_implementation="eager",
                                                                    output_loading_info=True)
    assert not info["missing_keys"], info["missing_keys"]
    assert not info["unexpected_keys"], info["unexpected_keys"]
    seqs = ft.SyntheticTokenSource(dims["vocab_size"], 64, seed=0).get_sequences(128)
    st = am.fwd_bwd(seqs, loss_scale_factor=1.0)
    total = 0.0
    with torch.no_grad():
        for s in seqs:
            logits = model(input_ids=s.tokens[None].long()).logits[0].float()
            total += float(torch.nn.functional.cross_entropy(logits, s.targets.long(), ignore_index=-100,
                                                             reduction="sum"))
    assert abs(st.loss_sum - total) / total < 2e-4, (case, st.loss_sum, total)


@pytest.mark.parametrize("name", ["llama", "qwen3", "gemma3", "qwen3_5"])
def test_lora_exports_against_transformers(name, tmp_path):
    """LoRA fine-tune of an HF checkpoint: (1) at B = 0 the loss is the base model's (the reference's
    tests/test_lora_step0_equivalence.py); (2) the exported PEFT-format adapter, applied to the HF model by the PEFT
    rule ``W + (alpha / r) * B @ A``, gives the engine's loss; (3) the merged export loads in ``transformers`` and
    gives it too."""
    import json
    import os
    from safetensors import safe_open
    from flextrain_b200.engine.host_memory import UnpinnedHostBackend
    from flextrain_b200.export import save_hf_merged, save_lora_adapter
    from test_hf_parity_cpu import _hf_model
    model = _hf_model(name)
    src = str(tmp_path / "base")
    model.save_pretrained(src, safe_serialization=True)
    f32 = torch.float32
    build = lambda: ft.from_pretrained(
        src, optimizer=ft.AdamW(lr=1e-3, state_dtype=f32), max_seq_len=64, max_global_batch_tokens=128,
        max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30, device="cpu", compute_dtype=f32, master_dtype=f32,
        grad_dtype=f32, host_backend=UnpinnedHostBackend(), lora_targets="all", lora_rank=4, lora_alpha=8.0,
        lora_adapter_compute_dtype=f32, lora_adapter_master_dtype=f32, lora_adapter_grad_dtype=f32,
        lora_adapter_opt_state_dtype=f32,
        working_set=ft.WorkingSetConfig.simple(max_seq_len=64, max_global_batch_tokens=128))
    V = model.config.vocab_size
    seqs = ft.SyntheticTokenSource(V, 64, seed=0).get_sequences(128)

    def hf_loss(m):
        tot = 0.0
        with torch.no_grad():
            for s in seqs:
                z = m(input_ids=s.tokens[None].long()).logits[0].float()
                tot += float(torch.nn.functional.cross_entropy(z, s.targets.long(), ignore_index=-100, reduction="sum"))
        return tot

    base = hf_loss(model)
    assert abs(build().fwd_bwd(seqs, loss_scale_factor=1.0).loss_sum - base) / base < 2e-4     # (1) step 0
    am = build()                       # a fresh engine: effective weights are cached between optimizer steps
    torch.manual_seed(3)
    for _, _, n, t in am.named_master_params():
        if n.endswith("_lora_b"):
            t.copy_(torch.randn_like(t) * 0.5)
    want = am.fwd_bwd(seqs, loss_scale_factor=1.0).loss_sum
    assert abs(want - base) / base > 1e-3                                                      # the adapters matter
    ad = str(tmp_path / "adapter")
    save_lora_adapter(am, ad)
    acfg = json.load(open(os.path.join(ad, "adapter_config.json")))
    scale = acfg["lora_alpha"] / acfg["r"]
    sd = dict(model.named_parameters())
    applied = 0
    with safe_open(os.path.join(ad, "adapter_model.safetensors"), framework="pt") as f, torch.no_grad():
        for k in f.keys():
            if k.endswith("lora_A.weight"):
                mod = k[len("base_model.model."): -len(".lora_A.weight")]
                a, b = f.get_tensor(k), f.get_tensor(k.replace("lora_A", "lora_B"))
                sd[mod + ".weight"].add_(scale * (b @ a))
                applied += 1
    assert applied >= 7
    assert abs(hf_loss(model) - want) / want < 2e-4                                            # (2) adapter
    merged = str(tmp_path / "merged")
    save_hf_merged(am, merged)
    m2, info = transformers.AutoModelForCausalLM.from_pretrained(merged, dtype=f32, attn_implementation="eager",
                                                                 output_loading_info=True)
    assert not info["missing_keys"] and not info["unexpected_keys"]
    assert abs(hf_loss(m2) - want) / want < 2e-4                                               # (3) merged


def test_moe_lora_adapter_export_carries_the_expert_adapters(tmp_path):
    """Per-expert adapters leave as one PEFT module per expert (gate / up share the expert's A and split B); base weight
    + scale * B @ A equals the merged export for every expert projection."""
    import json
    import os
    import flextrain_b200 as ft
    from safetensors import safe_open
    from flextrain_b200.export import save_hf_full, save_hf_merged, save_lora_adapter
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cat = json.load(open(os.path.join(root, "flextrain_b200", "configs", "model_dims.json")))
    d = dict(cat["tiny_moe"]); arch = d.pop("arch"); hyper = d.pop("hyperparams", None)
    f32 = torch.float32
    am = ft.from_dims(d, arch=arch, hyperparams=hyper, optimizer=ft.AdamW(lr=1e-2, state_dtype=f32), max_seq_len=64,
                      max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30, device="cpu",
                      compute_dtype=f32, master_dtype=f32, grad_dtype=f32, lora_targets="all", lora_rank=4, lora_alpha=8.0)
    src = ft.SyntheticTokenSource(d["vocab_size"], 64, seed=0, pin=False)
    for _ in range(2):
        am.fwd_bwd(src.get_sequences(256)); am.step()
    save_lora_adapter(am, str(tmp_path / "a")); save_hf_full(am, str(tmp_path / "b")); save_hf_merged(am, str(tmp_path / "m"))

    def load(p):
        with safe_open(p, "pt") as f:
            return {k: f.get_tensor(k) for k in f.keys()}

    ad, base, merged = (load(str(tmp_path / n / fn)) for n, fn in (("a", "adapter_model.safetensors"),
                                                                  ("b", "model.safetensors"), ("m", "model.safetensors")))
    cfg = json.load(open(tmp_path / "a" / "adapter_config.json"))
    assert {"gate_proj", "up_proj", "down_proj", "q_proj"} <= set(cfg["target_modules"])
    scale = cfg["lora_alpha"] / cfg["r"]
    checked = 0
    for k in ad:
        if ".experts." in k and k.endswith(".lora_A.weight"):
            mod = k[len("base_model.model."):-len(".lora_A.weight")]
            delta = scale * ad[k.replace("lora_A", "lora_B")] @ ad[k]
            assert float(delta.abs().max()) > 0                      # the adapters did train
            assert torch.allclose(base[mod + ".weight"].float() + delta, merged[mod + ".weight"].float(), atol=1e-6)
            checked += 1
    assert checked == d["n_layers"] * d["num_routed_experts"] * 3
