"""A family added from outside the package (``examples/extending_phi3.py``: fused ``qkv_proj`` / ``gate_up_proj``
checkpoint tensors, load by row slices, export through the spec's ``export_hook``) against ``transformers``' Phi-3."""
import os
import sys

import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.engine.host_memory import UnpinnedHostBackend
from flextrain_b200.export import save_hf_full

transformers = pytest.importorskip("transformers")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_phi3_example_matches_transformers(tmp_path):
    import examples.extending_phi3  # noqa: F401  (registers the family)
    cfg = transformers.Phi3Config(vocab_size=320, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                  num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                  original_max_position_embeddings=256, rms_norm_eps=1e-5, tie_word_embeddings=False,
                                  pad_token_id=None, sliding_window=None)
    cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    model = transformers.AutoModelForCausalLM.from_config(cfg).to(torch.float32)
    src = str(tmp_path / "phi3")
    model.save_pretrained(src, safe_serialization=True)
    f32 = torch.float32
    am = ft.from_pretrained(src, optimizer=ft.AdamW(lr=1e-3, state_dtype=f32), max_seq_len=64,
                            max_global_batch_tokens=128, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                            device="cpu", compute_dtype=f32, master_dtype=f32, grad_dtype=f32, strict=True,
                            host_backend=UnpinnedHostBackend(),
                            working_set=ft.WorkingSetConfig.simple(max_seq_len=64, max_global_batch_tokens=128))
    assert am.model_config.arch == "phi3"
    seqs = ft.SyntheticTokenSource(320, 64, seed=0).get_sequences(128)

    def hf_loss(m, grad=False):
        tot = 0.0
        for s in seqs:
            z = m(input_ids=s.tokens[None].long()).logits[0].float()
            tot = tot + torch.nn.functional.cross_entropy(z, s.targets.long(), ignore_index=-100, reduction="sum")
        if grad:
            tot.backward()
        return float(tot)

    want = hf_loss(model, grad=True)
    st = am.fwd_bwd(seqs, loss_scale_factor=1.0)
    assert abs(st.loss_sum - want) / want < 2e-4
    g = am.buffers.grads(1)
    fused = dict(model.named_parameters())["model.layers.1.self_attn.qkv_proj.weight"].grad
    got = torch.cat([g["g_q"], g["g_k"], g["g_v"]], 0)
    assert float((got - fused).norm() / fused.norm()) < 2e-3
    fused = dict(model.named_parameters())["model.layers.1.mlp.gate_up_proj.weight"].grad
    got = torch.cat([g["g_1"], g["g_3"]], 0)
    assert float((got - fused).norm() / fused.norm()) < 2e-3
    # export writes the fused tensors again and loads in transformers
    out = str(tmp_path / "export")
    save_hf_full(am, out)
    m2, info = transformers.AutoModelForCausalLM.from_pretrained(out, dtype=f32, attn_implementation="eager",
                                                                 output_loading_info=True)
    assert not info["missing_keys"] and not info["unexpected_keys"], info
    with torch.no_grad():
        assert abs(hf_loss(m2) - want) / want < 2e-4


def test_finetune_and_export_example_runs_on_cpu(tmp_path):
    """``examples/finetune_and_export.py``: LoRA steps on the toy model, then the adapter / merged / base exports."""
    import subprocess, sys, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    p = subprocess.run([sys.executable, os.path.join(root, "examples", "finetune_and_export.py"), "--dims", "tiny_llama",
                        "--steps", "2", "--out", str(tmp_path / "x")], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert "exports written" in p.stdout
    for sub, name in (("adapter", "adapter_model.safetensors"), ("merged", "config.json"), ("base_only", "config.json")):
        assert os.path.exists(tmp_path / "x" / sub / name), (sub, os.listdir(tmp_path / "x" / sub))
