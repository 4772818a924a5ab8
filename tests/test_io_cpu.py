"""HF safetensors load / export, LoRA adapter and merged exports, token sources (CPU)."""
import json
import os

import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.engine.host_memory import UnpinnedHostBackend
from flextrain_b200.export import merge_lora_into_base, save_hf_full, save_hf_merged, save_lora_adapter
from conftest import build_tiny

BASE = dict(vocab_size=512, n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, expert_dim=256, ffn_dim=256,
            num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
MOE = dict(BASE, expert_dim=64, num_routed_experts=8, top_k=2)
NEXT = dict(MOE, num_shared_experts=1, shared_dim=64)


def _reload(path, **kw):
    return ft.from_pretrained(path, optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32), max_seq_len=64,
                              max_global_batch_tokens=128, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                              device="cpu", compute_dtype=torch.float32, master_dtype=torch.float32,
                              grad_dtype=torch.float32, host_backend=UnpinnedHostBackend(), strict=True,
                              working_set=ft.WorkingSetConfig.simple(max_seq_len=64, max_global_batch_tokens=128), **kw)


@pytest.mark.parametrize("arch,dims,hyper", [
    ("llama", BASE, {}), ("qwen2", BASE, {}), ("qwen3", BASE, {}), ("qwen3_moe", MOE, {}), ("olmoe", MOE, {}),
    ("gemma2", BASE, {"sliding_window": 16, "layer_pattern": "SF"}), ("gemma3", BASE, {"sliding_window": 16, "layer_pattern": "SF"}),
    ("gemma4", BASE, {"sliding_window": 16, "layer_pattern": "SF"}),
    ("qwen3_5", BASE, {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 2, "head_k_dim": 16, "head_v_dim": 32}}),
    ("qwen3_5_moe", NEXT, {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 4, "head_k_dim": 16, "head_v_dim": 16}}),
    ("qwen3_next", NEXT, {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 4, "head_k_dim": 16, "head_v_dim": 16}}),
])
def test_export_reload_roundtrip(tmp_path, arch, dims, hyper):
    am = build_tiny(arch=arch, dims=dims, hyper=hyper, max_seq_len=64, batch_tokens=128)
    torch.manual_seed(1)
    for _, _, name, t in am.named_master_params():
        if "norm" in name or "scalar" in name:
            t.add_(torch.randn_like(t) * 0.1)
    out = str(tmp_path / arch)
    save_hf_full(am, out)
    cfg = json.load(open(os.path.join(out, "config.json")))
    assert cfg["architectures"] and cfg["num_hidden_layers"] == 2
    bm = _reload(out)
    a = {(s, l, n): t for s, l, n, t in am.named_master_params()}
    for s, l, n, t in bm.named_master_params():
        torch.testing.assert_close(t, a[(s, l, n)], rtol=0, atol=1e-6, msg=f"{s}/{l}/{n}")
    seqs = ft.SyntheticTokenSource(512, 64, seed=0).get_sequences(128)
    assert abs(am.fwd_bwd(seqs).loss - bm.fwd_bwd(seqs).loss) < 1e-5


def test_hf_names_and_norm_offset(tmp_path):
    from safetensors import safe_open
    am = build_tiny(arch="gemma2", dims=BASE, hyper={"layer_pattern": "SF", "sliding_window": 16}, max_seq_len=64,
                    batch_tokens=128)
    out = str(tmp_path / "g")
    save_hf_full(am, out)
    with safe_open(os.path.join(out, "model.safetensors"), framework="pt") as f:
        keys = set(f.keys())
        assert "model.layers.0.pre_feedforward_layernorm.weight" in keys and "model.layers.1.mlp.gate_proj.weight" in keys
        assert "lm_head.weight" not in keys                      # tied embeddings are not duplicated
        # Gemma stores gamma - 1: the engine's ones become zeros on disk
        assert float(f.get_tensor("model.layers.0.input_layernorm.weight").abs().max()) < 1e-6


def test_training_after_export_continues_lower(tmp_path):
    """Train N steps, export, reload, train on the same data: the resumed losses must be lower
    (flextrain tests/io/test_export_roundtrip_loss.py:1-36)."""
    am = build_tiny(dims=BASE, max_seq_len=64, batch_tokens=128, optimizer=ft.AdamW(lr=3e-3, state_dtype=torch.float32))
    data = [ft.SyntheticTokenSource(512, 64, seed=5).get_sequences(128) for _ in range(3)]
    first = []
    for seqs in data * 2:
        first.append(am.fwd_bwd(seqs).loss); am.step()
    out = str(tmp_path / "ck")
    save_hf_full(am, out)
    bm = _reload(out)
    resumed = [bm.fwd_bwd(seqs).loss for seqs in data]
    assert all(r < o for r, o in zip(resumed, first[:3])), (resumed, first)


def test_lora_adapter_and_merged_export(tmp_path):
    from safetensors import safe_open
    am = build_tiny(dims=BASE, max_seq_len=64, batch_tokens=128, lora_targets="all", lora_rank=4, lora_alpha=8.0,
                    lora_adapter_compute_dtype=torch.float32, lora_adapter_master_dtype=torch.float32,
                    lora_adapter_grad_dtype=torch.float32, lora_adapter_opt_state_dtype=torch.float32)
    for _, _, name, t in am.named_master_params():
        if name.endswith("_lora_b"):
            t.copy_(torch.randn_like(t) * 0.05)
    seqs = ft.SyntheticTokenSource(512, 64, seed=0).get_sequences(128)
    want = am.fwd_bwd(seqs).loss
    ad = str(tmp_path / "adapter")
    save_lora_adapter(am, ad)
    acfg = json.load(open(os.path.join(ad, "adapter_config.json")))
    assert acfg["r"] == 4 and "q_proj" in acfg["target_modules"]
    with safe_open(os.path.join(ad, "adapter_model.safetensors"), framework="pt") as f:
        assert f.get_tensor("base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight").shape == (4, 128)
    merged = str(tmp_path / "merged")
    save_hf_merged(am, merged)
    bm = _reload(merged)
    assert abs(bm.fwd_bwd(seqs).loss - want) < 1e-4
    merge_lora_into_base(am)
    assert abs(am.fwd_bwd(seqs).loss - want) < 1e-4


def test_synthetic_source_is_deterministic_and_push_back():
    a = ft.SyntheticTokenSource(100, [8, 16], seed=3)
    b = ft.SyntheticTokenSource(100, [8, 16], seed=3)
    sa, sb = a.get_sequences(40), b.get_sequences(40)
    assert [len(s) for s in sa] == [8, 16, 8] and all(torch.equal(x.tokens, y.tokens) for x, y in zip(sa, sb))
    assert torch.equal(sa[0].targets, torch.roll(sa[0].tokens, -1))
    a.push_back(sa[1:])
    again = a.get_sequences(24)
    assert [s.seq_id for s in again] == [1, 2]


def test_shard_source(tmp_path):
    import numpy as np
    p = tmp_path / "shard.bin"
    np.arange(1000, dtype=np.uint16).tofile(p)
    src = ft.ShardTokenSource(str(p), 64, loop=False)
    seqs = src.get_sequences(64 * 3)
    assert len(seqs) == 3 and int(seqs[1].tokens[0]) == 64 and int(seqs[1].targets[0]) == 65


class _Tok:
    eos_token_id = 2

    def encode(self, text, add_special_tokens=False):
        return [3 + (ord(c) % 50) for c in text]


def test_json_sft_masks_prompt(tmp_path):
    p = tmp_path / "d.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in [{"instruction": "add 1 1", "output": "2"},
                                                     {"prompt": "x" * 500, "completion": "y"}]))
    src = ft.JsonSFTTokenSource(str(p), _Tok(), max_seq_len=64, loop=False)
    seqs = list(src.iter_sequences())
    assert len(seqs) == 1 and src.dropped == 1                  # the long record is dropped
    s = seqs[0]
    n_prompt = len(_Tok().encode("Instruction:\nadd 1 1\n\nResponse:\n"))
    assert int((s.targets[: n_prompt - 1] != -100).sum()) == 0
    assert int(s.targets[n_prompt - 1]) == s.tokens[n_prompt] and int(s.targets[-1]) == -100
    assert s.active_token_count == 2                             # "2" and EOS
