"""Full training-state checkpoints (weights + optimizer state + step): a run that is stopped, restored in a new engine
and continued reproduces the uninterrupted run exactly — single process with resident state, with host rings, with
Muon, and two tensor-parallel / expert-parallel ranks (gloo, per-rank state files) through ``train.py``."""
import os
import re
import subprocess
import sys

import pytest
import torch

import flextrain_b200 as ft
from conftest import build_tiny

def _free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DIMS = dict(vocab_size=256, n_layers=3, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, expert_dim=128, ffn_dim=128,
            num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)


def _run(am, src, steps):
    out = []
    for _ in range(steps):
        st = am.fwd_bwd(src.get_sequences(128))
        assert am.step() == 0
        out.append(st.loss)
    return out


@pytest.mark.parametrize("variant", ["resident", "rings", "muon", "lora", "moe_lora"])
def test_resume_is_exact(variant, tmp_path):
    kw = dict(dims=DIMS, max_seq_len=64, batch_tokens=128)
    if variant == "rings":
        kw["ws"] = ft.WorkingSetConfig.simple(max_seq_len=64, max_global_batch_tokens=128, n_gpu_layers=2, n_gpu_grads=2,
                                              n_gpu_opt_layers=2)
    if variant == "muon":
        kw["optimizer"] = ft.HybridMuonAdamW(muon=ft.Muon(lr=2e-3, state_dtype=torch.float32),
                                             adamw=ft.AdamW(lr=2e-3, state_dtype=torch.float32))
    else:
        kw["optimizer"] = ft.AdamW(lr=2e-3, weight_decay=0.1, state_dtype=torch.float32)
    if variant == "moe_lora":            # per-expert adapters on the routed expert stacks
        kw["dims"] = dict(DIMS, expert_dim=64, ffn_dim=64, num_routed_experts=4, top_k=2)
        kw["arch"] = "qwen3_moe"
    if variant in ("lora", "moe_lora"):
        f32 = torch.float32
        kw.update(lora_targets="all", lora_rank=4, lora_alpha=8.0, lora_adapter_compute_dtype=f32,
                  lora_adapter_master_dtype=f32, lora_adapter_grad_dtype=f32, lora_adapter_opt_state_dtype=f32)
    straight = _run(build_tiny(**kw), ft.SyntheticTokenSource(256, 64, seed=1), 5)
    a = build_tiny(**kw)
    src = ft.SyntheticTokenSource(256, 64, seed=1)
    first = _run(a, src, 3)
    a.save_training_state(str(tmp_path / "ck"), extra={"note": "hello"})
    b = build_tiny(**kw)
    for _, _, _, t in b.named_master_params():                 # make sure nothing survives from the fresh init
        t.add_(1.0)
    info = b.load_training_state(str(tmp_path / "ck"))
    assert info["step"] == 3 and info["note"] == "hello" and b.step_num == 3
    rest = _run(b, src, 2)
    assert first + rest == straight, (first + rest, straight)


def test_mismatched_model_is_refused(tmp_path):
    a = build_tiny(dims=DIMS, max_seq_len=64, batch_tokens=128)
    a.save_training_state(str(tmp_path / "ck"))
    other = build_tiny(dims=dict(DIMS, n_layers=2), max_seq_len=64, batch_tokens=128)
    with pytest.raises(ValueError, match="does not match"):
        other.load_training_state(str(tmp_path / "ck"))


def _losses(out):
    return [float(m) for m in re.findall(r"\[step\s+\d+\].*? loss ([\d.]+)", out)]


@pytest.mark.parametrize("launch", ["single", "tp2", "ep2"])
def test_train_py_resume(launch, tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    base = [sys.executable] if launch == "single" else \
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", str(_free_port())]
    common = [os.path.join(ROOT, "train.py"), "--model", "dims:tiny_moe" if launch == "ep2" else "dims:tiny_llama",
              "--mode", "full", "--data-source",
              "synthetic", "--max-seq-len", "128", "--max-global-batch-tokens", "512", "--lr", "1e-3", "--steps", "5"] + \
        {"tp2": ["--tp", "2"], "ep2": ["--ep", "2"]}.get(launch, [])
    run = lambda extra: subprocess.run(base + common + extra, capture_output=True, text=True, env=env, timeout=900,
                                       cwd=str(tmp_path))
    full = run(["--output-dir", str(tmp_path / "full")])
    assert full.returncode == 0, full.stderr[-3000:]
    # same 5-step schedule, stopped after step 3 with the state written there
    three = run(["--output-dir", str(tmp_path / "three"), "--save-state-every", "3", "--stop-after", "3"])
    assert three.returncode == 0, three.stderr[-3000:]
    assert os.path.exists(os.path.join(str(tmp_path / "three" / "state"), "training_state.json"))
    resumed = run(["--output-dir", str(tmp_path / "resumed"), "--resume-state", str(tmp_path / "three" / "state")])
    assert resumed.returncode == 0, resumed.stderr[-3000:]
    a, b, c = _losses(full.stdout), _losses(three.stdout), _losses(resumed.stdout)
    assert len(a) == 5 and len(b) == 3 and len(c) == 2
    assert b + c == a, (a, b, c)
