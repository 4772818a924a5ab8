"""Comparison harness: spec merging / templating, command construction for every backend, step-throughput
extraction, and a dry-run sweep (no GPU, nothing is launched)."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from baseline.baseline_harness.backends import BACKENDS, format_command, get_backend  # noqa: E402
from baseline.baseline_harness.spec import RunSpec, load_sweep, spec_from_sections, substitute  # noqa: E402
from baseline.scripts.sweep import extract_step_throughput, main as sweep_main  # noqa: E402


def test_template_substitution_and_merge():
    assert substitute("${NUM_GPUS}", {"NUM_GPUS": 8}) == 8
    assert substitute("dp${NUM_GPUS}x", {"NUM_GPUS": 4}) == "dp4x"
    assert substitute({"a": ["${NUM_GPUS}", 2]}, {"NUM_GPUS": 2}) == {"a": [2, 2]}
    spec = spec_from_sections("flextrain_b200", {"seq_length": 2048, "num_steps": 3, "num_gpus": "${NUM_GPUS}"},
                              {"dp_shard": "opt+grad", "micro_batch_size": 4}, {"num_steps": 1}, num_gpus=8)
    assert (spec.seq_length, spec.num_steps, spec.num_gpus, spec.micro_batch_size) == (2048, 1, 8, 4)
    assert spec.extra == {"dp_shard": "opt+grad"} and spec.tokens_per_step == 2048 * 4 * 8
    with pytest.raises(ValueError):
        RunSpec(backend="x", num_steps=0).validate()


def test_every_backend_builds_a_command(tmp_path):
    for name, b in BACKENDS.items():
        spec = RunSpec(backend=name, model_path=str(tmp_path), num_gpus=2, seq_length=512, micro_batch_size=2,
                       gradient_accumulation_steps=4, extra={"zero_stage": 3, "dp_shard": "opt+grad"})
        cmd, env = b.command(spec)
        line = format_command(cmd, env)
        assert "torch.distributed.run" in line and "--nproc-per-node=2" in line and "127.0.0.1" in line, name
        assert ROOT in env["PYTHONPATH"]
    cmd, env = get_backend("nccl_library").command(RunSpec(backend="nccl_library"))
    assert env["FTB_DP_BACKEND"] == "collective" and env["FTB_GEMM_BACKEND"] == "library"
    assert cmd[1].endswith("train.py") and "dims:llama3_1_8B" in cmd
    with pytest.raises(KeyError):
        get_backend("nope")
    ok, why = get_backend("megatron").available()
    assert ok or "not installed" in why


def test_extract_step_throughput_formats():
    log = "\n".join([
        "[step    2] lr 3.000e-05 loss 11.7612 ema 11.80 tok/step 524288 tok/s 21,950 TFLOPS_eff 1005.1",
        "warmup 0: loss 12.1  900.0 ms  100.0 tok/s",
        "step 1: loss 11.9021  812.0 ms  20177.3 tok/s  max_alloc 71.2 GiB",
        '{"metric": "train tokens/sec/box", "value": 22050.5, "loss": 12.5}',
        "unrelated line",
    ])
    rows = extract_step_throughput(log)
    assert [r["step"] for r in rows] == [2, 1, -1]
    assert rows[0]["tok_s"] == 21950.0 and rows[1]["tok_s"] == 20177.3 and rows[2]["tok_s"] == 22050.5


def test_dry_run_sweep_of_the_shipped_configs(capsys):
    for cfg in ("llama3_8b_b200.toml", "llama3_128k_maxmem.toml"):
        path = os.path.join(ROOT, "baseline", "configs", cfg)
        data = load_sweep(path)
        assert "common" in data and len(data) >= 4
        common = dict(data["common"])
        if "model_path" in common:              # the model directory is not on this machine
            continue
        assert sweep_main([path, "--dry-run", "--num-gpus", "8", "--num-steps", "1"]) == 0
        out = capsys.readouterr().out
        assert "train.py" in out and "hf_fsdp2.py" in out and "--nproc-per-node=8" in out


def test_torchtitan_launcher_trains_a_tiny_model_on_cpu():
    """The TorchTitan backend's own script (its model, loss and activation checkpointing) runs end to end on CPU and
    prints step lines the sweep can parse; the preset's FFN width survives TorchTitan's multiplier arithmetic."""
    import subprocess
    pytest = __import__("pytest")
    pytest.importorskip("torchtitan")
    script = os.path.join(ROOT, "baseline", "backends", "torchtitan_synthetic.py")
    p = subprocess.run([sys.executable, script, "--preset", "tiny_llama", "--seq-length", "64", "--micro-batch-size", "2",
                        "--gradient-accumulation-steps", "2", "--num-steps", "2", "--device", "cpu", "--ac-mode", "full"],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-1500:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("step ")]
    assert len(lines) == 2 and all("tok/s" in l for l in lines), p.stdout
    sys.path.insert(0, os.path.join(ROOT, "baseline", "backends"))
    import importlib
    tt = importlib.import_module("torchtitan_synthetic")
    a = tt.model_args_from_preset("llama3_1_8B", 1024)
    hidden = a.multiple_of * ((int(a.ffn_dim_multiplier * int(2 * 4 * a.dim / 3)) + a.multiple_of - 1) // a.multiple_of)
    assert (a.dim, a.n_layers, a.n_heads, a.n_kv_heads, hidden) == (4096, 32, 32, 8, 14336)


def test_named_knob_flags_reach_the_backend_command(capsys):
    """The launcher's named knobs (the reference's flag spellings) and raw pass-through arguments end up on the
    backend's command line exactly like ``--set``."""
    from baseline.run_baseline import main as run_main
    rc = run_main(["--backend", "hf_fsdp2", "--dry-run", "--activation-checkpointing", "--attn-implementation", "eager",
                   "--seed", "7", "--backend-extra-arg=--n-layers", "--backend-extra-arg", "2"])
    out = capsys.readouterr().out
    assert rc == 0 and "--activation-checkpointing" in out and "--attn-implementation eager" in out
    assert "--seed 7" in out and out.strip().endswith("--n-layers 2")
    rc = run_main(["--backend", "torchtitan", "--dry-run", "--set", "ac_mode=selective", "--zero-stage", "3"])
    out = capsys.readouterr().out
    assert rc == 0 and "--ac-mode selective" in out and "zero" not in out      # a knob the backend does not know is dropped
