"""Command-line entry points on CPU with tiny models: ``python -m flextrain_b200 {info, init, pretrain}`` with the
reference's flag spellings (flextrain/scripts/pretrain.py:518-571, flextrain/scripts/init_hf.py) and this
package's shorter aliases."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from flextrain_b200.scripts.pretrain import lr_at, parse_count, resolve_shards

def _free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*argv, timeout=600):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-m", "flextrain_b200", *argv], capture_output=True, text=True, env=env,
                       timeout=timeout, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return r.stdout


def _write_shards(d, vocab=200):
    rng = np.random.default_rng(0)
    os.makedirs(d, exist_ok=True)
    for kind, idx in (("train", 1), ("train", 2), ("val", 0)):
        toks = rng.integers(0, vocab, size=6000, dtype=np.uint16)
        head = np.zeros(256, dtype=np.int32)
        head[0], head[1], head[2] = 20240520, 1, toks.size
        with open(os.path.join(d, f"fineweb_{kind}_{idx:06d}.bin"), "wb") as f:
            f.write(head.tobytes())
            f.write(toks.tobytes())


def test_helpers(tmp_path):
    assert parse_count("1B") == 10 ** 9 and parse_count("250M") == 250_000_000 and parse_count("16384") == 16384
    assert parse_count("2.5e3") == 2500 and parse_count("3k") == 3000
    assert lr_at(1, 100, 1.0, 0.1) == pytest.approx(0.1) and lr_at(10, 100, 1.0, 0.1) == pytest.approx(1.0)
    assert lr_at(100, 100, 1.0, 0.1) == pytest.approx(0.1)
    d = str(tmp_path / "data")
    _write_shards(d)
    assert [os.path.basename(p) for p in resolve_shards(d, "1-99", "train")] == ["fineweb_train_000001.bin",
                                                                                  "fineweb_train_000002.bin"]
    assert len(resolve_shards(d, "0", "val")) == 1
    assert len(resolve_shards(None, os.path.join(d, "fineweb_train_*.bin"), "train")) == 2
    with pytest.raises(FileNotFoundError):
        resolve_shards(d, "7-9", "train")


def test_info_lists_architectures():
    out = _run("info")
    assert "architectures:" in out and "gemma4" in out and "qwen3_5_moe" in out


def test_check_reports_tool_chain_libraries_and_no_gpu():
    """``python -m flextrain_b200 check --json``: every native library is built, loads and exports its entry point;
    without a GPU nothing is a problem (the report says so instead)."""
    rep = json.loads(_run("check", "--json").strip().splitlines()[-1])
    assert rep["problems"] == [] and rep["toolchain"]["sm_100a"] and rep["toolchain"]["nvcc"]
    libs = rep["libraries"]
    assert set(libs) >= {"gemm_tcgen05", "attention", "comm", "moe", "elementwise", "gdn", "seqmix", "noalloc",
                         "dp_solver", "copy_engine", "fastcall"}
    assert all(r["ok"] for r in libs.values())
    assert rep["gpus"]["available"] is False and rep["gpus"]["devices"] == [] and rep["gpus"]["host_memory_gib"] > 0
    # a missing entry point or a GPU of another generation is named
    from flextrain_b200.scripts.post_install import problems
    rep["libraries"]["attention"] = {"ok": False, "error": "entry point ftb_attn_fwd is missing"}
    rep["gpus"]["devices"] = [{"index": 0, "cc": "9.0", "supported": False}]
    rep["gpus"]["peer_access"] = False
    bad = problems(rep)
    assert len(bad) == 3 and "attention" in bad[0] and "9.0" in bad[1] and "peer access" in bad[2]


def test_pretrain_with_reference_flags_then_skip(tmp_path):
    d, out = str(tmp_path / "data"), str(tmp_path / "run")
    _write_shards(d)
    argv = ["pretrain", "--arch", "llama", "--d-model", "64", "--n-layers", "2", "--vocab-size", "200", "--head-dim", "16",
            "--n-kv-heads", "2", "--total-tokens", "2K", "--batch-tokens", "256", "--max-seq-len", "64",
            "--data-dir", d, "--train-shards", "1-99", "--val-shard", "0", "--out", out, "--peak-lr", "3e-3",
            "--warmup-frac", "0.25", "--weight-decay", "0.0", "--init-seed", "7", "--eval-every", "4",
            "--eval-tokens", "256", "--log-every", "2", "--max-gpu-gib", "4", "--max-host-gib", "4"]
    _run(*argv)
    meta = json.load(open(os.path.join(out, "meta.json")))
    assert meta["total_steps"] == 8 and meta["dims"]["n_heads"] == 4 and meta["dims"]["expert_dim"] == 176
    train = [json.loads(l) for l in open(os.path.join(out, "train.jsonl"))]
    assert [r["step"] for r in train] == [1, 2, 4, 6, 8] and all(r["tok_per_s"] > 0 for r in train)
    assert train[0]["lr"] == pytest.approx(3e-3 / 2)
    ev = [json.loads(l) for l in open(os.path.join(out, "eval.jsonl"))]
    assert [r["step"] for r in ev] == [4, 8] and ev[0]["val_ppl"] == pytest.approx(np.exp(ev[0]["val_loss"]), rel=1e-6)
    fin = json.load(open(os.path.join(out, "final.json")))
    assert fin["steps"] == 8 and fin["tokens"] == 8 * 256 and fin["val_loss"] is not None
    assert "nothing to do" in _run(*argv)                       # final.json exists: the run is skipped


def test_pretrain_flop_budget_and_named_dims(tmp_path):
    d, out = str(tmp_path / "data"), str(tmp_path / "run")
    _write_shards(d)
    dims = {"tiny": {"arch": "qwen3", "vocab_size": 200, "n_layers": 2, "d_model": 64, "n_heads": 4, "n_kv_heads": 2,
                     "head_dim": 16, "expert_dim": 128, "ffn_dim": 128, "num_routed_experts": 0, "top_k": 0,
                     "num_shared_experts": 0, "is_causal": True}}
    dj = str(tmp_path / "dims.json")
    json.dump(dims, open(dj, "w"))
    _run("pretrain", "--dims-json", dj, "--model-name", "tiny", "--total-flops", "6e8", "--batch-tokens", "256",
         "--max-seq-len", "64", "--train-shards", os.path.join(d, "fineweb_train_*.bin"), "--out", out,
         "--log-every", "1", "--use-muon")
    meta = json.load(open(os.path.join(out, "meta.json")))
    assert meta["arch"] == "qwen3" and meta["optimizer"] == "muon+adamw"
    assert meta["total_tokens"] == int(np.ceil(6e8 / (6.0 * meta["n_params"])))
    fin = json.load(open(os.path.join(out, "final.json")))
    assert fin["val_loss"] is None and fin["steps"] == meta["total_steps"]


def test_init_writes_a_loadable_hf_directory(tmp_path):
    out = str(tmp_path / "m")
    _run("init", "--arch", "gemma3", "--d-model", "64", "--n-layers", "2", "--vocab-size", "200", "--head-dim", "16",
         "--layer-pattern", "SF", "--out", out, "--dtype", "float32")
    cfg = json.load(open(os.path.join(out, "config.json")))
    assert cfg["model_type"] == "gemma3_text" and cfg["num_hidden_layers"] == 2
    assert cfg["layer_types"] == ["sliding_attention", "full_attention"]
    assert os.path.exists(os.path.join(out, "model.safetensors"))


def test_download_cli_stages_local_dataset_and_keeps_complete_models(tmp_path):
    """``download.py`` runs without importing the package; a local dataset is normalised to JSONL, and a model target
    that is already complete is left alone (no network is touched)."""
    src = tmp_path / "raw.json"
    json.dump([{"prompt": "2+2?", "completion": "4"}, {"messages": [{"role": "user", "content": "hi"},
                                                                   {"role": "assistant", "content": "hello"}]},
               {"unrelated": 1}], open(src, "w"))
    tgt = tmp_path / "out" / "sft.jsonl"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "download.py"), "dataset", str(src), "--target", str(tgt)],
                       capture_output=True, text=True, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [json.loads(l) for l in open(tgt)]
    assert rows[0] == {"instruction": "2+2?", "response": "4"} and len(rows) == 2
    model = tmp_path / "m"
    model.mkdir()
    json.dump({}, open(model / "config.json", "w"))
    (model / "model.safetensors").write_bytes(b"")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "download.py"), "model", "org/name", "--target", str(model)],
                       capture_output=True, text=True, cwd=str(tmp_path))
    assert r.returncode == 0 and r.stdout.strip() == str(model), r.stderr[-2000:]


def _steps(out):
    import re
    return [float(m) for m in re.findall(r"\[step\s+\d+\].*? loss ([\d.]+)", out)]


def test_train_tensor_parallel_matches_single_rank_and_saves(tmp_path):
    """``train.py --tp 2`` (two gloo ranks on CPU): the ranks of a tensor-parallel group read the same batch, the
    reported loss is the whole batch's, and ``--save`` (a collective gather of the parts) completes and writes one
    file that holds the unsharded tensors."""
    from safetensors import safe_open
    common = ["--model", "dims:tiny_llama", "--mode", "full", "--data-source", "synthetic", "--max-seq-len", "128",
              "--max-global-batch-tokens", "512", "--steps", "3", "--lr", "1e-3", "--eval-every", "2",
              "--eval-tokens", "1024", "--max-grad-norm", "0.5"]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    one = subprocess.run([sys.executable, os.path.join(ROOT, "train.py"), *common, "--output-dir", str(tmp_path / "a")],
                         capture_output=True, text=True, env=env, timeout=600, cwd=str(tmp_path))
    assert one.returncode == 0, one.stderr[-3000:]
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "train.py"),
                          *common, "--tp", "2", "--save", "--output-dir", str(tmp_path / "b")],
                         capture_output=True, text=True, env=env, timeout=600, cwd=str(tmp_path))
    assert two.returncode == 0, two.stderr[-3000:]
    a, b = _steps(one.stdout), _steps(two.stdout)
    assert len(a) == 3 and len(b) == 3 and max(abs(x - y) for x, y in zip(a, b)) < 2e-4, (a, b)
    import re
    ev = lambda out: [(int(s), float(l), int(n)) for s, l, n in re.findall(r"\[eval\s+(\d+)\] loss ([\d.]+) over (\d+)", out)]
    assert [e[0] for e in ev(one.stdout)] == [2, 3] and all(e[2] == 1024 for e in ev(one.stdout))     # validation, forward only
    assert max(abs(x[1] - y[1]) for x, y in zip(ev(one.stdout), ev(two.stdout))) < 2e-4
    gn = lambda out: [float(v) for v in re.findall(r"gnorm ([\d.]+)", out)]
    assert len(gn(one.stdout)) == 3 and min(gn(one.stdout)) > 0.5                      # clipped every step
    assert max(abs(x - y) for x, y in zip(gn(one.stdout), gn(two.stdout))) < 2e-4      # parts summed over the group
    with safe_open(str(tmp_path / "b" / "final.safetensors"), framework="pt") as f:
        assert f.get_tensor("model.layers.0.mlp.gate_proj.weight").shape == (688, 256)      # gathered, not a shard
        assert f.get_tensor("model.layers.1.self_attn.o_proj.weight").shape == (256, 256)


def test_rank_strided_source_partitions_the_stream():
    import flextrain_b200 as ft
    base = lambda: ft.SyntheticTokenSource(100, 16, seed=3)
    whole = [s.tokens.tolist() for s in base().get_sequences(16 * 8)]
    parts = [[s.tokens.tolist() for s in ft.RankStridedSource(base(), r, 2).get_sequences(16 * 4)] for r in range(2)]
    assert parts[0] == whole[0::2] and parts[1] == whole[1::2]
    src = ft.RankStridedSource(base(), 1, 2)
    first = src.get_sequences(32)
    src.push_back(first)
    assert [s.tokens.tolist() for s in src.get_sequences(32)] == [s.tokens.tolist() for s in first]


def _tiny_hf_dir_with_tokenizer(path):
    """A two-layer random Llama in HF layout with a character-level tokenizer (digits, operators, letters)."""
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, models, pre_tokenizers
    chars = ["<unk>", "</s>", "<pad>"] + [chr(c) for c in range(32, 127)] + ["\n"]
    tok = Tokenizer(models.WordLevel({c: i for i, c in enumerate(chars)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split("", behavior="isolated")
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="</s>",
                                                pad_token="<pad>")
    _run("init", "--arch", "llama", "--d-model", "64", "--n-layers", "2", "--vocab-size", str(len(chars)), "--head-dim",
         "16", "--n-kv-heads", "2", "--out", path, "--dtype", "float32")
    fast.save_pretrained(path)
    return len(chars)


def test_train_lora_sft_on_an_hf_directory_learns_and_saves(tmp_path):
    """``train.py --mode lora`` on an HF directory with its tokenizer and the bundled toy arithmetic set: the prompt is
    masked, the loss falls, ``--save`` writes the weights, and ``--truncate-long`` / chat-template flags parse."""
    model = str(tmp_path / "model")
    _tiny_hf_dir_with_tokenizer(model)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    out = str(tmp_path / "run")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "train.py"), "--model", model, "--mode", "lora",
                        "--lora-rank", "8", "--lora-alpha", "16", "--max-seq-len", "96", "--max-global-batch-tokens",
                        "768", "--steps", "12", "--lr", "2e-2", "--truncate-long", "--save", "--output-dir", out],
                       capture_output=True, text=True, env=env, timeout=900, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-3000:]
    losses = _steps(r.stdout)
    assert len(losses) == 12 and losses[-1] < losses[0] - 0.3, losses
    assert os.path.exists(os.path.join(out, "final.safetensors"))
    # LoRA mode also leaves what was trained: a PEFT adapter whose B matrices moved away from their zero start
    from safetensors.torch import load_file
    cfg = json.load(open(os.path.join(out, "adapter", "adapter_config.json")))
    assert cfg["r"] == 8 and cfg["lora_alpha"] == 16
    ad = load_file(os.path.join(out, "adapter", "adapter_model.safetensors"))
    assert any(k.endswith("lora_B.weight") and float(v.abs().max()) > 0 for k, v in ad.items())


def test_train_from_yaml_with_state_checkpoint(tmp_path):
    """``python -m flextrain_b200 train <yaml>``: the YAML front end drives the same loop as ``train.py``; the run
    writes a training state that a second YAML resumes."""
    y1, y2 = tmp_path / "a.yaml", tmp_path / "b.yaml"
    body = ("model: {dims: tiny_llama, mode: full}\noptimizer: {name: adamw, lr: 1.0e-3, state_dtype: float32}\n"
            "train: {steps: 4, max_seq_len: 128, max_global_batch_tokens: 512}\ndata: {source: synthetic}\n")
    y1.write_text(body + f"io: {{output_dir: {tmp_path}/r1, save_state_every: 2}}\n")
    out = _run("train", str(y1))
    assert len(_steps(out)) == 4 and out.count("[state]") == 2
    rows = [json.loads(l) for l in open(tmp_path / "r1" / "metrics.jsonl")]
    assert [r["step"] for r in rows] == [1, 2, 3, 4] and rows[0]["tokens"] == 512 and rows[0]["tok_per_s"] > 0
    assert abs(rows[2]["loss"] - _steps(out)[2]) < 1e-3 and rows[0]["chunks"] >= 1 and rows[0]["optimizer_rc"] == 0
    y2.write_text(body.replace("steps: 4", "steps: 6") + f"io: {{output_dir: {tmp_path}/r2, resume_state: {tmp_path}/r1/state}}\n")
    out2 = _run("train", str(y2))
    assert "continuing at step 5" in out2 and len(_steps(out2)) == 2


def test_train_auto_layout_on_two_ranks_stays_data_parallel(tmp_path):
    """``--tp auto`` on two CPU ranks: a model that fits is kept data parallel (each rank reads its own half of the
    batch), and the losses match the single-rank run of the same global batch."""
    common = ["--model", "dims:tiny_llama", "--mode", "full", "--data-source", "synthetic", "--max-seq-len", "128",
              "--max-global-batch-tokens", "512", "--steps", "2", "--lr", "1e-3"]
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    two = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "train.py"),
                          *common, "--tp", "auto", "--ep", "auto", "--verbose", "--output-dir", str(tmp_path / "b")],
                         capture_output=True, text=True, env=env, timeout=600, cwd=str(tmp_path))
    assert two.returncode == 0, two.stderr[-3000:]
    assert "layout tp=1 ep=1" in two.stdout, two.stdout[-2000:]          # (this model's FFN width does not split in two)
    assert len(_steps(two.stdout)) == 2
