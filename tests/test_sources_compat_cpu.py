"""Token sources with the reference's constructor spellings and behaviours (flextrain/io/sources.py): a script written
against the reference's sources keeps working after the import changes.  Also the reference's run-file layout
(flextrain/config.py) through ``python -m flextrain_b200 train``."""
import json
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.config import RunConfig, is_reference_schema

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _CharTok:
    eos_token_id = 1

    def encode(self, s, add_special_tokens=False):
        return [ord(c) % 200 + 2 for c in s]


def test_raw_source_takes_lists_dicts_and_a_dict_of_lists():
    a, b = torch.arange(5), torch.arange(7)
    tg = torch.full((5,), -100)
    for payload in ([a, b], [{"tokens": a, "targets": tg}, {"tokens": b}],
                    {"tokens": [a, b], "targets": [tg, None]}):
        src = ft.RawTokenSource(payload)
        got = src.get_sequences(100)
        assert [len(s) for s in got] == [5, 7] and src.get_sequences(100) == []
        if not isinstance(payload, list) or isinstance(payload[0], dict):
            assert torch.equal(got[0].targets, tg) and got[0].active_token_count == 0
        assert torch.equal(got[1].targets, torch.roll(b, -1))
        src.reset()
        assert len(src.get_sequences(5)) == 1
    m = torch.tensor([0, 1, 1, 0, 1])
    s = ft.RawTokenSource({"tokens": [a], "loss_mask": [m]}).get_sequences(10)[0]
    assert s.active_token_count == 3


def test_shard_source_document_mode_and_numbered_pattern(tmp_path):
    EOT = 50256
    docs = [list(range(10, 50)), list(range(100, 104)), list(range(200, 300)), list(range(7, 47))]
    for i, chunk in enumerate((docs[:2], docs[2:]), start=1):
        toks = []
        for d in chunk:
            toks += [EOT] + d                       # every document opens with the delimiter, as in the FineWeb files
        head = np.zeros(256, dtype=np.int32)
        head[0], head[1], head[2] = 20240520, 1, len(toks)
        with open(tmp_path / f"fw_train_{i:06d}.bin", "wb") as f:
            f.write(head.tobytes())
            f.write(np.asarray(toks, dtype=np.uint16).tobytes())
    pat = str(tmp_path / "fw_train_{shard_index:06d}.bin")
    src = ft.ShardTokenSource(shard_pattern=pat, num_shards=2, min_seq_len=8, max_seq_len=64, vocab_size=256, loop=False)
    got = list(src.iter_sequences())
    # the 4-token document is skipped, the 100-token one is cut to 64, ids above the vocabulary are clipped
    assert [len(s) for s in got] == [40, 64, 40]
    assert got[0].tokens.tolist() == docs[0] and got[1].tokens.tolist() == [min(t, 255) for t in docs[2][:64]]
    assert torch.equal(got[0].targets, torch.roll(got[0].tokens, -1))
    src.reset()
    assert len(list(src.iter_sequences())) == 3
    only_first = ft.ShardTokenSource(str(tmp_path / "fw_train_*.bin"), num_shards=1, max_seq_len=64, min_seq_len=1, loop=False)
    assert [len(s) for s in only_first.iter_sequences()] == [40, 4]
    with pytest.raises(ValueError):
        ft.ShardTokenSource(pat, max_seq_len=64)                     # a numbered pattern needs num_shards
    with pytest.raises(ValueError):
        ft.ShardTokenSource(str(tmp_path / "fw_train_*.bin"))        # neither windows nor documents asked for


def test_json_sft_field_names_and_length_floor(tmp_path):
    rows = [{"question_text": "2+2?", "context": "arithmetic", "final": "4"},
            {"question_text": "a", "final": "b"},
            {"instruction": "usual schema", "output": "still read"}]
    p = tmp_path / "rows.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in rows))
    src = ft.JsonSFTTokenSource(str(p), tokenizer=_CharTok(), prompt_field="question_text", response_field="final",
                                input_field="context", min_seq_len=30, max_seq_len=256, loop=False)
    got = list(src.iter_sequences())
    assert len(got) == 2 and src.dropped == 1                         # the two-character record is under the floor
    text = "".join(chr((t - 2) % 200) for t in got[0].tokens.tolist()[:-1])
    assert "2+2?\narithmetic" in text and text.endswith("4")
    assert int((got[0].targets != -100).sum()) == 2                   # the answer and the end-of-text token


def test_custom_schema_source_extract_contract():
    recs = [{"ids": [1, 2, 3]}, {"skip": True}, {"ids": [4, 5]}]
    extract = lambda r: None if r.get("skip") else ft.Sequence(torch.tensor(r["ids"]))
    src = ft.CustomSchemaTokenSource(records=recs, extract=extract)
    got = list(src.iter_sequences())
    assert [s.tokens.tolist() for s in got] == [[1, 2, 3], [4, 5]] and src.skipped == 1
    src.reset()
    assert len(src.get_sequences(3)) == 1
    looped = ft.CustomSchemaTokenSource(recs, extract, loop=True)
    assert [len(s) for s in looped.get_sequences(12)] == [3, 2, 3, 2]
    # an iterator is consumed lazily, once
    seen = []
    def gen():
        for r in recs:
            seen.append(1)
            yield r
    lazy = ft.CustomSchemaTokenSource(gen(), extract)
    assert len(lazy.get_sequences(3)) == 1 and len(seen) <= 3
    # text pairs with a tokenizer
    pairs = ft.CustomSchemaTokenSource([{"q": "hi", "a": "yo"}], lambda r: (r["q"], r["a"]), tokenizer=_CharTok(),
                                       max_seq_len=64)
    s = pairs.get_sequences(64)[0]
    assert int((s.targets != -100).sum()) == 3
    with pytest.raises(TypeError):
        list(ft.CustomSchemaTokenSource([{"q": 1}], lambda r: ("a", "b")).iter_sequences())


def test_hf_source_documents_and_windows_from_a_local_json_dataset(tmp_path):
    pytest.importorskip("datasets")
    rows = [{"body": "x" * 50}, {"body": "short"}, {"body": ""}, {"body": "y" * 300}]
    p = tmp_path / "docs.jsonl"
    p.write_text("\n".join(json.dumps(r) for r in rows))
    src = ft.HFTokenSource("json", tokenizer=_CharTok(), text_field="body", min_seq_len=10, max_seq_len=128,
                           streaming=False, data_files=str(p))
    got = list(src.iter_sequences())
    assert [len(s) for s in got] == [50, 128]                          # short and empty skipped, long one cut
    win = ft.HFTokenSource("json", _CharTok(), 64, text_column="body", streaming=True, data_files=str(p))
    w = list(win.iter_sequences())
    assert all(len(s) == 64 for s in w) and len(w) == (50 + 5 + 0 + 300 + 4 - 1) // 64
    assert torch.equal(w[0].targets[:-1], w[0].tokens[1:])


def test_synthetic_source_reference_spelling():
    a = ft.SyntheticTokenSource(vocab_size=100, seq_lens=[8, 16], seed=3)
    assert [len(s) for s in a.get_sequences(48)] == [8, 16, 8, 16]
    b = ft.SyntheticTokenSource(100, 8, seed=3)
    assert torch.equal(b.get_sequences(8)[0].tokens, ft.SyntheticTokenSource(100, seq_lens=8, seed=3).get_sequences(8)[0].tokens)


REF_YAML = """
model:
  arch: llama
  vocab_size: 512
  n_layers: 2
  d_model: 64
  n_heads: 4
  n_kv_heads: 2
  head_dim: 16
  expert_dim: 128
  rms_norm_eps: 0.00001
  rope_theta: 10000.0
  is_causal: true
train:
  global_batch_tokens: 512
  max_seq_len: 128
  total_steps: 3
  warmup_pct: 0.2
  cooldown_pct: 0.25
  final_lr_fraction: 0.1
  optimizer: {kind: adamw, lr: 0.001, beta1: 0.9, beta2: 0.95, eps: 0.00000001, weight_decay: 0.0}
hardware: {device_id: 0, max_gpu_mem_gib: 4.0, leeway_gpu_mem_gib: 1.0, max_chunk_size: 256}
io:
  output_dir: OUT
  save_final_checkpoint: false
  data: DATA
"""


def _ref_cfg(tmp_path, data: str, **repl):
    txt = REF_YAML.replace("OUT", str(tmp_path / "out")).replace("DATA", data)
    for k, v in repl.items():
        txt = txt.replace(k, v)
    p = tmp_path / "run.yaml"
    p.write_text(txt)
    return str(p)


def test_reference_run_file_layout_is_translated(tmp_path):
    import yaml
    cfg = RunConfig.from_yaml(_ref_cfg(tmp_path, "{synthetic: true, synthetic_seq_len: 128, min_seq_len: 64, max_seq_len: 128}"))
    assert cfg.model.inline_dims["d_model"] == 64 and cfg.model.hyperparams == {"rms_norm_eps": 1e-5, "rope_theta": 10000.0}
    assert cfg.train.steps == 3 and cfg.train.max_global_batch_tokens == 512 and cfg.train.max_chunk_size == 256
    assert cfg.optimizer.name == "adamw" and cfg.optimizer.lr == 1e-3 and cfg.optimizer.cooldown_start_pct == 0.75
    assert cfg.optimizer.final_pct == 0.1 and cfg.hardware.device_id == 0 and cfg.io.save is False
    assert cfg.data.source == "synthetic" and cfg.data.synthetic_seq_len == 128 and cfg.data.min_seq_len == 64
    assert is_reference_schema(yaml.safe_load(open(tmp_path / "run.yaml")))
    assert not is_reference_schema({"model": {"dims": "tiny_llama"}, "train": {"steps": 2}})
    # every source kind of the reference's data block
    (tmp_path / "rows.json").write_text("[]")
    kinds = {"{hf_dataset: org/name, hf_subset: s, hf_split: validation, hf_text_field: body, hf_streaming: false}":
             ("hf", "org/name"),
             "{shard_pattern: 'fw_{shard_index:06d}.bin', shard_num_shards: 3}": ("shards", "fw_{shard_index:06d}.bin"),
             "{raw_path: toks.pt}": ("raw", "toks.pt"),
             "{json_sft_path: rows.json, json_sft_prompt_field: q, json_sft_response_field: a, json_sft_loop: true}":
             ("json_sft", str(tmp_path / "rows.json")),
             "{custom_factory: 'pkg.mod:build'}": ("custom", None)}
    for block, (source, path) in kinds.items():
        c = RunConfig.from_yaml(_ref_cfg(tmp_path, block))
        assert (c.data.source, c.data.path) == (source, path), block
    c = RunConfig.from_yaml(_ref_cfg(tmp_path, "{hf_dataset: org/name, hf_subset: s, hf_split: validation, hf_streaming: false}"))
    assert (c.data.hf_subset, c.data.hf_split, c.data.hf_streaming) == ("s", "validation", False)
    c = RunConfig.from_yaml(_ref_cfg(tmp_path, "{shard_pattern: 'a*.bin', shard_num_shards: 3}"))
    assert c.data.shard_documents and c.data.shard_num_shards == 3
    # nothing is dropped silently
    with pytest.raises(ValueError, match="not understood"):
        RunConfig.from_yaml(_ref_cfg(tmp_path, "{synthetic: true, packing: dense}"))
    with pytest.raises(ValueError, match="exactly one data source"):
        RunConfig.from_yaml(_ref_cfg(tmp_path, "{synthetic: true, raw_path: x.pt}"))
    with pytest.raises(ValueError, match="causal"):
        RunConfig.from_yaml(_ref_cfg(tmp_path, "{synthetic: true}", **{"is_causal: true": "is_causal: false"}))


def _train(tmp_path, yaml_path, extra_env=None):
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT, str(tmp_path), os.environ.get("PYTHONPATH", "")]),
               CUDA_VISIBLE_DEVICES="", **(extra_env or {}))
    r = subprocess.run([sys.executable, "-m", "flextrain_b200", "train", yaml_path], capture_output=True, text=True,
                       env=env, timeout=600, cwd=str(tmp_path))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    return r.stdout


def test_reference_run_files_train_with_synthetic_raw_and_custom_sources(tmp_path):
    out = _train(tmp_path, _ref_cfg(tmp_path, "{synthetic: true, synthetic_seq_len: 128}"))
    assert out.count("[step") == 3 and "tok/step 512" in out
    dims = json.load(open(tmp_path / "out" / "model_dims.json"))
    assert dims["n_layers"] == 2 and dims["arch"] == "llama" and dims["hyperparams"]["rope_theta"] == 10000.0
    # pre-tokenised tensors
    g = torch.Generator().manual_seed(0)
    torch.save([torch.randint(0, 512, (128,), generator=g) for _ in range(12)], tmp_path / "toks.pt")
    out = _train(tmp_path, _ref_cfg(tmp_path, "{raw_path: toks.pt}"))
    assert out.count("[step") == 3 and "tok/step 512" in out
    # a user module: (records, extract)
    (tmp_path / "my_data.py").write_text(textwrap.dedent('''
        import torch
        from flextrain_b200.io import Sequence
        def build():
            records = [{"n": n} for n in range(64)]
            def extract(r):
                if r["n"] % 4 == 3:
                    return None
                return Sequence(torch.full((128,), r["n"] % 512, dtype=torch.int64))
            return records, extract
    '''))
    out = _train(tmp_path, _ref_cfg(tmp_path, "{custom_factory: 'my_data:build'}"))
    assert out.count("[step") == 3 and "tok/step 512" in out


def test_reference_run_file_with_json_sft_and_a_tokenizer_directory(tmp_path):
    """``io.tokenizer`` + ``io.data.json_sft_path`` with the record's own field names, on a model whose dimensions are
    written out in the file: the prompt is masked (fewer scored tokens than tokens) and the loss falls."""
    transformers = pytest.importorskip("transformers")
    from tokenizers import Tokenizer, models, pre_tokenizers
    chars = ["<unk>", "</s>"] + [chr(c) for c in range(32, 127)] + ["\n"]
    tok = Tokenizer(models.WordLevel({c: i for i, c in enumerate(chars)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split("", behavior="isolated")
    transformers.PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="</s>").save_pretrained(
        str(tmp_path / "tok"))
    rows = [{"q": f"{a}+{b}=", "a": str(a + b)} for a in range(6) for b in range(6)]
    (tmp_path / "rows.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    data = "{json_sft_path: rows.jsonl, json_sft_prompt_field: q, json_sft_response_field: a, json_sft_input_field: null}"
    path = _ref_cfg(tmp_path, data, **{"vocab_size: 512": f"vocab_size: {len(chars)}", "total_steps: 3": "total_steps: 12",
                                       "lr: 0.001": "lr: 0.01", "save_final_checkpoint: false":
                                       "save_final_checkpoint: false\n  tokenizer: tok"})
    cfg = RunConfig.from_yaml(path)
    assert cfg.data.tokenizer == str(tmp_path / "tok") and cfg.data.prompt_field == "q" and cfg.data.input_field is None
    out = _train(tmp_path, path)
    import re
    losses = [float(m) for m in re.findall(r"\[step\s+\d+\].*? loss ([\d.]+)", out)]
    assert len(losses) == 12 and losses[-1] < losses[0] - 0.3, losses
