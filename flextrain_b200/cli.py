"""``python -m flextrain_b200 {info,check,train <yaml>,pretrain,init}`` (flextrain/cli.py:669-697)."""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List


def _info(args) -> int:
    import torch

    import flextrain_b200 as ft
    from .build import CSRC, LIB
    from .core._memory import get_available_gpu_memory, get_available_host_memory
    from .io.arch import ARCH_MODULES
    print(f"flextrain_b200 {ft.__version__}")
    print(f"torch {torch.__version__}, CUDA available: {torch.cuda.is_available()}")
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            print(f"  cuda:{i} {p.name} sm_{p.major}{p.minor} {p.total_memory / 2**30:.0f} GiB, {p.multi_processor_count} SMs")
        print(f"free GPU memory: {get_available_gpu_memory('cuda:0') / 2**30:.1f} GiB")
    print(f"available host memory: {get_available_host_memory() / 2**30:.1f} GiB")
    print("architectures:", ", ".join(sorted(set(ARCH_MODULES.values()))))
    libs = sorted(p.name for p in LIB.glob("*.so")) if LIB.exists() else []
    print("native libraries:", ", ".join(libs) or "(not built; run python -m flextrain_b200.build)")
    return 0


def _train_argv(cfg) -> List[str]:
    """Translate a RunConfig into train.py flags: both front ends drive the same loop."""
    m, o, t, h, d, io = cfg.model, cfg.optimizer, cfg.train, cfg.hardware, cfg.data, cfg.io
    model = m.path or f"dims:{m.dims}"
    if not m.path and m.inline_dims:
        # dimensions written out in the run file: handed to train.py as a dims file next to the run's outputs
        os.makedirs(io.output_dir, exist_ok=True)
        dims_file = os.path.join(io.output_dir, "model_dims.json")
        with open(dims_file, "w") as f:
            json.dump(dict(m.inline_dims, arch=m.arch, **({"hyperparams": m.hyperparams} if m.hyperparams else {})), f)
        model = f"dims:{dims_file}"
    argv = ["--model", model, "--mode", m.mode, "--max-seq-len", str(t.max_seq_len),
            "--max-global-batch-tokens", str(t.max_global_batch_tokens), "--steps", str(t.steps),
            "--data-source", d.source, "--lr", str(o.lr), "--lr-warmup-pct", str(o.warmup_pct),
            "--lr-cooldown-start-pct", str(o.cooldown_start_pct), "--lr-final-pct", str(o.final_pct),
            "--lora-rank", str(m.lora_rank), "--lora-alpha", str(m.lora_alpha), "--opt-state-dtype", o.state_dtype,
            "--attn-backend", h.attn_backend, "--leeway-gpu-mem-gib", str(h.leeway_gpu_mem_gib),
            "--leeway-host-mem-gib", str(h.leeway_host_mem_gib), "--output-dir", io.output_dir, "--seed", str(t.seed),
            "--tp", str(h.tp), "--ep", str(h.ep)]
    if d.path:
        argv += ["--dataset", d.path]
    if d.synthetic_seq_len:
        argv += ["--synthetic-seq-len", str(d.synthetic_seq_len)]
    if o.name == "muon":
        argv.append("--use-muon")
    for flag, val in (("--max-gpu-mem-gib", h.max_gpu_mem_gib), ("--max-host-mem-gib", h.max_host_mem_gib),
                      ("--force-save-level", t.force_save_level), ("--min-chunk-size", t.min_chunk_size),
                      ("--max-chunk-size", t.max_chunk_size), ("--dp-shard", h.dp_shard),
                      ("--save-state-every", io.save_state_every or None), ("--resume-state", io.resume_state),
                      ("--eval-every", io.eval_every or None), ("--eval-tokens", io.eval_tokens if io.eval_every else None),
                      ("--eval-dataset", d.eval_path), ("--max-grad-norm", o.max_grad_norm),
                      ("--device-id", h.device_id), ("--tokenizer", d.tokenizer), ("--min-seq-len", d.min_seq_len or None),
                      ("--hf-subset", d.hf_subset), ("--shard-num-shards", d.shard_num_shards),
                      ("--custom-factory", d.custom_factory)):
        if val is not None:
            argv += [flag, str(val)]
    argv += ["--hf-split", d.hf_split, "--hf-text-field", d.hf_text_field, "--sft-prompt-field", d.prompt_field,
             "--sft-response-field", d.response_field, "--sft-input-field", d.input_field or ""]
    for flag, on in (("--save", io.save), ("--apply-chat-template", d.apply_chat_template),
                     ("--truncate-long", d.truncate_long), ("--no-hf-streaming", not d.hf_streaming),
                     ("--shard-documents", d.shard_documents)):
        if on:
            argv.append(flag)
    return argv


def _train(args) -> int:
    from .config import RunConfig
    cfg = RunConfig.from_yaml(args.config)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import train as train_mod
    argv = _train_argv(cfg)
    if cfg.io.resume_from:
        # weights-only resume: the exported HF directory of the earlier run becomes the model to load
        i = argv.index("--model")
        argv[i + 1] = cfg.io.resume_from
    return train_mod.main(argv)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m flextrain_b200")
    sub = p.add_subparsers(dest="cmd", required=True)
    sub.add_parser("info", help="versions, devices, memory, architectures, native libraries")
    t = sub.add_parser("train", help="train from a YAML run config")
    t.add_argument("config")
    c = sub.add_parser("check", help="build the native libraries and check tool chain, libraries, GPUs, peer access")
    c.add_argument("--no-build", action="store_true")
    c.add_argument("--json", action="store_true")
    from .scripts import init_hf, pretrain
    pretrain.add_subparser(sub)
    init_hf.add_subparser(sub)
    args = p.parse_args(argv)
    if args.cmd == "info":
        return _info(args)
    if args.cmd == "check":
        from .scripts import post_install
        return post_install.main((["--no-build"] if args.no_build else []) + (["--json"] if args.json else []))
    if args.cmd == "train":
        return _train(args)
    return args.func(args)


if __name__ == "__main__":
    sys.exit(main())
