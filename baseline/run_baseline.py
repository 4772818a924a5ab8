"""Unified launcher of the comparison harness: one run of one backend on synthetic tokens.

    python baseline/run_baseline.py --backend flextrain_b200 --model-preset llama3_1_8B --seq-length 1024 \
        --micro-batch-size 64 --gradient-accumulation-steps 8 --num-steps 3 --num-gpus 1 [--dry-run]
    python baseline/run_baseline.py --list

The run's stdout/stderr go to ``<output-dir>/<run-name>/stdout.log`` together with ``command.txt`` and, after the run,
``throughput.csv`` (one row per reported step).  ``--dry-run`` prints the command and exits
(reference: baseline/run_baseline.py in the reference tree).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from baseline.baseline_harness.backends import BACKENDS, format_command, get_backend  # noqa: E402
from baseline.baseline_harness.spec import RunSpec, detect_num_gpus  # noqa: E402
from baseline.scripts.sweep import extract_step_throughput, write_csv  # noqa: E402


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--backend", choices=sorted(BACKENDS))
    ap.add_argument("--list", action="store_true", help="list the backends and whether each is installed")
    ap.add_argument("--model-path", default=None)
    ap.add_argument("--model-preset", default="llama3_1_8B")
    ap.add_argument("--seq-length", type=int, default=1024)
    ap.add_argument("--micro-batch-size", type=int, default=1)
    ap.add_argument("--gradient-accumulation-steps", type=int, default=1)
    ap.add_argument("--num-steps", type=int, default=3)
    ap.add_argument("--warmup-steps", type=int, default=1)
    ap.add_argument("--num-gpus", type=int, default=None)
    ap.add_argument("--output-dir", default=os.path.join(HERE, "runs"))
    ap.add_argument("--run-name", default=None)
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE",
                    help="backend-specific knob (repeatable), e.g. --set dp_shard=opt+grad")
    ap.add_argument("--timeout", type=int, default=3600)
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--master-port", type=int, default=None)
    # Named spellings of the backend knobs (the reference's launcher spells them out one by one,
    # baseline/run_baseline.py there); each lands in the same dictionary as --set key=value, and a backend uses the
    # ones it knows.
    g = ap.add_argument_group("backend knobs (same as --set <name with underscores>=VALUE)")
    for flag, kind in KNOB_FLAGS:
        if kind is bool:
            g.add_argument("--" + flag, action="store_true", default=None)
        else:
            g.add_argument("--" + flag, type=kind, default=None)
    g.add_argument("--no-use-liger-kernel", dest="use_liger_kernel", action="store_false")
    g.add_argument("--backend-extra-arg", action="append", default=[], metavar="ARG",
                   help="raw argument appended to the backend's command line (repeatable)")
    return ap.parse_args(argv)


KNOB_FLAGS = (("activation-checkpointing", bool), ("activation-checkpoint-fraction", float),
              ("activation-checkpoint-interval", int), ("activation-checkpoint-selective-option", str),
              ("activation-offload", bool), ("attn-implementation", str), ("context-parallel-size", int),
              ("cpu-offloading-num-layers", int), ("fsdp-replicate-degree", int), ("fsdp-shard-degree", int),
              ("learning-rate", float), ("weight-decay", float), ("liger-kernel", bool), ("use-liger-kernel", bool),
              ("megatron-script", str), ("moe-kernel-backend", str), ("num-grad-slabs", int), ("offload-modules", str),
              ("optimizer-offload", bool), ("param-offload", bool), ("pipeline-parallel-size", int),
              ("recompute-granularity", str), ("recompute-method", str), ("recompute-modules", str),
              ("recompute-num-layers", int), ("save-activation-layer-fraction", float), ("sequence-parallel-size", int),
              ("tensor-parallel-size", int), ("tiled-loss-shards", int), ("tiled-mlp", bool),
              ("torchtitan-config", str), ("torchtitan-module", str), ("zero-stage", int))


def knob_extras(args) -> dict:
    out = {}
    for flag, _ in KNOB_FLAGS:
        v = getattr(args, flag.replace("-", "_"), None)
        if v is not None:
            out[flag.replace("-", "_")] = v
    if args.backend_extra_arg:
        out["backend_extra_args"] = list(args.backend_extra_arg)
    return out


def _parse_sets(items):
    out = {}
    for it in items:
        k, _, v = it.partition("=")
        if v.lower() in ("true", "false"):
            out[k] = v.lower() == "true"
        else:
            try:
                out[k] = int(v)
            except ValueError:
                out[k] = v
    return out


def run_spec(spec: RunSpec, *, dry_run: bool = False, timeout: int = 3600) -> dict:
    """Run (or print) one spec; returns a result record for sweeps."""
    backend = get_backend(spec.backend)
    ok, why = backend.available()
    cmd, env = backend.command(spec)
    line = format_command(cmd, env)
    rec = {"backend": spec.backend, "run": spec.name, "command": line, "status": "dry-run", "steps": []}
    if dry_run:
        print(line)
        return rec
    if not ok:
        rec.update(status="skipped", reason=why)
        print(f"[baseline] {spec.backend}: skipped ({why})")
        return rec
    os.makedirs(spec.run_dir, exist_ok=True)
    with open(os.path.join(spec.run_dir, "command.txt"), "w") as f:
        f.write(line + "\n")
    log = os.path.join(spec.run_dir, "stdout.log")
    with open(log, "w") as f:
        try:
            p = subprocess.run(cmd, env={**os.environ, **env}, stdout=f, stderr=subprocess.STDOUT, timeout=timeout)
            rec["status"] = "ok" if p.returncode == 0 else ("skipped" if p.returncode == 3 else "failed")
            rec["returncode"] = p.returncode
        except subprocess.TimeoutExpired:
            rec.update(status="failed", reason=f"timeout after {timeout}s")
    with open(log) as f:
        rec["steps"] = extract_step_throughput(f.read())
    write_csv(os.path.join(spec.run_dir, "throughput.csv"), [dict(backend=spec.backend, run=spec.name, **s)
                                                             for s in rec["steps"]])
    with open(os.path.join(spec.run_dir, "result.json"), "w") as f:
        json.dump(rec, f, indent=1)
    print(f"[baseline] {spec.backend}: {rec['status']}; {len(rec['steps'])} step lines; log {log}")
    return rec


def main(argv=None) -> int:
    args = parse_args(argv)
    if args.list:
        for name, b in sorted(BACKENDS.items()):
            ok, why = b.available()
            print(f"{name:18s} {'available' if ok else why:40s} {b.describe}")
        return 0
    if not args.backend:
        print("--backend is required (or --list)", file=sys.stderr)
        return 2
    spec = RunSpec(backend=args.backend, model_path=args.model_path, model_preset=args.model_preset,
                   seq_length=args.seq_length, micro_batch_size=args.micro_batch_size,
                   gradient_accumulation_steps=args.gradient_accumulation_steps, num_steps=args.num_steps,
                   warmup_steps=args.warmup_steps, num_gpus=args.num_gpus or detect_num_gpus() or 1,
                   output_dir=args.output_dir, run_name=args.run_name,
                   extra={**knob_extras(args), **_parse_sets(args.set)})
    if args.seed is not None:
        spec.seed = args.seed
    if args.master_port is not None:
        spec.master_port = args.master_port
    spec.validate()
    rec = run_spec(spec, dry_run=args.dry_run, timeout=args.timeout)
    return 0 if rec["status"] in ("ok", "dry-run", "skipped") else 1


if __name__ == "__main__":
    sys.exit(main())
