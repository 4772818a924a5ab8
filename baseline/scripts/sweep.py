"""TOML-driven sweep over backends, with per-step throughput extraction.

    python baseline/scripts/sweep.py baseline/configs/llama3_8b_b200.toml [--backends a,b] [--num-steps N]
                                     [--num-gpus N] [--dry-run]

The config has a ``[common]`` section (model, sequence length, batch shape, steps, GPUs) and one ``[<backend>]``
section per backend with that backend's knobs; ``${NUM_GPUS}`` in any string value is substituted at launch.  Sections
run in file order; a failing or missing backend is recorded and the sweep goes on.  At the end ``throughput.csv`` (one
row per reported step) and ``summary.json`` are written next to the run directories
(reference: baseline/scripts/sweep.py and extract_step_throughput.py in the reference tree).
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import re
import sys
from typing import Dict, List

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)

# "[step   3] ... loss 2.1 ... tok/s 21,950 ..."   (train.py of this repository)
_OURS = re.compile(r"\[step\s+(\d+)\].*?loss\s+([0-9.eE+-]+).*?tok/s\s+([0-9,\.]+)")
# "step 3: loss 2.1  812.0 ms  20177.3 tok/s ..."  (baseline/backends/hf_fsdp2.py and most third-party loops)
_GENERIC = re.compile(r"^\s*step\s+(\d+)\s*[:|].*?loss\s+([0-9.eE+-]+).*?([0-9][0-9,\.]*)\s*tok(?:ens)?/s", re.I)


def extract_step_throughput(text: str) -> List[Dict[str, float]]:
    """Per-step ``{"step", "loss", "tok_s"}`` records found in a training log; a ``bench.py`` JSON line counts as
    one record (step -1) with its ``value``."""
    out: List[Dict[str, float]] = []
    for line in text.splitlines():
        m = _OURS.search(line) or _GENERIC.search(line)
        if m:
            out.append({"step": int(m.group(1)), "loss": float(m.group(2)),
                        "tok_s": float(m.group(3).replace(",", ""))})
            continue
        s = line.strip()
        if s.startswith("{") and '"metric"' in s:
            try:
                d = json.loads(s)
                if "value" in d:
                    out.append({"step": -1, "loss": float(d.get("loss", float("nan"))), "tok_s": float(d["value"])})
            except ValueError:
                pass
    return out


def write_csv(path: str, rows: List[dict]) -> None:
    cols = ["backend", "run", "step", "loss", "tok_s"]
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=cols, extrasaction="ignore")
        w.writeheader()
        for r in rows:
            w.writerow(r)


def main(argv=None) -> int:
    from baseline.baseline_harness.spec import load_sweep, spec_from_sections
    from baseline.run_baseline import run_spec
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("config")
    ap.add_argument("--backends", default=None, help="comma-separated subset of the config's sections")
    ap.add_argument("--num-steps", type=int, default=None)
    ap.add_argument("--num-gpus", type=int, default=None)
    ap.add_argument("--output-dir", "--output-root", dest="output_dir", default=None)
    ap.add_argument("--timeout", type=int, default=3600)
    ap.add_argument("--dry-run", action="store_true")
    args = ap.parse_args(argv)
    data = load_sweep(args.config)
    common = dict(data["common"])
    sections = [k for k in data if k != "common"]
    if args.backends:
        want = args.backends.split(",")
        missing = [w for w in want if w not in sections]
        if missing:
            raise SystemExit(f"{args.config} has no section(s) {missing}; it has {sections}")
        sections = [s for s in sections if s in want]
    over = {}
    if args.num_steps is not None:
        over["num_steps"] = args.num_steps
    if args.output_dir:
        over["output_dir"] = args.output_dir
    records, rows = [], []
    for name in sections:
        section = dict(data[name])
        backend = section.pop("backend", name)           # several sections may drive the same backend
        section.setdefault("run_name", f"{os.path.splitext(os.path.basename(args.config))[0]}_{name}")
        try:
            spec = spec_from_sections(backend, common, section, over, num_gpus=args.num_gpus)
            rec = run_spec(spec, dry_run=args.dry_run, timeout=args.timeout)
        except Exception as e:                            # a broken section must not stop the sweep
            rec = {"backend": backend, "run": name, "status": "failed", "reason": f"{type(e).__name__}: {e}",
                   "steps": []}
            print(f"[sweep] {name}: {rec['reason']}")
        records.append(rec)
        rows += [dict(backend=rec["backend"], run=rec["run"], **s) for s in rec["steps"]]
    if not args.dry_run:
        out_dir = over.get("output_dir") or common.get("output_dir") or os.path.join(REPO, "baseline", "runs")
        os.makedirs(out_dir, exist_ok=True)
        write_csv(os.path.join(out_dir, "throughput.csv"), rows)
        with open(os.path.join(out_dir, "summary.json"), "w") as f:
            json.dump(records, f, indent=1)
    bad = [r for r in records if r["status"] == "failed"]
    print(f"[sweep] {len(records)} sections: " + ", ".join(f"{r['run']}={r['status']}" for r in records))
    return 1 if bad and not args.dry_run else 0


if __name__ == "__main__":
    sys.exit(main())
