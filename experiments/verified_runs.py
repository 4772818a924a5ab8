"""Regenerate the throughput table: one ``train.py`` subprocess per row, parse a chosen step's log line, write a
markdown table, optionally diff against a baseline directory (loss exact to 4 decimals, tok/s within 5 %)
(flextrain experiments/verified_runs.py:48-110).

    python experiments/verified_runs.py --rows llama3_1_8B:full,qwen3_8B:full --steps 5 --read-step 3 --out runs/table
"""
import argparse
import json
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LINE = re.compile(r"\[step\s+(\d+)\].*loss ([\d.]+).*tok/s ([\d,]+) TFLOPS_eff ([\d.]+) TFLOPS_hw ([\d.]+) max_alloc ([\d.]+)")


def run_row(model: str, mode: str, steps: int, read_step: int, seq_len: int, batch: int, gpus: int, extra, out_dir=None):
    base = [sys.executable] if gpus == 1 else [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                                               f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1"]
    cmd = base + [os.path.join(ROOT, "train.py"), "--model", f"dims:{model}" if not os.path.isdir(model) else model,
                  "--mode", mode, "--max-seq-len", str(seq_len), "--max-global-batch-tokens", str(batch), "--steps",
                  str(steps), "--data-source", "synthetic"] + list(extra)
    if out_dir and "--output-dir" not in extra:        # keep each row's train.py outputs under this table's directory
        cmd += ["--output-dir", os.path.join(out_dir, f"{os.path.basename(str(model))}_{mode}")]
    p = subprocess.run(cmd, capture_output=True, text=True)
    row = {"model": model, "mode": mode, "gpus": gpus, "rc": p.returncode}
    for m in LINE.finditer(p.stdout):
        if int(m.group(1)) == read_step:
            row.update(loss=float(m.group(2)), tok_s=float(m.group(3).replace(",", "")), tflops_eff=float(m.group(4)),
                       tflops_hw=float(m.group(5)), max_alloc_gib=float(m.group(6)))
    if "loss" not in row:
        row["error"] = (p.stderr or p.stdout)[-400:]
    return row


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default="llama3_2_1B:full,llama3_1_8B:full,llama3_1_8B:lora,qwen3_8B:full")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--read-step", type=int, default=3)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=65536)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--out", default="runs/verified")
    ap.add_argument("--baseline", default=None)
    ap.add_argument("--tok-s-tolerance", type=float, default=0.05, help="allowed relative throughput change vs --baseline")
    a, extra = ap.parse_known_args()
    os.makedirs(a.out, exist_ok=True)
    rows = [run_row(*r.split(":"), a.steps, a.read_step, a.seq_len, a.batch, a.gpus, extra, a.out)
            for r in a.rows.split(",")]
    json.dump(rows, open(os.path.join(a.out, "rows.json"), "w"), indent=1)
    with open(os.path.join(a.out, "table.md"), "w") as f:
        f.write("| model | mode | gpus | loss | tok/s | TFLOPS eff | TFLOPS hw | max alloc GiB |\n|---|---|---|---|---|---|---|---|\n")
        for r in rows:
            f.write(f"| {r['model']} | {r['mode']} | {r['gpus']} | {r.get('loss', 'ERR')} | {r.get('tok_s', '')} | "
                    f"{r.get('tflops_eff', '')} | {r.get('tflops_hw', '')} | {r.get('max_alloc_gib', '')} |\n")
    bad = 0
    if a.baseline:
        old = {(r["model"], r["mode"]): r for r in json.load(open(os.path.join(a.baseline, "rows.json")))}
        for r in rows:
            o = old.get((r["model"], r["mode"]))
            if o and "loss" in o and "loss" in r:
                if abs(o["loss"] - r["loss"]) > 5e-5 or abs(o["tok_s"] - r["tok_s"]) > a.tok_s_tolerance * o["tok_s"]:
                    print("DIFF", r["model"], r["mode"], o["loss"], r["loss"], o["tok_s"], r["tok_s"])
                    bad += 1
    print(open(os.path.join(a.out, "table.md")).read())
    sys.exit(1 if bad else 0)
