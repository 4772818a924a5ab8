"""Regenerate the throughput table: one ``train.py`` subprocess per row, parse a chosen step's log line, write a
markdown table, optionally diff against a baseline directory (loss exact to 4 decimals, tok/s within 5 %)
(flextrain experiments/verified_runs.py:48-110).

    python experiments/verified_runs.py --rows llama3_1_8B:full,qwen3_8B:full --steps 5 --read-step 3 --out runs/table

The reference's sub-commands are available too (flextrain experiments/verified_runs.py:795-840):

    python experiments/verified_runs.py run-one  --row llama3_1_8B:full --out runs/table
    python experiments/verified_runs.py run-grid --out runs/table [--only llama3_1_8B:full qwen3_8B:full]
    python experiments/verified_runs.py report   --runs-dir runs/table
    python experiments/verified_runs.py compare  --baseline runs/trusted --rerun runs/table \
        [--loss-atol 1e-4] [--throughput-rel-tol 0.05]
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


DEFAULT_ROWS = "llama3_2_1B:full,llama3_1_8B:full,llama3_1_8B:lora,qwen3_8B:full"
HEADER = ("| model | mode | gpus | loss | tok/s | TFLOPS eff | TFLOPS hw | max alloc GiB |\n"
          "|---|---|---|---|---|---|---|---|\n")


def write_table(out_dir: str, rows) -> str:
    json.dump(rows, open(os.path.join(out_dir, "rows.json"), "w"), indent=1)
    path = os.path.join(out_dir, "table.md")
    with open(path, "w") as f:
        f.write(HEADER)
        for r in rows:
            f.write(f"| {r['model']} | {r['mode']} | {r['gpus']} | {r.get('loss', 'ERR')} | {r.get('tok_s', '')} | "
                    f"{r.get('tflops_eff', '')} | {r.get('tflops_hw', '')} | {r.get('max_alloc_gib', '')} |\n")
    return path


def load_rows(d: str):
    """Rows of a table directory: ``rows.json``, merged with any ``<model>_<mode>/row.json`` written by ``run-one``."""
    rows = {}
    p = os.path.join(d, "rows.json")
    if os.path.exists(p):
        for r in json.load(open(p)):
            rows[(r["model"], r["mode"])] = r
    for sub in sorted(os.listdir(d)):
        rp = os.path.join(d, sub, "row.json")
        if os.path.exists(rp):
            r = json.load(open(rp))
            rows[(r["model"], r["mode"])] = r
    return list(rows.values())


def compare(baseline_dir: str, rerun_dir: str, loss_atol: float, tput_rel_tol: float) -> int:
    """Number of rows whose loss moved by more than ``loss_atol`` or whose throughput moved by more than
    ``tput_rel_tol`` (relative), printed one per line."""
    old = {(r["model"], r["mode"]): r for r in load_rows(baseline_dir)}
    bad = 0
    for r in load_rows(rerun_dir):
        o = old.get((r["model"], r["mode"]))
        if o and "loss" in o and "loss" in r:
            if abs(o["loss"] - r["loss"]) > loss_atol or abs(o["tok_s"] - r["tok_s"]) > tput_rel_tol * o["tok_s"]:
                print("DIFF", r["model"], r["mode"], o["loss"], r["loss"], o["tok_s"], r["tok_s"])
                bad += 1
        elif o is not None or "loss" not in r:
            print("MISSING", r["model"], r["mode"])
            bad += 1
    return bad


def _common(ap):
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--read-step", type=int, default=3)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=65536)
    ap.add_argument("--gpus", type=int, default=1)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in ("run-one", "run-grid", "report", "compare"):
        ap = argparse.ArgumentParser(prog="verified_runs.py")
        sub = ap.add_subparsers(dest="cmd", required=True)
        p1 = sub.add_parser("run-one", help="one row: <dims name>:<mode>")
        p1.add_argument("--row", required=True)
        p1.add_argument("--out", required=True)
        _common(p1)
        p2 = sub.add_parser("run-grid", help="all rows (or --only some) and the table")
        p2.add_argument("--out", required=True)
        p2.add_argument("--only", nargs="+", default=None)
        p2.add_argument("--rows", default=os.environ.get("FLEXTRAIN_VERIFIED_ROWS", DEFAULT_ROWS))
        _common(p2)
        p3 = sub.add_parser("report", help="rebuild table.md from the rows found under a directory")
        p3.add_argument("--runs-dir", required=True)
        p4 = sub.add_parser("compare", help="diff two table directories (regression check)")
        p4.add_argument("--baseline", required=True)
        p4.add_argument("--rerun", required=True)
        p4.add_argument("--loss-atol", type=float, default=1e-4)
        p4.add_argument("--throughput-rel-tol", type=float, default=0.05)
        a, extra = ap.parse_known_args(argv)
        if a.cmd == "run-one":
            os.makedirs(a.out, exist_ok=True)
            model, mode = a.row.split(":")
            r = run_row(model, mode, a.steps, a.read_step, a.seq_len, a.batch, a.gpus, extra, a.out)
            d = os.path.join(a.out, f"{os.path.basename(model)}_{mode}")
            os.makedirs(d, exist_ok=True)
            json.dump(r, open(os.path.join(d, "row.json"), "w"), indent=1)
            print(json.dumps(r))
            return 0 if "loss" in r else 1
        if a.cmd == "run-grid":
            os.makedirs(a.out, exist_ok=True)
            names = a.only or a.rows.split(",")
            rows = [run_row(*n.split(":"), a.steps, a.read_step, a.seq_len, a.batch, a.gpus, extra, a.out) for n in names]
            print(open(write_table(a.out, rows)).read())
            return 0 if all("loss" in r for r in rows) else 1
        if a.cmd == "report":
            print(open(write_table(a.runs_dir, load_rows(a.runs_dir))).read())
            return 0
        return 1 if compare(a.baseline, a.rerun, a.loss_atol, a.throughput_rel_tol) else 0
    # flat form: run the rows, write the table, optionally diff against --baseline
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", default=DEFAULT_ROWS)
    _common(ap)
    ap.add_argument("--out", default="runs/verified")
    ap.add_argument("--baseline", default=None)
    ap.add_argument("--loss-atol", type=float, default=5e-5)
    ap.add_argument("--tok-s-tolerance", "--throughput-rel-tol", dest="tok_s_tolerance", type=float, default=0.05,
                    help="allowed relative throughput change vs --baseline")
    a, extra = ap.parse_known_args(argv)
    os.makedirs(a.out, exist_ok=True)
    rows = [run_row(*r.split(":"), a.steps, a.read_step, a.seq_len, a.batch, a.gpus, extra, a.out)
            for r in a.rows.split(",")]
    table = write_table(a.out, rows)
    bad = compare(a.baseline, a.out, a.loss_atol, a.tok_s_tolerance) if a.baseline else 0
    print(open(table).read())
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
