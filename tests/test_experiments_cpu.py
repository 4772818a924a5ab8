"""The experiment drivers run end to end on CPU with tiny models (flextrain experiments/verified_runs.py,
experiments/scaling_law.py): table regeneration + regression diff, and the IsoFLOP grid + parabola fit."""
import importlib.util
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "experiments", name + ".py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_verified_runs_table_and_regression_diff(tmp_path):
    out = tmp_path / "t1"
    cmd = [sys.executable, os.path.join(ROOT, "experiments", "verified_runs.py"), "--rows", "tiny_llama:full,tiny_llama:lora",
           "--steps", "3", "--read-step", "2", "--seq-len", "64", "--batch", "512", "--out", str(out)]
    p = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-800:]
    rows = json.load(open(out / "rows.json"))
    assert [r["mode"] for r in rows] == ["full", "lora"] and all("loss" in r and r["tok_s"] > 0 for r in rows), rows
    assert (out / "table.md").read_text().count("tiny_llama") == 2
    # a second run diffs clean against the first on loss (the throughput of a CPU run on a shared box can move by orders of magnitude: leave it out of the comparison)
    out2 = tmp_path / "t2"
    cmd2 = cmd[:-1] + [str(out2), "--baseline", str(out), "--tok-s-tolerance", "1000.0"]
    p2 = subprocess.run(cmd2, capture_output=True, text=True, cwd=ROOT)
    assert p2.returncode == 0, p2.stdout[-800:] + p2.stderr[-800:]
    # and a doctored baseline loss is caught
    rows[0]["loss"] += 0.01
    json.dump(rows, open(out / "rows.json", "w"))
    p3 = subprocess.run(cmd[:-1] + [str(tmp_path / "t3"), "--baseline", str(out), "--tok-s-tolerance", "1000.0"],
                        capture_output=True, text=True, cwd=ROOT)
    assert p3.returncode != 0


def test_verified_runs_subcommands(tmp_path):
    """The reference's sub-command surface: run-one, report, compare."""
    vr = os.path.join(ROOT, "experiments", "verified_runs.py")
    out = tmp_path / "t"
    p = subprocess.run([sys.executable, vr, "run-one", "--row", "tiny_llama:full", "--out", str(out), "--steps", "2",
                        "--read-step", "2", "--seq-len", "64", "--batch", "512"], capture_output=True, text=True, cwd=ROOT)
    assert p.returncode == 0, p.stderr[-800:]
    assert (out / "tiny_llama_full" / "row.json").exists()
    p = subprocess.run([sys.executable, vr, "report", "--runs-dir", str(out)], capture_output=True, text=True, cwd=ROOT)
    assert p.returncode == 0 and "tiny_llama" in p.stdout and (out / "table.md").exists()
    p = subprocess.run([sys.executable, vr, "compare", "--baseline", str(out), "--rerun", str(out)],
                       capture_output=True, text=True, cwd=ROOT)
    assert p.returncode == 0, p.stdout
    rows = json.load(open(out / "rows.json"))
    rows[0]["loss"] += 0.01
    other = tmp_path / "u"
    other.mkdir()
    json.dump(rows, open(other / "rows.json", "w"))
    p = subprocess.run([sys.executable, vr, "compare", "--baseline", str(out), "--rerun", str(other)],
                       capture_output=True, text=True, cwd=ROOT)
    assert p.returncode == 1 and "DIFF" in p.stdout


def test_scaling_law_synthetic_grid(tmp_path):
    sl = _load("scaling_law")
    train, val, ent = sl.write_synthetic_corpus(str(tmp_path / "corpus"), 200_000, 512)
    arr = np.memmap(train, dtype=np.uint16, mode="r", offset=1024)
    assert len(arr) == 200_000 and int(arr.max()) < 512 and 1.0 < ent < 2.2
    res = sl.main(["--synthetic-corpus", "200000", "--vocab-size", "512", "--budgets", "2e10,6e10", "--ladder",
                   "64:1,64:2,128:2", "--out", str(tmp_path / "grid"), "--batch-tokens", "2048", "--seq-len", "64",
                   "--peak-lr", "3e-3", "--device", "cpu", "--eval-tokens", "4096"])
    assert len(res["rows"]) == 6 and set(res["fits"]) == {"2e+10", "6e+10"}
    for r in res["rows"]:
        assert np.isfinite(r["val_loss"]) and r["val_loss"] < np.log(512) + 0.1      # no worse than uniform guessing
    # more compute reaches a lower best loss
    best = {b: min(r["val_loss"] for r in res["rows"] if r["budget"] == b) for b in (2e10, 6e10)}
    assert best[6e10] < best[2e10]
    assert (tmp_path / "grid" / "table.md").exists()


def test_scaling_law_subcommands(tmp_path):
    """run-one adds a run directory; plot re-fits from what is on disk."""
    sl = _load("scaling_law")
    out = str(tmp_path / "g")
    common = ["--synthetic-corpus", "100000", "--vocab-size", "512", "--batch-tokens", "2048", "--seq-len", "64",
              "--peak-lr", "3e-3", "--device", "cpu", "--eval-tokens", "4096"]
    for d, L in ((64, 1), (64, 2), (128, 2)):
        sl.main(["run-one", "--d-model", str(d), "--n-layers", str(L), "--total-flops", "2e10", "--out", out] + common)
    res = sl.main(["plot", "--runs-dir", out])
    assert len(res["rows"]) == 3 and set(res["fits"]) == {"2e+10"}
    assert os.path.exists(os.path.join(out, "table.md")) and os.path.exists(os.path.join(out, "fit.json"))
    smoke = sl.main(["run-grid", "--out", str(tmp_path / "s"), "--smoke", "--budgets", "1e10,2e10,4e10", "--ladder",
                     "64:1,64:2,128:2"] + common)
    assert len(smoke["rows"]) == 4                         # 2 budgets x 2 sizes


def test_parabola_fit_recovers_a_known_optimum():
    sl = _load("scaling_law")
    ns = np.array([1e6, 3e6, 1e7, 3e7, 1e8])
    ls = 2.0 + 0.05 * (np.log(ns) - np.log(8e6)) ** 2
    fit = sl.fit_parabola(ns, ls)
    assert abs(fit["n_opt"] / 8e6 - 1) < 1e-6 and abs(fit["loss_opt"] - 2.0) < 1e-9
