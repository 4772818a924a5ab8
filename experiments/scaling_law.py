"""IsoFLOP (Chinchilla-style) grid over ``from_dims`` models (flextrain experiments/scaling_law.py:1-70): for each
compute budget, train a ladder of widths / depths to that budget with ``python -m flextrain_b200 pretrain`` and fit
``L(N) = a + b * (log N - log N_opt)^2`` per budget.

    python experiments/scaling_law.py --train-shards 'data/fineweb_train_*.bin' --val-shards 'data/fineweb_val_*.bin' \
        --budgets 1e17,3e17,1e18 --out runs/scaling_law
"""
import argparse
import json
import math
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LADDER = [(384, 6), (512, 8), (640, 10), (768, 10), (896, 12), (1024, 14), (1280, 16)]      # (d_model, layers)


def dims_for(d: int, L: int, vocab: int = 50304) -> dict:
    hd = 128 if d % 128 == 0 else 64
    return {"arch": "llama", "vocab_size": vocab, "n_layers": L, "d_model": d, "n_heads": d // hd, "n_kv_heads": d // hd,
            "head_dim": hd, "expert_dim": ((4 * d * 2 // 3) + 127) // 128 * 128,
            "hyperparams": {"rope_theta": 10000.0, "norm_eps": 1e-5}}


def fit_parabola(ns, ls):
    import numpy as np
    x = np.log(np.asarray(ns)); y = np.asarray(ls)
    c = np.polyfit(x, y, 2)
    xo = -c[1] / (2 * c[0])
    return {"n_opt": float(math.exp(xo)), "loss_opt": float(np.polyval(c, xo)), "coef": [float(v) for v in c]}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--train-shards", required=True)
    ap.add_argument("--val-shards", required=True)
    ap.add_argument("--budgets", default="1e17,3e17,1e18")
    ap.add_argument("--out", default="runs/scaling_law")
    ap.add_argument("--batch-tokens", type=int, default=131072)
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    fits = {}
    for b in [float(x) for x in a.budgets.split(",")]:
        pts = []
        for d, L in LADDER:
            run = os.path.join(a.out, f"F{b:.0e}_d{d}_L{L}")
            os.makedirs(run, exist_ok=True)
            dj = os.path.join(run, "dims.json")
            json.dump(dims_for(d, L), open(dj, "w"))
            subprocess.run([sys.executable, "-m", "flextrain_b200", "pretrain", "--dims", dj, "--train-shards",
                            a.train_shards, "--val-shards", a.val_shards, "--out", run, "--flop-budget", str(b),
                            "--batch-tokens", str(a.batch_tokens)], cwd=ROOT, check=False)
            fj = os.path.join(run, "final.json")
            if os.path.exists(fj):
                fin, meta = json.load(open(fj)), json.load(open(os.path.join(run, "meta.json")))
                if fin.get("val_loss") is not None:
                    pts.append((meta["n_params"], fin["val_loss"]))
        if len(pts) >= 3:
            fits[f"{b:.0e}"] = fit_parabola(*zip(*pts))
    json.dump(fits, open(os.path.join(a.out, "fit.json"), "w"), indent=1)
    print(json.dumps(fits, indent=1))
