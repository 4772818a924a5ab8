"""IsoFLOP (Chinchilla-style) grid over ``from_dims`` models (flextrain experiments/scaling_law.py:1-70): for each
compute budget, train a ladder of widths / depths to that budget with ``python -m flextrain_b200 pretrain`` and fit
``L(N) = c0 * (log N)^2 + c1 * log N + c2`` per budget; the vertex is the compute-optimal size.

    python experiments/scaling_law.py --train-shards 'data/fineweb_train_*.bin' --val-shards 'data/fineweb_val_*.bin' \
        --budgets 1e17,3e17,1e18 --out runs/scaling_law

The reference's sub-commands are available too (flextrain experiments/scaling_law.py:625-660): ``run-one --d-model D
--n-layers L --total-flops F --out DIR``, ``run-grid --out DIR [--smoke]`` (``--smoke``: 2 budgets x 2 sizes) and ``plot
--runs-dir DIR`` (re-fit and re-write the tables from the ``final.json`` / ``meta.json`` files found there; draws
``isoflop.png`` when matplotlib is importable).  They take the same corpus flags as the flat form.

Without a corpus (``--synthetic-corpus TOKENS``) the grid runs on token shards drawn from a fixed sparse second-order
Markov source, so the curve has structure to learn and an entropy floor that is known in closed form; the shards
are written once under ``<out>/corpus`` in the FineWeb shard format.
"""
import argparse
import json
import math
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LADDER = [(384, 6), (512, 8), (640, 10), (768, 10), (896, 12), (1024, 14), (1280, 16)]      # (d_model, layers)
MAGIC = 20240520


def dims_for(d: int, L: int, vocab: int = 50304) -> dict:
    hd = 128 if d % 128 == 0 else 64
    return {"arch": "llama", "vocab_size": vocab, "n_layers": L, "d_model": d, "n_heads": d // hd, "n_kv_heads": d // hd,
            "head_dim": hd, "expert_dim": ((4 * d * 2 // 3) + 127) // 128 * 128,
            "hyperparams": {"rope_theta": 10000.0, "norm_eps": 1e-5}}


def fit_parabola(ns, ls):
    x = np.log(np.asarray(ns, dtype=np.float64)); y = np.asarray(ls, dtype=np.float64)
    c = np.polyfit(x, y, 2)
    out = {"coef": [float(v) for v in c], "points": [[float(n), float(l)] for n, l in zip(ns, ls)]}
    if c[0] > 0:                                   # a minimum exists inside or outside the ladder
        xo = -c[1] / (2 * c[0])
        out.update(n_opt=float(math.exp(xo)), loss_opt=float(np.polyval(c, xo)))
    else:                                          # monotone over the ladder: report the best measured point
        i = int(np.argmin(y))
        out.update(n_opt=float(ns[i]), loss_opt=float(ls[i]), monotone=True)
    return out


def markov_source(vocab: int, branch: int = 8, seed: int = 0, context_classes: int = 64):
    """Sparse second-order source: the pair (class of a, b) hashes to ``branch`` candidate successors with fixed
    geometric weights, where ``class of a = a mod context_classes``.  A bigram model can only average over the classes;
    the full table has ``context_classes * vocab * branch`` entries, so within a small compute budget a larger model
    learns more of it per token while a smaller one sees more tokens: the IsoFLOP trade-off has something to act on.
    Returns ``(successor fn, weights, entropy in nats per token)``."""
    w = 0.5 ** np.arange(1, branch + 1); w[-1] *= 2.0; w /= w.sum()
    ent = float(-(w * np.log(w)).sum())
    rng = np.random.default_rng(seed)
    mul = rng.integers(1, 2 ** 31 - 1, size=(branch, 2), dtype=np.int64) | 1

    def successors(a, b):
        a = a % context_classes
        return ((a[:, None] * mul[None, :, 0] + b[:, None] * mul[None, :, 1] + np.arange(branch)[None, :] * 40503)
                % 2147483647) % vocab
    return successors, w, ent


def write_synthetic_corpus(out_dir: str, n_tokens: int, vocab: int, seed: int = 0, streams: int = 4096):
    """Write ``train`` and ``val`` shards (uint16 with the 256-int32 header) and return ``(train glob, val path, entropy)``."""
    os.makedirs(out_dir, exist_ok=True)
    succ, w, ent = markov_source(vocab, seed=seed)
    rng = np.random.default_rng(seed + 1)
    paths = {}
    for kind, n in (("train", n_tokens), ("val", max(n_tokens // 20, 65536))):
        p = os.path.join(out_dir, f"fineweb_{kind}_000001.bin")
        paths[kind] = p
        if os.path.exists(p) and os.path.getsize(p) == 1024 + 2 * n:
            continue
        steps = (n + streams - 1) // streams
        a = rng.integers(0, vocab, streams); b = rng.integers(0, vocab, streams)
        toks = np.empty((steps, streams), dtype=np.uint16)
        for t in range(steps):                       # `streams` independent chains advance together (vectorised)
            pick = rng.choice(len(w), size=streams, p=w)
            c = succ(a, b)[np.arange(streams), pick]
            toks[t] = c
            a, b = b, c
        flat = toks.T.reshape(-1)[:n]                # one chain after another: contiguous windows stay in-chain
        head = np.zeros(256, dtype=np.int32); head[0], head[1], head[2] = MAGIC, 1, n
        with open(p, "wb") as f:
            f.write(head.tobytes()); f.write(flat.tobytes())
    return paths["train"], paths["val"], ent


def collect(out_dir: str):
    """``(rows, fits)`` from the ``F<budget>_d<d>_L<L>`` run directories under ``out_dir``."""
    rows = []
    for name in sorted(os.listdir(out_dir)):
        run = os.path.join(out_dir, name)
        fj, mj = os.path.join(run, "final.json"), os.path.join(run, "meta.json")
        if not (name.startswith("F") and os.path.exists(fj) and os.path.exists(mj)):
            continue
        fin, meta = json.load(open(fj)), json.load(open(mj))
        if fin.get("val_loss") is None:
            continue
        b = float(name[1:].split("_")[0])
        rows.append({"budget": b, "d_model": meta["dims"]["d_model"], "n_layers": meta["dims"]["n_layers"],
                     "n_params": meta["n_params"], "val_loss": fin["val_loss"], "steps": fin.get("steps"),
                     "tokens": fin.get("tokens")})
    rows.sort(key=lambda r: (r["budget"], r["n_params"]))
    fits = {}
    for b in sorted({r["budget"] for r in rows}):
        pts = [(r["n_params"], r["val_loss"]) for r in rows if r["budget"] == b]
        if len(pts) >= 3:
            fits[f"{b:.0e}"] = fit_parabola(*zip(*pts))
    return rows, fits


def write_tables(out_dir: str, rows, fits, entropy=None) -> None:
    json.dump({"fits": fits, "rows": rows, "source_entropy_nats": entropy}, open(os.path.join(out_dir, "fit.json"), "w"),
              indent=1)
    with open(os.path.join(out_dir, "table.md"), "w") as f:
        f.write("| FLOP budget | d_model | layers | parameters | steps | val loss |\n|---|---|---|---|---|---|\n")
        for r in rows:
            f.write(f"| {r['budget']:.0e} | {r['d_model']} | {r['n_layers']} | {r['n_params']:,} | {r['steps']} | "
                    f"{r['val_loss']:.4f} |\n")
        f.write("\n| FLOP budget | compute-optimal parameters (fit) | loss at optimum |\n|---|---|---|\n")
        for k, v in fits.items():
            f.write(f"| {k} | {v['n_opt']:,.0f}{' (monotone over the ladder)' if v.get('monotone') else ''} | "
                    f"{v['loss_opt']:.4f} |\n")
        if entropy is not None:
            f.write(f"\nEntropy of the synthetic source: {entropy:.4f} nats per token (the loss floor).\n")


def plot(out_dir: str, rows, fits) -> bool:
    """IsoFLOP curves as ``isoflop.png`` (best effort: needs matplotlib)."""
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        return False
    fig, ax = plt.subplots(figsize=(6, 4))
    for b in sorted({r["budget"] for r in rows}):
        pts = sorted((r["n_params"], r["val_loss"]) for r in rows if r["budget"] == b)
        ax.plot([p[0] for p in pts], [p[1] for p in pts], "o-", label=f"{b:.0e} FLOPs")
    ax.set_xscale("log"); ax.set_xlabel("parameters"); ax.set_ylabel("validation loss"); ax.legend()
    fig.tight_layout(); fig.savefig(os.path.join(out_dir, "isoflop.png"), dpi=120)
    return True


def train_one(a, d: int, L: int, budget: float, run: str, vocab: int) -> None:
    os.makedirs(run, exist_ok=True)
    dj = os.path.join(run, "dims.json")
    json.dump(dims_for(d, L, vocab), open(dj, "w"))
    cmd = [sys.executable, "-m", "flextrain_b200", "pretrain", "--dims", dj, "--train-shards", a.train_shards,
           "--val-shards", a.val_shards, "--out", run, "--flop-budget", str(budget), "--batch-tokens",
           str(a.batch_tokens), "--max-seq-len", str(a.seq_len)]
    if a.peak_lr:
        cmd += ["--peak-lr", str(a.peak_lr)]
    if getattr(a, "init_seed", None) is not None:
        cmd += ["--init-seed", str(a.init_seed)]
    if a.device:
        cmd += ["--device", a.device]
    if a.eval_tokens:
        cmd += ["--eval-tokens", str(a.eval_tokens)]
    subprocess.run(cmd, cwd=ROOT, check=False)


def _corpus_flags(ap) -> None:
    ap.add_argument("--train-shards", default=None)
    ap.add_argument("--val-shards", default=None)
    ap.add_argument("--synthetic-corpus", type=int, default=0, metavar="TOKENS",
                    help="write a Markov-source corpus of this many training tokens and use it")
    ap.add_argument("--vocab-size", type=int, default=None, help="default 50304, or 4096 with --synthetic-corpus")
    ap.add_argument("--batch-tokens", type=int, default=131072)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--peak-lr", type=float, default=None)
    ap.add_argument("--device", default=None)
    ap.add_argument("--eval-tokens", type=int, default=None)


def _resolve_corpus(ap, a):
    vocab = a.vocab_size or (4096 if a.synthetic_corpus else 50304)
    entropy = None
    if a.synthetic_corpus:
        a.train_shards, a.val_shards, entropy = write_synthetic_corpus(os.path.join(a.out, "corpus"), a.synthetic_corpus,
                                                                       vocab)
    if not a.train_shards or not a.val_shards:
        ap.error("give --train-shards and --val-shards, or --synthetic-corpus")
    return vocab, entropy


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    sub_cmd = argv[0] if argv and argv[0] in ("run-one", "run-grid", "plot") else None
    ap = argparse.ArgumentParser()
    if sub_cmd == "plot":
        ap.add_argument("--runs-dir", required=True)
        a = ap.parse_args(argv[1:])
        rows, fits = collect(a.runs_dir)
        write_tables(a.runs_dir, rows, fits)
        drew = plot(a.runs_dir, rows, fits)
        print(json.dumps({"rows": len(rows), "fits": fits, "png": drew}, indent=1))
        return {"fits": fits, "rows": rows}
    if sub_cmd == "run-one":
        ap.add_argument("--d-model", type=int, required=True)
        ap.add_argument("--n-layers", type=int, required=True)
        ap.add_argument("--total-flops", type=float, required=True)
        ap.add_argument("--out", required=True)
        ap.add_argument("--init-seed", type=int, default=42)
        _corpus_flags(ap)
        a = ap.parse_args(argv[1:])
        os.makedirs(a.out, exist_ok=True)
        vocab, _ = _resolve_corpus(ap, a)
        train_one(a, a.d_model, a.n_layers, a.total_flops,
                  os.path.join(a.out, f"F{a.total_flops:.0e}_d{a.d_model}_L{a.n_layers}"), vocab)
        rows, fits = collect(a.out)
        return {"fits": fits, "rows": rows}
    _corpus_flags(ap)
    ap.add_argument("--budgets", default="1e17,3e17,1e18")
    ap.add_argument("--ladder", default=None, help="'d:L,d:L,...' replacing the default width / depth ladder")
    ap.add_argument("--out", default="runs/scaling_law")
    ap.add_argument("--smoke", action="store_true", help="2 budgets x 2 sizes")
    a = ap.parse_args(argv[1:] if sub_cmd == "run-grid" else argv)
    os.makedirs(a.out, exist_ok=True)
    vocab, entropy = _resolve_corpus(ap, a)
    ladder = [tuple(int(v) for v in p.split(":")) for p in a.ladder.split(",")] if a.ladder else LADDER
    budgets = [float(x) for x in a.budgets.split(",")]
    if a.smoke:
        ladder, budgets = ladder[:2], budgets[:2]
    for b in budgets:
        for d, L in ladder:
            train_one(a, d, L, b, os.path.join(a.out, f"F{b:.0e}_d{d}_L{L}"), vocab)
    rows, fits = collect(a.out)
    write_tables(a.out, rows, fits, entropy)
    plot(a.out, rows, fits)
    print(json.dumps(fits, indent=1))
    return {"fits": fits, "rows": rows, "source_entropy_nats": entropy}


if __name__ == "__main__":
    main()
