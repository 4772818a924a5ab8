"""IsoFLOP (Chinchilla-style) grid over ``from_dims`` models (flextrain experiments/scaling_law.py:1-70): for each
compute budget, train a ladder of widths / depths to that budget with ``python -m flextrain_b200 pretrain`` and fit
``L(N) = c0 * (log N)^2 + c1 * log N + c2`` per budget; the vertex is the compute-optimal size.

    python experiments/scaling_law.py --train-shards 'data/fineweb_train_*.bin' --val-shards 'data/fineweb_val_*.bin' \
        --budgets 1e17,3e17,1e18 --out runs/scaling_law

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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--train-shards", default=None)
    ap.add_argument("--val-shards", default=None)
    ap.add_argument("--synthetic-corpus", type=int, default=0, metavar="TOKENS",
                    help="write a Markov-source corpus of this many training tokens and use it")
    ap.add_argument("--vocab-size", type=int, default=None, help="default 50304, or 4096 with --synthetic-corpus")
    ap.add_argument("--budgets", default="1e17,3e17,1e18")
    ap.add_argument("--ladder", default=None, help="'d:L,d:L,...' replacing the default width / depth ladder")
    ap.add_argument("--out", default="runs/scaling_law")
    ap.add_argument("--batch-tokens", type=int, default=131072)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--peak-lr", type=float, default=None)
    ap.add_argument("--device", default=None)
    ap.add_argument("--eval-tokens", type=int, default=None)
    a = ap.parse_args(argv)
    os.makedirs(a.out, exist_ok=True)
    vocab = a.vocab_size or (4096 if a.synthetic_corpus else 50304)
    ladder = [tuple(int(v) for v in p.split(":")) for p in a.ladder.split(",")] if a.ladder else LADDER
    entropy = None
    if a.synthetic_corpus:
        a.train_shards, a.val_shards, entropy = write_synthetic_corpus(os.path.join(a.out, "corpus"), a.synthetic_corpus,
                                                                       vocab)
    if not a.train_shards or not a.val_shards:
        ap.error("give --train-shards and --val-shards, or --synthetic-corpus")
    fits, rows = {}, []
    for b in [float(x) for x in a.budgets.split(",")]:
        pts = []
        for d, L in ladder:
            run = os.path.join(a.out, f"F{b:.0e}_d{d}_L{L}")
            os.makedirs(run, exist_ok=True)
            dj = os.path.join(run, "dims.json")
            json.dump(dims_for(d, L, vocab), open(dj, "w"))
            cmd = [sys.executable, "-m", "flextrain_b200", "pretrain", "--dims", dj, "--train-shards", a.train_shards,
                   "--val-shards", a.val_shards, "--out", run, "--flop-budget", str(b), "--batch-tokens",
                   str(a.batch_tokens), "--max-seq-len", str(a.seq_len)]
            if a.peak_lr:
                cmd += ["--peak-lr", str(a.peak_lr)]
            if a.device:
                cmd += ["--device", a.device]
            if a.eval_tokens:
                cmd += ["--eval-tokens", str(a.eval_tokens)]
            subprocess.run(cmd, cwd=ROOT, check=False)
            fj = os.path.join(run, "final.json")
            if os.path.exists(fj):
                fin, meta = json.load(open(fj)), json.load(open(os.path.join(run, "meta.json")))
                if fin.get("val_loss") is not None:
                    pts.append((meta["n_params"], fin["val_loss"]))
                    rows.append({"budget": b, "d_model": d, "n_layers": L, "n_params": meta["n_params"],
                                 "val_loss": fin["val_loss"], "steps": fin.get("steps"), "tokens": fin.get("tokens")})
        if len(pts) >= 3:
            fits[f"{b:.0e}"] = fit_parabola(*zip(*pts))
    result = {"fits": fits, "rows": rows, "source_entropy_nats": entropy}
    json.dump(result, open(os.path.join(a.out, "fit.json"), "w"), indent=1)
    with open(os.path.join(a.out, "table.md"), "w") as f:
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
    print(json.dumps(fits, indent=1))
    return result


if __name__ == "__main__":
    main()
