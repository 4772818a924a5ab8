"""Pre-staging of HF model snapshots and SFT datasets (flextrain/io/download.py:40-304).

Network access is optional: every function first looks for a local copy and raises a clear error when the
artifact is absent and cannot be fetched (air-gapped machines stage ``models/`` and ``datasets/`` by hand)."""
from __future__ import annotations

import json
import os
import sys
from typing import Iterable, Optional

DEFAULT_PATTERNS = ["*.json", "*.safetensors", "*.model", "*.txt", "*.jinja", "*.tiktoken"]


def _looks_complete(target: str) -> bool:
    """A model directory is usable when it has a config and every shard its index (if any) names."""
    if not os.path.exists(os.path.join(target, "config.json")):
        return False
    idx = os.path.join(target, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            shards = set(json.load(f).get("weight_map", {}).values())
        return all(os.path.exists(os.path.join(target, s)) for s in shards)
    return any(n.endswith(".safetensors") for n in os.listdir(target))


def hf_checkpoint_is_complete(local_path) -> bool:
    """True when ``local_path`` holds ``config.json`` and every weight file it needs (one ``model.safetensors`` or all
    shards of the index), so an interrupted download is not mistaken for a model (flextrain/io/download.py:40-68)."""
    return os.path.isdir(str(local_path)) and _looks_complete(str(local_path))


def download_model(repo_id: str, target: Optional[str] = None, revision: Optional[str] = None,
                   allow_patterns: Optional[Iterable[str]] = None, force: bool = False, *,
                   target_dir: Optional[str] = None, verbose: bool = True) -> str:
    """Mirror an HF model repository into ``target`` (explicit path, created if needed; ``target_dir`` is the
    reference's name for it).  A target that already looks complete is left alone unless ``force``."""
    target = str(target if target is not None else target_dir)
    if not force and os.path.isdir(target) and _looks_complete(target):
        if verbose:
            print(f"[download] {target} is complete; nothing to do", file=sys.stderr)
        return target
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:
        raise FileNotFoundError(f"{target} is incomplete and huggingface_hub is not installed") from e
    os.makedirs(target, exist_ok=True)
    try:
        snapshot_download(repo_id, local_dir=target, revision=revision,
                          allow_patterns=list(allow_patterns) if allow_patterns else DEFAULT_PATTERNS)
    except Exception as e:
        raise FileNotFoundError(f"could not download {repo_id!r} (offline?): {e}") from e
    return target


def download_dataset(spec: Optional[str] = None, target: Optional[str] = None, split: str = "train",
                     config: Optional[str] = None, force: bool = False, limit: Optional[int] = None, *,
                     dataset_spec: Optional[str] = None, target_path: Optional[str] = None, verbose: bool = True) -> str:
    """Write an SFT dataset (local JSON / JSONL file, or HF dataset id) as normalised JSONL at ``target``
    (``dataset_spec`` / ``target_path`` are the reference's names for the two arguments)."""
    spec = spec if spec is not None else dataset_spec
    target = str(target if target is not None else target_path)
    if not force and os.path.exists(target) and os.path.getsize(target) > 0:
        if verbose:
            print(f"[download] {target} exists; nothing to do", file=sys.stderr)
        return target
    if force and os.path.exists(target):
        os.remove(target)
    return materialize_sft_dataset(spec if os.path.exists(spec) or ":" in spec else f"{spec}:{split}", target, limit,
                                   config=config)


def normalise_sft_record(rec: dict) -> Optional[dict]:
    """Accepts ``instruction/output``, ``prompt/completion``, ``question/answer`` or chat ``messages``."""
    for a, b, extra in (("instruction", "output", "input"), ("prompt", "completion", "input"),
                        ("prompt", "response", "input"), ("question", "answer", "context"),
                        ("query", "response", "context"), ("input", "output", None), ("instruction", "response", "input")):
        if a in rec and b in rec:
            ins = rec[a]
            if extra and extra != a and rec.get(extra):
                ins = f"{ins}\n{rec[extra]}"
            return {"instruction": str(ins), "response": str(rec[b])}
    msgs = rec.get("messages") or rec.get("conversations")
    if msgs:
        user = [m for m in msgs if m.get("role", m.get("from")) in ("user", "human")]
        asst = [m for m in msgs if m.get("role", m.get("from")) in ("assistant", "gpt")]
        if user and asst:
            return {"instruction": str(user[0].get("content", user[0].get("value", ""))),
                    "response": str(asst[0].get("content", asst[0].get("value", ""))), "messages": msgs}
    return None


normalize_sft_record = normalise_sft_record          # the reference's spelling


def maybe_download_hf_snapshot(repo_id: str, models_dir: str = "models") -> str:
    """Return a local directory for ``repo_id``; downloads with ``huggingface_hub`` when it is not there."""
    local = os.path.join(models_dir, repo_id.split("/")[-1])
    if os.path.isdir(local) and os.path.exists(os.path.join(local, "config.json")):
        return local
    try:
        from huggingface_hub import snapshot_download
    except ImportError as e:
        raise FileNotFoundError(f"{local} does not exist and huggingface_hub is not installed") from e
    os.makedirs(models_dir, exist_ok=True)
    try:
        return snapshot_download(repo_id, local_dir=local,
                                 allow_patterns=["*.json", "*.safetensors", "*.model", "*.txt", "*.jinja"])
    except Exception as e:
        raise FileNotFoundError(f"could not download {repo_id!r} (offline?): {e}") from e


def materialize_sft_dataset(spec: str, out_path: str, limit: Optional[int] = None, config: Optional[str] = None) -> str:
    """Normalise a dataset to JSONL records ``{"instruction", "response"}``.

    ``spec`` is a local JSON / JSONL file or an HF dataset id (``name`` or ``name:split``).  Accepted schemas:
    ``instruction/output``, ``prompt/completion``, ``question/answer`` and chat ``messages``."""
    if os.path.exists(out_path):
        return out_path
    records: Iterable[dict]
    if os.path.exists(spec):
        with open(spec) as f:
            txt = f.read().strip()
        records = json.loads(txt) if txt.startswith("[") else [json.loads(l) for l in txt.splitlines() if l.strip()]
    else:
        try:
            import datasets
        except ImportError as e:
            raise FileNotFoundError(f"{spec!r} is not a file and the `datasets` package is not installed") from e
        name, _, split = spec.partition(":")
        records = datasets.load_dataset(name, config, split=split or "train")
    os.makedirs(os.path.dirname(out_path) or ".", exist_ok=True)
    n = 0
    with open(out_path, "w") as f:
        for rec in records:
            r = normalise_sft_record(dict(rec))
            if r is None:
                continue
            f.write(json.dumps({"instruction": r["instruction"], "response": r["response"]}) + "\n")
            n += 1
            if limit and n >= limit:
                break
    return out_path
