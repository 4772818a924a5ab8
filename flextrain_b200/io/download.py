"""Pre-staging of HF model snapshots and SFT datasets (flextrain/io/download.py:40-304).

Network access is optional: every function first looks for a local copy and raises a clear error when the
artifact is absent and cannot be fetched (air-gapped machines stage ``models/`` and ``datasets/`` by hand)."""
from __future__ import annotations

import json
import os
from typing import Iterable, Optional

from .sources import normalise_sft_record


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


def materialize_sft_dataset(spec: str, out_path: str, limit: Optional[int] = None) -> str:
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
        records = datasets.load_dataset(name, split=split or "train")
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
