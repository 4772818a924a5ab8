"""Stage models and datasets ahead of a run:  python download.py --model <hf id> [--dataset <spec> --out data.jsonl]"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from flextrain_b200.io.download import materialize_sft_dataset, maybe_download_hf_snapshot  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--models-dir", default=os.environ.get("FLEXTRAIN_MODELS_DIR", "models"))
    ap.add_argument("--dataset", default=None)
    ap.add_argument("--out", default="datasets/sft.jsonl")
    ap.add_argument("--limit", type=int, default=None)
    a = ap.parse_args()
    if a.model:
        print(maybe_download_hf_snapshot(a.model, a.models_dir))
    if a.dataset:
        print(materialize_sft_dataset(a.dataset, a.out, a.limit))
