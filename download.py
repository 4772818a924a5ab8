"""Stage models and datasets ahead of a run, on a machine that has network access:

    python download.py model meta-llama/Llama-3.1-8B --target models/Llama-3.1-8B [--revision R] [--force]
    python download.py dataset HuggingFaceH4/no_robots --target datasets/no_robots.jsonl [--split train] [--config C]

then point ``train.py --model`` / ``--dataset`` at the targets on the (possibly air-gapped) training machine.
The older spelling ``python download.py --model <id> [--dataset <spec> --out data.jsonl]`` still works.

This script does not import the package (no torch, no CUDA needed on a login node): it loads
``flextrain_b200/io/download.py`` by path."""
import argparse
import importlib.util
import os
import sys


def _load():
    here = os.path.dirname(os.path.abspath(__file__))
    src = os.path.join(here, "flextrain_b200", "io", "download.py")
    spec = importlib.util.spec_from_file_location("flextrain_b200_download_standalone", src,
                                                  submodule_search_locations=None)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    dl = _load()
    if argv and argv[0] in ("model", "dataset"):
        ap = argparse.ArgumentParser(prog="download.py")
        sub = ap.add_subparsers(dest="kind", required=True)
        m = sub.add_parser("model", help="mirror an HF model repository into a local directory")
        m.add_argument("repo_id")
        m.add_argument("--target", required=True)
        m.add_argument("--revision", default=None)
        m.add_argument("--allow-patterns", nargs="+", default=None)
        m.add_argument("--force", action="store_true")
        d = sub.add_parser("dataset", help="write an SFT dataset as normalised JSONL")
        d.add_argument("spec", help="HF dataset id, or a local JSON / JSONL file")
        d.add_argument("--target", required=True)
        d.add_argument("--split", default="train")
        d.add_argument("--config", default=None)
        d.add_argument("--limit", type=int, default=None)
        d.add_argument("--force", action="store_true")
        a = ap.parse_args(argv)
        if a.kind == "model":
            print(dl.download_model(a.repo_id, a.target, a.revision, a.allow_patterns, a.force))
        else:
            print(dl.download_dataset(a.spec, a.target, a.split, a.config, a.force, a.limit))
        return 0
    ap = argparse.ArgumentParser(prog="download.py")
    ap.add_argument("--model", default=None)
    ap.add_argument("--models-dir", default=os.environ.get("FLEXTRAIN_MODELS_DIR", "models"))
    ap.add_argument("--dataset", default=None)
    ap.add_argument("--out", default="datasets/sft.jsonl")
    ap.add_argument("--limit", type=int, default=None)
    a = ap.parse_args(argv)
    if a.model:
        print(dl.maybe_download_hf_snapshot(a.model, a.models_dir))
    if a.dataset:
        print(dl.materialize_sft_dataset(a.dataset, a.out, a.limit))
    return 0


if __name__ == "__main__":
    sys.exit(main())
