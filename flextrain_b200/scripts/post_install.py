"""Post-install step (flextrain/scripts/post_install.py:1-28).

The reference uses this hook to download prebuilt flash-attn and causal-conv1d wheels.  This package carries its
own attention and convolution kernels, so the hook only builds the in-tree native libraries and reports what it
found; nothing is fetched from the network."""
from __future__ import annotations


def main() -> int:
    from ..build import build_all
    built = build_all()
    for name, path in sorted(built.items()):
        print(f"[post-install] {name}: {path}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
