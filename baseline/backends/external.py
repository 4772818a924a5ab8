"""Entry point for the third-party trainers the comparison harness knows about (TRL + DeepSpeed, TRL + FSDP2,
DeepSpeed-Arctic with Ulysses sequence parallelism, MegaTrain, TorchTitan, Megatron-Core).

None of these frameworks ships with this repository or its image.  The harness builds their command lines and gates
them on importability (``Backend.available``); when a sweep is run where one of them IS installed, this script hands
over to the framework's own synthetic-data launcher module, named by ``BASELINE_EXTERNAL_ENTRY`` (for example
``BASELINE_EXTERNAL_ENTRY=my_site.trl_deepspeed_synthetic``), with the harness arguments unchanged.  Without such a
module it explains what is missing and exits with status 3 so the sweep records the backend as skipped
(reference: baseline/backends/*/train_synthetic.py in the reference tree are such launchers).
"""
from __future__ import annotations

import importlib
import os
import sys


def main() -> int:
    entry = os.environ.get("BASELINE_EXTERNAL_ENTRY")
    if not entry:
        print("[baseline] no launcher module configured for this third-party backend "
              "(set BASELINE_EXTERNAL_ENTRY=<module with main(argv)>); skipping", file=sys.stderr)
        return 3
    try:
        mod = importlib.import_module(entry)
    except ImportError as e:
        print(f"[baseline] cannot import {entry}: {e}; skipping", file=sys.stderr)
        return 3
    return int(mod.main(sys.argv[1:]) or 0)


if __name__ == "__main__":
    sys.exit(main())
