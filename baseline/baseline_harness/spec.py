"""Run description shared by every backend of the comparison harness.

A :class:`RunSpec` says WHAT to train (model directory or dims preset, sequence length, batch shape, steps, GPUs);
a backend (``backends.py``) turns it into the command line of one trainer.  Specs come from the command line of
``run_baseline.py`` or from the ``[common]`` + ``[<backend>]`` sections of a sweep TOML
(reference: baseline/baseline_harness/spec.py, baseline/scripts/sweep.py).
"""
from __future__ import annotations

import dataclasses
import os
import re
import subprocess
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional

_TEMPLATE = re.compile(r"\$\{([A-Z_]+)\}")


@dataclass
class RunSpec:
    backend: str
    model_path: Optional[str] = None          # HF directory; None = random init from ``model_preset``
    model_preset: str = "llama3_1_8B"         # key of flextrain_b200/configs/model_dims.json
    seq_length: int = 1024
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    num_steps: int = 3
    warmup_steps: int = 1
    num_gpus: int = 1
    dtype: str = "bf16"
    seed: int = 1234
    output_dir: str = "baseline/runs"
    run_name: Optional[str] = None
    master_port: int = 29531
    extra: Dict[str, Any] = field(default_factory=dict)     # backend-specific knobs from the TOML section

    @property
    def tokens_per_step(self) -> int:
        return self.seq_length * self.micro_batch_size * self.gradient_accumulation_steps * self.num_gpus

    @property
    def name(self) -> str:
        return self.run_name or f"{self.backend}_{self.model_preset}_s{self.seq_length}_g{self.num_gpus}"

    @property
    def run_dir(self) -> str:
        return os.path.join(self.output_dir, self.name)

    def validate(self) -> None:
        for k in ("seq_length", "micro_batch_size", "gradient_accumulation_steps", "num_steps", "num_gpus"):
            if int(getattr(self, k)) < 1:
                raise ValueError(f"{k} must be >= 1, got {getattr(self, k)}")
        if self.dtype not in ("bf16", "fp16", "fp32"):
            raise ValueError(f"unknown dtype {self.dtype!r}")
        if self.model_path is not None and not os.path.isdir(self.model_path):
            raise FileNotFoundError(f"model_path {self.model_path!r} is not a directory")


def detect_num_gpus() -> int:
    """GPUs visible to ``nvidia-smi -L`` (0 when there is no driver)."""
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=20).stdout
        return sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except Exception:
        return 0


def substitute(value: Any, variables: Mapping[str, Any]) -> Any:
    """Replace ``${NAME}`` in strings (recursively through lists / dicts); a string that is exactly one
    placeholder of an int variable becomes an int."""
    if isinstance(value, str):
        m = _TEMPLATE.fullmatch(value)
        if m and m.group(1) in variables:
            return variables[m.group(1)]
        return _TEMPLATE.sub(lambda mm: str(variables.get(mm.group(1), mm.group(0))), value)
    if isinstance(value, list):
        return [substitute(v, variables) for v in value]
    if isinstance(value, dict):
        return {k: substitute(v, variables) for k, v in value.items()}
    return value


_SPEC_FIELDS = {f.name for f in dataclasses.fields(RunSpec)} - {"extra", "backend"}


def spec_from_sections(backend: str, common: Mapping[str, Any], section: Mapping[str, Any],
                       overrides: Optional[Mapping[str, Any]] = None, num_gpus: Optional[int] = None) -> RunSpec:
    """Merge ``[common]``, the backend's own section and command-line overrides into a spec; keys that are not
    spec fields land in ``extra`` for the backend to interpret."""
    merged: Dict[str, Any] = {**common, **section, **(overrides or {})}
    n = int(num_gpus or merged.get("num_gpus") or detect_num_gpus() or 1)
    merged["num_gpus"] = n
    merged = substitute(merged, {"NUM_GPUS": n})
    known = {k: v for k, v in merged.items() if k in _SPEC_FIELDS}
    extra = {k: v for k, v in merged.items() if k not in _SPEC_FIELDS and k != "backend"}
    spec = RunSpec(backend=backend, extra=extra, **known)
    spec.validate()
    return spec


def load_sweep(path: str) -> Dict[str, Dict[str, Any]]:
    """Parse a sweep TOML: returns ``{"common": {...}, "<backend>": {...}, ...}`` in file order."""
    import tomllib
    with open(path, "rb") as f:
        data = tomllib.load(f)
    if "common" not in data:
        raise ValueError(f"{path}: a sweep needs a [common] section")
    return data
