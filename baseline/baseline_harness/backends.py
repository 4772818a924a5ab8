"""Backend registry of the comparison harness: spec -> command line (+ environment) of one trainer.

In-repo backends (always runnable on a GPU box with this image):

* ``flextrain_b200``  this framework through ``train.py`` (peer-memory kernels, tcgen05 GEMMs);
* ``nccl_library``    this framework's engine with library collectives and library GEMM / attention
                      (``FTB_DP_BACKEND=collective FTB_GEMM_BACKEND=library``): the "NCCL + cuBLAS" baseline;
* ``reference``       the unmodified reference engine installed under ``baseline/_ref`` (``bench.py --impl reference``);
* ``hf_fsdp2``        HuggingFace ``transformers`` model + PyTorch FSDP2 (``baseline/backends/hf_fsdp2.py``).
* ``torchtitan``      TorchTitan's Llama-3 model, FSDP2 and activation checkpointing (``baseline/backends/torchtitan_synthetic.py``).

Third-party backends the reference project compares against (baseline/baseline_harness/backends.py in its tree):
``trl_deepspeed``, ``trl_fsdp``, ``deepspeed_arctic``, ``megatrain``, ``megatron``.  Their command
lines are built the same way; a backend whose Python package is not importable reports ``available() == False`` and
a sweep records it as skipped instead of failing.
"""
from __future__ import annotations

import importlib.util
import os
import shlex
import sys
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

from .spec import RunSpec

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@dataclass
class Backend:
    name: str
    describe: str
    requires: Tuple[str, ...]                         # importable modules the trainer needs
    build: Callable[[RunSpec], Tuple[List[str], Dict[str, str]]]

    def available(self) -> Tuple[bool, str]:
        missing = [m for m in self.requires if importlib.util.find_spec(m) is None]
        return (not missing, "" if not missing else "not installed: " + ", ".join(missing))

    def command(self, spec: RunSpec) -> Tuple[List[str], Dict[str, str]]:
        cmd, env = self.build(spec)
        cmd = list(cmd) + [str(a) for a in spec.extra.get("backend_extra_args", [])]     # raw pass-through arguments
        env = {"PYTHONPATH": REPO_ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), **env}
        return cmd, env


def _torchrun(spec: RunSpec, script: str, args: List[str]) -> List[str]:
    if spec.num_gpus == 1:
        return [sys.executable, script, *args]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={spec.num_gpus}",
            "--master-addr", "127.0.0.1", "--master-port", str(spec.master_port), script, *args]


def _flag_args(extra: Dict[str, object], allowed: Tuple[str, ...]) -> List[str]:
    out: List[str] = []
    for k in allowed:
        if k not in extra:
            continue
        v, flag = extra[k], "--" + k.replace("_", "-")
        if isinstance(v, bool):
            if v:
                out.append(flag)
        else:
            out += [flag, str(v)]
    return out


# ----------------------------------------------------------------------------------------------- in-repo backends
def _ours(spec: RunSpec, env_extra: Optional[Dict[str, str]] = None):
    args = ["--model", spec.model_path or f"dims:{spec.model_preset}",
            "--mode", "lora" if spec.extra.get("lora") else "full",
            "--data-source", "synthetic", "--synthetic-seq-len", str(spec.seq_length),
            "--max-seq-len", str(spec.seq_length), "--max-global-batch-tokens", str(spec.tokens_per_step),
            "--steps", str(spec.num_steps), "--seed", str(spec.seed)]
    args += _flag_args(spec.extra, ("dp_shard", "tp", "ep", "max_chunk_size", "max_gpu_mem_gib", "max_host_mem_gib",
                                    "use_muon", "force_save_level", "attn_backend"))
    return _torchrun(spec, os.path.join(REPO_ROOT, "train.py"), args), dict(env_extra or {})


def _nccl_library(spec: RunSpec):
    return _ours(spec, {"FTB_DP_BACKEND": "collective", "FTB_GEMM_BACKEND": "library",
                        "FTB_ATTN_BACKEND": "library"})


def _reference(spec: RunSpec):
    args = ["--impl", "reference", "--gpus", str(spec.num_gpus), "--steps", str(spec.num_steps),
            "--warmup", str(max(spec.warmup_steps, 1))]
    return _torchrun(spec, os.path.join(REPO_ROOT, "bench.py"), args), {}


def _hf_fsdp2(spec: RunSpec):
    args = ["--preset", spec.model_preset, "--seq-length", str(spec.seq_length),
            "--micro-batch-size", str(spec.micro_batch_size),
            "--gradient-accumulation-steps", str(spec.gradient_accumulation_steps),
            "--num-steps", str(spec.num_steps), "--warmup-steps", str(spec.warmup_steps), "--seed", str(spec.seed)]
    if spec.model_path:
        args += ["--model-path", spec.model_path]
    args += _flag_args(spec.extra, ("activation_checkpointing", "cpu_offload", "attn_implementation", "n_layers"))
    return _torchrun(spec, os.path.join(REPO_ROOT, "baseline", "backends", "hf_fsdp2.py"), args), {}


def _torchtitan(spec: RunSpec):
    args = ["--preset", spec.model_preset, "--seq-length", str(spec.seq_length),
            "--micro-batch-size", str(spec.micro_batch_size),
            "--gradient-accumulation-steps", str(spec.gradient_accumulation_steps),
            "--num-steps", str(spec.num_steps), "--warmup-steps", str(spec.warmup_steps), "--seed", str(spec.seed)]
    args += _flag_args(spec.extra, ("ac_mode", "cpu_offload", "n_layers"))
    return _torchrun(spec, os.path.join(REPO_ROOT, "baseline", "backends", "torchtitan_synthetic.py"), args), {}


# --------------------------------------------------------------------------------------------- third-party backends
def _external(script_rel: str, allowed: Tuple[str, ...]):
    def build(spec: RunSpec):
        if not spec.model_path:
            raise ValueError("third-party backends train from an HF model directory: set model_path")
        args = ["--model-path", spec.model_path, "--seq-length", str(spec.seq_length),
                "--micro-batch-size", str(spec.micro_batch_size),
                "--gradient-accumulation-steps", str(spec.gradient_accumulation_steps),
                "--num-steps", str(spec.num_steps), "--output-dir", spec.run_dir]
        args += _flag_args(spec.extra, allowed)
        return _torchrun(spec, os.path.join(REPO_ROOT, "baseline", "backends", script_rel), args), {}
    return build


BACKENDS: Dict[str, Backend] = {b.name: b for b in (
    Backend("flextrain_b200", "this framework (train.py)", ("torch",), _ours),
    Backend("nccl_library", "this engine on NCCL collectives + library GEMM/attention", ("torch",), _nccl_library),
    Backend("reference", "unmodified reference engine (bench.py --impl reference)", ("torch",), _reference),
    Backend("hf_fsdp2", "HF transformers + PyTorch FSDP2", ("torch", "transformers"), _hf_fsdp2),
    Backend("trl_deepspeed", "TRL SFTTrainer + DeepSpeed ZeRO", ("trl", "deepspeed"),
            _external("external.py", ("zero_stage", "offload_optimizer", "offload_param", "activation_checkpointing"))),
    Backend("trl_fsdp", "TRL SFTTrainer + accelerate FSDP2", ("trl", "accelerate"),
            _external("external.py", ("fsdp_cpu_offload", "activation_checkpointing"))),
    Backend("deepspeed_arctic", "DeepSpeed + Ulysses sequence parallelism", ("deepspeed", "arctic_training"),
            _external("external.py", ("sequence_parallel_size", "zero_stage", "offload_optimizer", "tiled_mlp"))),
    Backend("megatrain", "MegaTrain CPU-master training", ("megatrain",),
            _external("external.py", ("grad_slab_gib", "activation_checkpointing"))),
    Backend("torchtitan", "TorchTitan Llama-3 model + FSDP2 + activation checkpointing on synthetic tokens",
            ("torch", "torchtitan"), _torchtitan),
    Backend("megatron", "Megatron-Core + TransformerEngine", ("megatron", "transformer_engine"),
            _external("external.py", ("tensor_model_parallel_size", "context_parallel_size", "recompute_granularity",
                                      "optimizer_cpu_offload"))),
)}


def get_backend(name: str) -> Backend:
    if name not in BACKENDS:
        raise KeyError(f"unknown backend {name!r}; known: {', '.join(sorted(BACKENDS))}")
    return BACKENDS[name]


def format_command(cmd: List[str], env: Dict[str, str]) -> str:
    shown = {k: v for k, v in env.items() if k != "PYTHONPATH"}
    prefix = " ".join(f"{k}={shlex.quote(v)}" for k, v in shown.items())
    return (prefix + " " if prefix else "") + " ".join(shlex.quote(c) for c in cmd)
