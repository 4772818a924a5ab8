"""Run configuration dataclasses for ``python -m flextrain_b200 train <yaml>`` (flextrain/config.py:29-183).

Unlike the reference, ``IOConfig.resume_from`` is consumed: it names an HF directory written by a previous run
(``save_hf_full``) whose weights are loaded before training starts (weights-only resume, as in the reference's
documented workflow)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class ModelConfig:
    path: Optional[str] = None            # HF directory
    dims: Optional[str] = None            # or a name from configs/model_dims.json
    arch: str = "llama"
    mode: str = "full"                    # "full" | "lora"
    lora_rank: int = 16
    lora_alpha: float = 16.0


@dataclass(frozen=True)
class OptimizerConfig:
    name: str = "adamw"                   # "adamw" | "muon"
    lr: float = 3e-5
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.0
    state_dtype: str = "bfloat16"
    warmup_pct: float = 0.1
    cooldown_start_pct: float = 0.8
    final_pct: float = 0.1
    max_grad_norm: Optional[float] = None  # clip the global gradient norm before every update


@dataclass(frozen=True)
class TrainConfig:
    steps: int = 20
    max_seq_len: int = 2048
    max_global_batch_tokens: int = 65536
    seed: int = 0
    force_save_level: Optional[int] = None
    min_chunk_size: Optional[int] = None
    max_chunk_size: Optional[int] = None


@dataclass(frozen=True)
class HardwareConfig:
    max_gpu_mem_gib: Optional[float] = None
    max_host_mem_gib: Optional[float] = None
    leeway_gpu_mem_gib: float = 5.0
    leeway_host_mem_gib: float = 10.0
    dp_shard: Optional[str] = None
    tp: int = 1
    ep: int = 1
    attn_backend: str = "auto"


@dataclass(frozen=True)
class DataConfig:
    source: str = "synthetic"             # "synthetic" | "json_sft" | "shards" | "mm_json"
    path: Optional[str] = None
    eval_path: Optional[str] = None       # validation file(s) of the same kind
    synthetic_seq_len: Optional[int] = None
    apply_chat_template: bool = False
    truncate_long: bool = False


@dataclass(frozen=True)
class IOConfig:
    output_dir: str = "runs/default"
    save: bool = False
    resume_from: Optional[str] = None          # weights only: an exported HF directory becomes the model to load
    log_every: int = 1
    eval_every: int = 0                        # validation loss every N steps (needs data.eval_path unless synthetic)
    eval_tokens: int = 65536
    save_state_every: int = 0                  # full training state (weights, optimizer state, step) every N steps
    resume_state: Optional[str] = None         # continue exactly from a directory written by save_state_every


@dataclass(frozen=True)
class RunConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    train: TrainConfig = field(default_factory=TrainConfig)
    hardware: HardwareConfig = field(default_factory=HardwareConfig)
    data: DataConfig = field(default_factory=DataConfig)
    io: IOConfig = field(default_factory=IOConfig)

    @staticmethod
    def from_dict(d: dict) -> "RunConfig":
        mk = lambda cls, key: cls(**{k: v for k, v in (d.get(key) or {}).items() if k in cls.__dataclass_fields__})
        return RunConfig(mk(ModelConfig, "model"), mk(OptimizerConfig, "optimizer"), mk(TrainConfig, "train"),
                         mk(HardwareConfig, "hardware"), mk(DataConfig, "data"), mk(IOConfig, "io"))

    @staticmethod
    def from_yaml(path: str) -> "RunConfig":
        import yaml
        with open(path) as f:
            return RunConfig.from_dict(yaml.safe_load(f) or {})
