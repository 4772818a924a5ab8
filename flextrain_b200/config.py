"""Run configuration dataclasses for ``python -m flextrain_b200 train <yaml>`` (flextrain/config.py:29-183).

Unlike the reference, ``IOConfig.resume_from`` is consumed: it names an HF directory written by a previous run
(``save_hf_full``) whose weights are loaded before training starts (weights-only resume, as in the reference's
documented workflow)."""
from __future__ import annotations

import os
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
    inline_dims: Optional[dict] = None    # or the dimensions themselves (vocab_size, n_layers, d_model, ...)
    hyperparams: Optional[dict] = None    # with inline_dims: rms_norm_eps, rope_theta, rope_scaling, ...


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
    device_id: Optional[int] = None


@dataclass(frozen=True)
class DataConfig:
    source: str = "synthetic"             # "synthetic" | "json_sft" | "shards" | "mm_json" | "hf" | "raw" | "custom"
    path: Optional[str] = None            # file(s) / shard pattern / dataset id of the source
    eval_path: Optional[str] = None       # validation file(s) of the same kind
    synthetic_seq_len: Optional[int] = None
    apply_chat_template: bool = False
    truncate_long: bool = False
    tokenizer: Optional[str] = None       # tokenizer directory / hub id when it is not the model directory
    min_seq_len: int = 0
    hf_subset: Optional[str] = None
    hf_split: str = "train"
    hf_text_field: str = "text"
    hf_streaming: bool = True
    shard_documents: bool = False         # shards: one sequence per document instead of fixed windows
    shard_num_shards: Optional[int] = None
    prompt_field: str = "instruction"
    response_field: str = "output"
    input_field: Optional[str] = "input"
    custom_factory: Optional[str] = None  # "module:callable" returning (records, extract)


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
    def from_dict(d: dict, config_dir: Optional[str] = None) -> "RunConfig":
        if is_reference_schema(d):
            d = translate_reference_schema(d, config_dir)
        sections = {"model": ModelConfig, "optimizer": OptimizerConfig, "train": TrainConfig, "hardware": HardwareConfig,
                    "data": DataConfig, "io": IOConfig}
        unknown = [k for k in d if k not in sections]
        unknown += [f"{sec}.{k}" for sec, cls in sections.items() for k in (d.get(sec) or {})
                    if k not in cls.__dataclass_fields__]
        if unknown:
            raise ValueError(f"run file keys that are not understood: {unknown}")
        mk = lambda cls, key: cls(**{k: v for k, v in (d.get(key) or {}).items() if k in cls.__dataclass_fields__})
        return RunConfig(mk(ModelConfig, "model"), mk(OptimizerConfig, "optimizer"), mk(TrainConfig, "train"),
                         mk(HardwareConfig, "hardware"), mk(DataConfig, "data"), mk(IOConfig, "io"))

    @staticmethod
    def from_yaml(path: str) -> "RunConfig":
        import yaml
        with open(path) as f:
            return RunConfig.from_dict(yaml.safe_load(f) or {}, os.path.dirname(os.path.abspath(path)))


_DIM_KEYS = ("vocab_size", "n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "expert_dim",
             "num_shared_experts", "num_routed_experts", "top_k")


def is_reference_schema(d: dict) -> bool:
    """True for a run file in the reference's layout (flextrain/config.py:29-183): model dimensions written out under
    ``model``, the optimizer nested under ``train``, the data source nested under ``io``."""
    model, train, io = d.get("model") or {}, d.get("train") or {}, d.get("io") or {}
    return ("n_layers" in model or "optimizer" in train or "global_batch_tokens" in train or "total_steps" in train
            or "data" in io or "hf_checkpoint" in io or "save_final_checkpoint" in io)


def translate_reference_schema(d: dict, config_dir: Optional[str] = None) -> dict:
    """A run file in the reference's layout -> this package's layout.  Every key of the reference's dataclasses is
    either mapped or refused by name; nothing is dropped silently."""
    model, train, hw, io = (dict(d.get(k) or {}) for k in ("model", "train", "hardware", "io"))
    data = dict(io.pop("data", None) or {})
    opt = dict(train.pop("optimizer", None) or {})

    def local(p):
        """Paths in a run file may be relative to it."""
        if p and config_dir and not os.path.isabs(p) and os.path.exists(os.path.join(config_dir, p)):
            return os.path.join(config_dir, p)
        return p

    out = {"model": {}, "optimizer": {}, "train": {}, "hardware": {}, "data": {}, "io": {}}
    # ---- model
    m = out["model"]
    m["arch"] = model.pop("arch", "llama")
    dims = {k: model.pop(k) for k in _DIM_KEYS if k in model}
    hyper = {k: model.pop(k) for k in ("rms_norm_eps", "rope_theta", "rope_scaling") if model.get(k) is not None}
    for k in ("rope_scaling",):
        model.pop(k, None)
    causal = model.pop("is_causal", True)
    wl, wr = model.pop("window_size_left", -1), model.pop("window_size_right", 0)
    model.pop("dtypes", None)                    # dtypes follow the device here (bf16 on a GPU, fp32 on CPU)
    if not causal or wr != 0:
        raise ValueError("only causal models are supported (is_causal: true, window_size_right: 0)")
    if wl not in (-1, None):
        hyper["sliding_window"] = int(wl)
    ckpt = io.pop("hf_checkpoint", None) or io.pop("hf_repo_id", None)
    io.pop("hf_repo_id", None)
    if io.pop("hf_revision", None):
        raise ValueError("io.hf_revision is not supported: stage the revision with download.py and name its directory")
    if ckpt:
        m["path"] = local(ckpt)
    elif dims:
        m["inline_dims"], m["hyperparams"] = dims, hyper or None
    for k in ("mode", "lora_rank", "lora_alpha", "path", "dims"):
        if k in model:
            m[k] = model.pop(k)
    # ---- optimizer and schedule
    o = out["optimizer"]
    o["name"] = opt.pop("kind", opt.pop("name", "adamw"))
    for k in ("lr", "beta1", "beta2", "eps", "weight_decay", "state_dtype", "max_grad_norm"):
        if k in opt:
            o[k] = opt.pop(k)
    if "warmup_pct" in train:
        o["warmup_pct"] = train.pop("warmup_pct")
    if "cooldown_pct" in train:
        o["cooldown_start_pct"] = 1.0 - float(train.pop("cooldown_pct"))
    if "final_lr_fraction" in train:
        o["final_pct"] = train.pop("final_lr_fraction")
    # ---- train
    t = out["train"]
    for src, dst in (("global_batch_tokens", "max_global_batch_tokens"), ("total_steps", "steps"),
                     ("max_seq_len", "max_seq_len"), ("seed", "seed"), ("force_save_level", "force_save_level")):
        if src in train:
            t[dst] = train.pop(src)
    train.pop("fixed_seq_len", None)
    # ---- hardware
    h = out["hardware"]
    for k in ("max_gpu_mem_gib", "max_host_mem_gib", "leeway_gpu_mem_gib", "leeway_host_mem_gib", "device_id",
              "dp_shard", "tp", "ep", "attn_backend"):
        if k in hw:
            h[k] = hw.pop(k)
    for k in ("min_chunk_size", "max_chunk_size"):
        if k in hw:
            t[k] = hw.pop(k)
    # ---- io
    i = out["io"]
    if "output_dir" in io:
        i["output_dir"] = io.pop("output_dir")
    if "save_final_checkpoint" in io:
        i["save"] = bool(io.pop("save_final_checkpoint"))
    if io.get("resume_from"):
        i["resume_from"] = local(io.pop("resume_from"))
    io.pop("resume_from", None)
    tok = io.pop("tokenizer", None)
    # ---- data: exactly one source
    dd = out["data"]
    picks = [k for k in ("hf_dataset", "shard_pattern", "synthetic", "raw_path", "json_sft_path", "custom_factory")
             if data.get(k)]
    if len(picks) != 1:
        raise ValueError(f"exactly one data source must be set under io.data, got: {picks}")
    kind = picks[0]
    if kind == "hf_dataset":
        dd.update(source="hf", path=data.pop("hf_dataset"), hf_subset=data.pop("hf_subset", None),
                  hf_split=data.pop("hf_split", "train"), hf_text_field=data.pop("hf_text_field", "text"),
                  hf_streaming=bool(data.pop("hf_streaming", True)))
    elif kind == "shard_pattern":
        dd.update(source="shards", path=data.pop("shard_pattern"), shard_documents=True,
                  shard_num_shards=data.pop("shard_num_shards", None))
    elif kind == "synthetic":
        data.pop("synthetic")
        sl = data.pop("synthetic_seq_len", 512)
        if isinstance(sl, (list, tuple)):
            if len(set(sl)) != 1:
                raise ValueError("synthetic_seq_len: a cycle of lengths is available from the API "
                                 "(SyntheticTokenSource(seq_lens=[...])), the run file takes one length")
            sl = sl[0]
        dd.update(source="synthetic", synthetic_seq_len=int(sl))
    elif kind == "raw_path":
        dd.update(source="raw", path=local(data.pop("raw_path")))
    elif kind == "json_sft_path":
        dd.update(source="json_sft", path=local(data.pop("json_sft_path")),
                  prompt_field=data.pop("json_sft_prompt_field", "instruction"),
                  response_field=data.pop("json_sft_response_field", "output"),
                  input_field=data.pop("json_sft_input_field", "input"))
        data.pop("json_sft_loop", None)          # the training loop decides: it cycles the file for --steps steps
    else:
        dd.update(source="custom", custom_factory=data.pop("custom_factory"))
    for k in ("hf_dataset", "hf_subset", "hf_split", "hf_text_field", "hf_streaming", "shard_pattern", "shard_num_shards",
              "synthetic", "synthetic_seq_len", "raw_path", "json_sft_path", "json_sft_prompt_field",
              "json_sft_response_field", "json_sft_input_field", "json_sft_loop", "custom_factory"):
        data.pop(k, None)                        # defaults written out next to the chosen source
    if "min_seq_len" in data:
        dd["min_seq_len"] = int(data.pop("min_seq_len"))
    if "max_seq_len" in data:
        t.setdefault("max_seq_len", int(data.pop("max_seq_len")))
        data.pop("max_seq_len", None)
    if tok:
        dd["tokenizer"] = local(tok)
    left = {k: v for k, v in (("model", model), ("train.optimizer", opt), ("train", train), ("hardware", hw), ("io", io),
                              ("io.data", data)) if v}
    if left:
        raise ValueError(f"run file keys that are not understood: {left}")
    return out
