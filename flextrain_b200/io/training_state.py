"""Full training-state checkpoints: master weights + optimizer state + step counter, so that a resumed run continues
bit-for-bit where the saved one stopped.

The reference project resumes from weights only (its exported HF directory becomes the model of the next run,
flextrain/io/hf_weights.py:491-530; optimizer moments restart from zero).  This module adds the rest.  Layout of a
checkpoint directory::

    training_state.json               step, world size, parallel layout, optimizer, per-tensor fingerprint
    state_rank00000.safetensors       what rank 0 holds: every master tensor it owns + its optimizer state
    state_rank00001.safetensors ...   other ranks: only what differs per rank (tensor- / expert-parallel parts, their
                                      optimizer state, this rank's shard of the data-parallel optimizer state)

Every rank calls :func:`save_training_state` / :func:`load_training_state` (they contain barriers when a process group
exists); a checkpoint must be loaded with the world size and layout it was saved with.  Tensors are stored under
``<scope>.<layer>.<name>`` keys (``p.`` masters, ``o.`` optimizer state, ``dp.`` data-parallel shards)."""
from __future__ import annotations

import json
import os
from typing import Dict, Optional

import torch

FORMAT = 1


def _rank_world(am):
    return int(getattr(am, "rank", 0) or 0), int(getattr(am, "world_size", 1) or 1)


def _opt_views(am):
    """Yield ``(scope, layer, {name: tensor})`` of the optimizer state this process holds in its buffer manager."""
    bm = am.buffers
    yield "embed", -1, bm.embed_opt()
    yield "head", -1, bm.head_opt()
    for l in range(len(am.layers)):
        yield "layer", l, bm.master_opt_state(l)


def _local_names(am) -> Dict[tuple, bool]:
    """``(scope, layer, tensor name) -> is this a rank-local part`` for every master tensor."""
    out = {}
    units = [("embed", -1, am.embed.param_spec), ("head", -1, am.head.param_spec)] + \
        [("layer", l, layer.param_spec) for l, layer in enumerate(am.layers)]
    for scope, l, spec in units:
        for t in spec.tensors:
            out[(scope, l, t.name)] = bool(t.is_local_part)
    return out


def _fingerprint(am) -> Dict[str, list]:
    return {f"{s}.{l}.{n}": [list(t.shape), str(t.dtype)] for s, l, n, t in am.named_master_params()}


def _sync(am) -> None:
    if am.device.type == "cuda":
        torch.cuda.synchronize(am.device)
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and _rank_world(am)[1] > 1:
        dist.barrier()


def save_training_state(am, out_dir: str, extra: Optional[dict] = None) -> str:
    """Write this rank's part of the checkpoint; rank 0 also writes ``training_state.json``.  ``extra`` (JSON-able) is
    stored verbatim: data-loader position, learning-rate schedule, anything the caller needs back."""
    from safetensors.torch import save_file
    rank, world = _rank_world(am)
    os.makedirs(out_dir, exist_ok=True)
    dp = getattr(am, "dp", None)
    if dp is not None and hasattr(dp, "finish_param_gather"):
        dp.finish_param_gather()                    # deferred parameter all-gather: make this rank's copy current
    _sync(am)
    local = _local_names(am)
    state: Dict[str, torch.Tensor] = {}
    keep = lambda t: t.detach().to("cpu").contiguous().clone()
    for scope, l, name, t in am.named_master_params():
        if rank == 0 or local[(scope, l, name)]:
            state[f"p.{scope}.{l}.{name}"] = keep(t)
    sharded = dp is not None and getattr(dp, "m", None) is not None       # peer-memory data parallel: fp32 shards
    if sharded:
        state["dp.m"], state["dp.v"] = keep(dp.m), keep(dp.v)
        for key, tensors in getattr(dp, "local_state", {}).items():
            for n, t in tensors.items():
                state[f"dp.local.{key}.{n}"] = keep(t)
        for key, tensors in getattr(dp, "owned_state", {}).items():       # Muon momentum of the tensors this rank owns
            for n, t in tensors.items():
                state[f"dp.owned.{key}.{n}"] = keep(t)
    else:
        owner = {s.key: s.param for _, _, spec in ([("embed", -1, am.embed.param_spec), ("head", -1, am.head.param_spec)]
                                                   + [("layer", l, la.param_spec) for l, la in enumerate(am.layers)])
                 for s in am.optimizer.state_specs(spec)}
        for scope, l, views in _opt_views(am):
            for n, t in views.items():
                if rank == 0 or local.get((scope, l, owner.get(n, "")), False):
                    state[f"o.{scope}.{l}.{n}"] = keep(t)
    if rank == 0 and getattr(am.embed, "train_encoders", False):          # a trainable vision tower: replicated
        state.update({k: keep(v) for k, v in am.embed.encoder_state_dict().items()})
    save_file(state, os.path.join(out_dir, f"state_rank{rank:05d}.safetensors"), metadata={"format": "pt"})
    if rank == 0:
        opt = am.optimizer
        meta = {"format": FORMAT, "step": int(am.step_num), "world_size": world, "arch": am.model_config.arch,
                "tp": am.tp.world if am.tp is not None else 1, "ep": am.ep.world if am.ep is not None else 1,
                "dp_sharded_state": bool(sharded), "optimizer": type(opt).__name__,
                "fingerprint": _fingerprint(am), "extra": extra or {}}
        tmp = os.path.join(out_dir, "training_state.json.tmp")
        with open(tmp, "w") as f:
            json.dump(meta, f, indent=1)
        os.replace(tmp, os.path.join(out_dir, "training_state.json"))      # the JSON appears last: its presence = complete
    _sync(am)
    return out_dir


def load_training_state(am, src_dir: str, strict: bool = True) -> dict:
    """Restore weights, optimizer state and the step counter; returns the stored ``extra`` dict (plus ``step``)."""
    from safetensors import safe_open
    rank, world = _rank_world(am)
    with open(os.path.join(src_dir, "training_state.json")) as f:
        meta = json.load(f)
    if meta.get("format") != FORMAT:
        raise ValueError(f"unknown training-state format {meta.get('format')!r}")
    layout = (world, am.tp.world if am.tp is not None else 1, am.ep.world if am.ep is not None else 1)
    saved = (meta["world_size"], meta["tp"], meta["ep"])
    if layout != saved:
        raise ValueError(f"checkpoint was saved with (world, tp, ep) = {saved}, this job runs {layout}")
    if strict and rank == 0:
        mine = _fingerprint(am)
        bad = [k for k, v in meta["fingerprint"].items() if mine.get(k) != v] + [k for k in mine if k not in meta["fingerprint"]]
        if bad:
            raise ValueError(f"model does not match the checkpoint: {bad[:6]}{' ...' if len(bad) > 6 else ''}")
    _sync(am)
    local = _local_names(am)
    files = {r: os.path.join(src_dir, f"state_rank{r:05d}.safetensors") for r in {0, rank}}
    handles = {r: safe_open(p, framework="pt") for r, p in files.items()}
    keys = {r: set(h.keys()) for r, h in handles.items()}

    def fetch(key: str, is_local: bool):
        r = rank if is_local else 0
        if key not in keys[r]:
            raise KeyError(f"{key} is missing from {files[r]}")
        return handles[r].get_tensor(key)

    for scope, l, name, t in am.named_master_params():
        src = fetch(f"p.{scope}.{l}.{name}", local[(scope, l, name)])
        t.copy_(src.to(t.dtype).reshape(t.shape))
    dp = getattr(am, "dp", None)
    sharded = dp is not None and getattr(dp, "m", None) is not None
    if sharded != bool(meta["dp_sharded_state"]):
        raise ValueError("checkpoint and job disagree on the data-parallel backend (sharded vs replicated optimizer state)")
    if sharded:
        dp.m.copy_(fetch("dp.m", True))
        dp.v.copy_(fetch("dp.v", True))
        for key, tensors in getattr(dp, "local_state", {}).items():
            for n, t in tensors.items():
                t.copy_(fetch(f"dp.local.{key}.{n}", True))
        for key, tensors in getattr(dp, "owned_state", {}).items():
            for n, t in tensors.items():
                t.copy_(fetch(f"dp.owned.{key}.{n}", True))
    else:
        owner = {s.key: s.param for _, _, spec in ([("embed", -1, am.embed.param_spec), ("head", -1, am.head.param_spec)]
                                                   + [("layer", l, la.param_spec) for l, la in enumerate(am.layers)])
                 for s in am.optimizer.state_specs(spec)}
        for scope, l, views in _opt_views(am):
            for n, t in views.items():
                src = fetch(f"o.{scope}.{l}.{n}", local.get((scope, l, owner.get(n, "")), False))
                t.copy_(src.to(t.dtype).reshape(t.shape))
    if getattr(am.embed, "train_encoders", False):
        enc_keys = [k for k in keys[0] if k.startswith("enc.")]
        if strict and not any(k.startswith("enc.master.") for k in enc_keys):
            raise KeyError("the checkpoint has no vision-tower state but the tower is trainable in this job")
        am.embed.load_encoder_state_dict({k: handles[0].get_tensor(k) for k in enc_keys})
    am.step_num = int(meta["step"])
    am._zero_grad = True
    if dp is not None:
        dp.after_weights_loaded(am)                 # re-establish what the group derives from the weights
    for l, layer in enumerate(am.layers):
        if am.buffers.params_resident:
            layer.end_of_step(am.buffers.params(l))  # drop cached effective (LoRA) weights
    _sync(am)
    return {"step": int(meta["step"]), **meta.get("extra", {})}
