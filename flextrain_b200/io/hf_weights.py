"""Direct safetensors reader / writer for HF checkpoints (flextrain/io/hf_weights.py:81-530).

No ``AutoModel``: an :class:`ArchSpec` lists, for the embedding, the head and each layer, which
checkpoint tensors feed which engine tensor.  Linear weights need no transpose (both sides are
``(out, in)``).  An entry may combine several checkpoint tensors (MoE expert stacks, bundled
linear-attention projections) through ``combine`` / ``split`` callables, which replaces the
reference's ``post_load_hook`` / ``pre_export_hook`` pair.  Loading is shard-index aware and strict:
every non-optional entry must find at least one of its alternates.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch


@dataclass
class WeightMapEntry:
    name: str                                   # engine tensor name (e.g. "w_q")
    hf_names: Sequence[str]                     # checkpoint names (already formatted with the layer index)
    optional: bool = False
    alternates: Sequence[Sequence[str]] = ()    # other complete name sets that can satisfy this entry
    combine: Optional[Callable[[List[torch.Tensor]], torch.Tensor]] = None
    split: Optional[Callable[[torch.Tensor], List[torch.Tensor]]] = None
    plus_one: bool = False                      # checkpoint stores gamma - 1
    transpose: bool = False


@dataclass
class ArchSpec:
    name: str
    embed: Callable[[object], List[WeightMapEntry]]
    head: Callable[[object], List[WeightMapEntry]]
    layer: Callable[[int, object], List[WeightMapEntry]]
    hf_architectures: Sequence[str] = ()
    # optional: ``export_hook(state, model_config) -> state`` runs on the collected ``{hf_name: tensor}`` dict, for
    # checkpoints that fuse several engine tensors into one (the reference's ``pre_export_hook``)
    export_hook: Optional[Callable[[Dict[str, torch.Tensor], object], Dict[str, torch.Tensor]]] = None


class SafetensorsDir:
    """Index-aware access to the tensors of an HF model directory."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open
        self.dir = model_dir
        self._open = safe_open
        self.where: Dict[str, str] = {}
        idx = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                self.where = dict(json.load(f)["weight_map"])
        else:
            for fn in sorted(os.listdir(model_dir)):
                if fn.endswith(".safetensors") and not fn.startswith("adapter_"):
                    with safe_open(os.path.join(model_dir, fn), framework="pt") as sf:
                        for k in sf.keys():
                            self.where[k] = fn
        self._handles: Dict[str, object] = {}
        self.consumed = set()

    def has(self, name: str) -> bool:
        return name in self.where

    def get(self, name: str) -> torch.Tensor:
        fn = self.where[name]
        if fn not in self._handles:
            self._handles[fn] = self._open(os.path.join(self.dir, fn), framework="pt")
        self.consumed.add(name)
        return self._handles[fn].get_tensor(name)

    def unconsumed(self) -> List[str]:
        return sorted(set(self.where) - self.consumed)


# multimodal wrappers (and text-only saves of families that have one) nest the decoder under another prefix
_NESTED_PREFIXES = ("model.language_model.", "language_model.model.")


def _name_sets(entry: WeightMapEntry):
    sets = [list(entry.hf_names), *[list(a) for a in entry.alternates]]
    yield from sets
    for names in sets:
        if all(n.startswith("model.") for n in names):
            for pre in _NESTED_PREFIXES:
                yield [pre + n[len("model."):] for n in names]


def _resolve(entry: WeightMapEntry, src: SafetensorsDir) -> Optional[List[torch.Tensor]]:
    for names in _name_sets(entry):
        if all(src.has(n) for n in names):
            return [src.get(n) for n in names]
    return None


def _load_entries(entries: List[WeightMapEntry], dst: Dict[str, torch.Tensor], src: SafetensorsDir, where: str,
                  strict: bool, specs=None) -> None:
    for e in entries:
        if e.name not in dst:
            if strict:
                raise KeyError(f"{where}: engine has no tensor {e.name!r}")
            continue
        ts = _resolve(e, src)
        if ts is None:
            if e.optional:
                continue
            raise KeyError(f"{where}: none of {list(e.hf_names)[:3]}... found in checkpoint for {e.name!r}")
        t = e.combine(ts) if e.combine is not None else ts[0]
        if e.transpose:
            t = t.t()
        if e.plus_one:
            t = t.to(torch.float32) + 1.0
        d = dst[e.name]
        ts_spec = specs.get(e.name) if specs is not None else None
        if ts_spec is not None and ts_spec.is_local_part:
            dim, a, b = ts_spec.local_slice          # tensor / expert parallel: keep this rank's part
            t = t.narrow(dim, a, b - a)
        if tuple(t.shape) != tuple(d.shape):
            raise ValueError(f"{where}: shape mismatch for {e.name!r}: checkpoint {tuple(t.shape)} vs engine "
                             f"{tuple(d.shape)}")
        d.copy_(t.to(d.dtype))


def load_hf_into_model(am, model_dir: str, strict: bool = False) -> None:
    """Fill the engine's master tensors from an HF directory (flextrain/engine/active_model.py:700-793)."""
    from .arch import select_arch_module
    mc = am.model_config
    spec: ArchSpec = select_arch_module(mc.arch).ARCH_SPEC
    src = SafetensorsDir(model_dir)
    bm = am.buffers
    by_name = lambda ps: {t.name: t for t in ps.tensors}
    _load_entries(spec.embed(mc), bm.embed_params(), src, "embed", strict, by_name(am.embed.param_spec))
    # which prefix the checkpoint nests its decoder under (multimodal wrappers): the export writes the same names
    am.hf_nested_prefix = None
    for e in spec.embed(mc):
        names = _peek(e, src)
        if names:
            am.hf_nested_prefix = next((pre for pre in _NESTED_PREFIXES if names[0].startswith(pre)), None)
            break
    for i in range(len(am.layers)):
        _load_entries(spec.layer(i, mc), bm.host_params(i), src, f"layer {i}", strict,
                      by_name(am.layers[i].param_spec))
    head_entries = spec.head(mc)
    hp = bm.head_params()
    tied_missing = False
    for e in head_entries:
        if e.name == "w_head_proj" and _peek(e, src) is None:
            tied_missing = True
    _load_entries([e for e in head_entries if not (e.name == "w_head_proj" and tied_missing)], hp, src, "head", strict,
                  by_name(am.head.param_spec))
    if tied_missing or mc.tie_embeddings:
        # tied embeddings: the head arrives empty and mirrors the embedding table (reference FINDING 10)
        hp["w_head_proj"].copy_(bm.embed_params()["w_tok_embeddings"])
        am.head.tied = True
    if strict:
        left = [n for n in src.unconsumed() if "rotary_emb.inv_freq" not in n and not n.startswith("visual.")]
        if left:
            raise KeyError(f"checkpoint tensors not consumed: {left[:8]} ... ({len(left)} total)")


def _peek(entry: WeightMapEntry, src: SafetensorsDir):
    for names in _name_sets(entry):
        if all(src.has(n) for n in names):
            return names
    return None


def checkpoint_names(state: Dict[str, torch.Tensor], nested_prefix: Optional[str]) -> Dict[str, torch.Tensor]:
    """Tensor names as the source checkpoint spells them: ``model.X`` becomes ``<nested_prefix>X`` for a checkpoint
    that nests its decoder (``model.language_model.`` in the vision-language wrappers)."""
    if not nested_prefix:
        return state
    return {(nested_prefix + k[len("model."):] if k.startswith("model.") else k): v for k, v in state.items()}


def passthrough_tensors(source_dir: Optional[str], state: Dict[str, torch.Tensor]) -> int:
    """Add to ``state`` every tensor of the source checkpoint that the engine does not hold (vision tower,
    multi-token-prediction heads, ...), unchanged, so that the exported directory is a complete checkpoint again
    (flextrain/export/_hf_full.py:388-425).  ``lm_head.weight`` is left out when the export did not write one (tied
    embeddings).  Returns how many tensors were added."""
    if not source_dir or not os.path.isdir(source_dir):
        return 0
    try:
        src = SafetensorsDir(source_dir)
    except Exception:
        return 0
    n = 0
    for k in sorted(src.where):
        if k in state or k == "lm_head.weight" or "rotary_emb.inv_freq" in k:
            continue
        state[k] = src.get(k)
        n += 1
    return n


def is_export_writer(am) -> bool:
    """Rank 0 writes export files; the other ranks only take part in gathering tensor- / expert-parallel parts."""
    return int(getattr(am, "rank", 0) or 0) == 0


def collect_hf_state(am, lora_merge: bool = False) -> Dict[str, torch.Tensor]:
    """Engine masters → ``{hf_name: cpu tensor}`` (inverse of the load map).  Under tensor / expert parallelism this is
    a collective: every rank calls it; ranks other than the writer skip the tensors they hold completely and return
    only what they helped to gather."""
    from .arch import select_arch_module
    mc = am.model_config
    spec: ArchSpec = select_arch_module(mc.arch).ARCH_SPEC
    bm = am.buffers
    out: Dict[str, torch.Tensor] = {}
    if getattr(am, "dp", None) is not None and hasattr(am.dp, "finish_param_gather"):
        am.dp.finish_param_gather()         # deferred parameter all-gather: make every rank's copy current first

    writer = is_export_writer(am)

    def emit(entries: List[WeightMapEntry], params: Dict[str, torch.Tensor], specs=None):
        for e in entries:
            if e.name not in params:
                continue
            t = params[e.name].detach()
            ts_spec = specs.get(e.name) if specs is not None else None
            if not writer and not (ts_spec is not None and ts_spec.is_local_part):
                continue
            if lora_merge and (e.name + "_lora_a") in params:
                from ..export._merged import merged_weight
                t = merged_weight(params, e.name, am).to(t.device)      # merged locally, gathered below
            if ts_spec is not None and ts_spec.is_local_part:
                t = gather_local_parts(t, ts_spec, am)     # collective: every rank takes part in the export
            t = t.to("cpu")
            if e.plus_one:
                t = (t.to(torch.float32) - 1.0).to(t.dtype)
            if e.transpose:
                t = t.t()
            parts = e.split(t) if e.split is not None else [t]
            for n, p in zip(e.hf_names, parts):
                out[n] = p.contiguous()

    by_name = lambda ps: {t.name: t for t in ps.tensors}
    emit(spec.embed(mc), bm.embed_params(), by_name(am.embed.param_spec))
    for i in range(len(am.layers)):
        emit(spec.layer(i, mc), bm.host_params(i), by_name(am.layers[i].param_spec))
    head_entries = spec.head(mc)
    if am.head.tied or mc.tie_embeddings:
        head_entries = [e for e in head_entries if e.name != "w_head_proj"]
    emit(head_entries, bm.head_params(), by_name(am.head.param_spec))
    if spec.export_hook is not None and writer:
        out = spec.export_hook(out, mc)
    return out


def gather_local_parts(t: torch.Tensor, spec, am) -> torch.Tensor:
    """Reassemble a tensor- or expert-parallel tensor from the parts held by the ranks of its group."""
    import torch.distributed as dist
    dim, a, b = spec.local_slice
    count = spec.global_shape[dim] // (b - a)
    if count == 1 or not dist.is_initialized():
        return t
    group = getattr(am, "shard_group", None)
    parts = [torch.empty_like(t) for _ in range(count)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


def export_model_safetensors(am, out_dir: str, filename: str = "final.safetensors") -> str:
    """Single-shard export of the tensors the engine holds, in the source checkpoint's names
    (flextrain/io/hf_weights.py:491-530); :func:`flextrain_b200.export.save_hf_full` writes a complete directory."""
    from safetensors.torch import save_file
    os.makedirs(out_dir, exist_ok=True)
    if torch.device(am.device).type == "cuda":
        torch.cuda.synchronize()
    path = os.path.join(out_dir, filename)
    state = checkpoint_names(collect_hf_state(am), getattr(am, "hf_nested_prefix", None))
    encoders = getattr(am.embed, "encoder_export_state", None)
    if encoders is not None:
        state.update(encoders())                    # a vision tower that was trained belongs to the weights
    if is_export_writer(am):
        save_file(state, path, metadata={"format": "pt"})
    return path
