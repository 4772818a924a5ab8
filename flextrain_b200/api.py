"""Public construction API (flextrain/api.py:72-977): ``from_pretrained``, ``from_dims``,
``register_block_builder``, ``BuildContext``.

``from_pretrained`` reads an HF model directory (``config.json`` + safetensors shards) without
``AutoModel``; ``from_dims`` builds a randomly initialised model from a dims dict.  Both run the
working-set planner against the declared byte budgets and return an :class:`ActiveModel`.
Extra keyword arguments over the reference select the parallel layout on an NVSwitch box:
``world_size / rank / dp_shard / tp / ep`` (defaults: single GPU).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, Mapping, Optional

import torch

from .core.save_level import HardwareCost
from .core.working_set import WorkingSetConfig, determine_working_set_config
from .engine.active_model import ActiveModel
from .io.arch import select_arch_module
from .optim.base import as_engine_optimizer
from .io.arch.common import DTypePolicy, ModelConfig, build_model_parts, config_from_dims, resolve_lora

# ``builder(layer_id, decoder_config, model_config) -> Layer`` (the reference's alias of the same name takes
# ``(layer_id, BuildContext)``, flextrain/api.py:119)
BlockBuilder = Callable[[int, object, object], object]
_BLOCK_BUILDERS: Dict[str, BlockBuilder] = {}


@dataclass
class BuildContext:
    """What a custom block builder receives (flextrain/api.py:72-116)."""
    layer_id: int
    n_layers: int
    model_config: ModelConfig
    dtypes: DTypePolicy
    lora: object = None
    extra: dict = field(default_factory=dict)


def register_block_builder(hf_arch_ids, builder: Callable) -> None:
    """Register ``builder(layer_id, decoder_config, model_config) -> Layer`` for one HF ``architectures`` name or
    several (a string or an iterable of strings).  Registering the same builder again is a no-op; a different builder
    for a name that is taken raises (flextrain/api.py:123-137)."""
    names = [hf_arch_ids] if isinstance(hf_arch_ids, str) else list(hf_arch_ids)
    for name in names:
        have = _BLOCK_BUILDERS.get(name)
        if have is not None and have is not builder:
            raise ValueError(f"a block builder for {name!r} is already registered ({have!r})")
        _BLOCK_BUILDERS[name] = builder


def _hw_cost(hw_cost, device) -> HardwareCost:
    if hw_cost is not None:
        return hw_cost
    if torch.device(device).type == "cuda" and os.environ.get("FLEXTRAIN_SKIP_HW_PROBE", "1") != "1":
        from .core.hw_probe import probe_hardware
        return probe_hardware(device)
    return HardwareCost()


def _dims_of(mc: ModelConfig) -> dict:
    """The model's dimensions under the reference's keys (``am.dims["vocab_size"]`` and so on; ``expert_dim`` is the
    FFN width of a dense model and the per-expert width of a routed one, as in its catalogue)."""
    routed = mc.num_experts > 0
    return {"vocab_size": mc.vocab_size, "n_layers": mc.n_layers, "d_model": mc.d_model, "n_heads": mc.n_heads,
            "n_kv_heads": mc.n_kv_heads, "head_dim": mc.head_dim, "expert_dim": mc.expert_dim if routed else mc.ffn_dim,
            "ffn_dim": mc.ffn_dim, "num_routed_experts": mc.num_experts, "top_k": mc.top_k,
            "num_shared_experts": (1 if mc.shared_dim > 0 else 0) if routed else 1,
            "shared_expert_dim": mc.shared_dim, "is_causal": mc.is_causal}


def _build_active_model(mc: ModelConfig, *, optimizer, max_seq_len, max_global_batch_tokens, max_gpu_mem_bytes,
                        max_host_mem_bytes, device, leeway_gpu_mem_bytes, leeway_host_mem_bytes, dt: DTypePolicy,
                        lora, hw_cost, force_saved_act_level, head_chunk_size, verbose, min_chunk_size,
                        max_chunk_size, ws: Optional[WorkingSetConfig], world_size, rank, dp_shard, tp, ep,
                        opt_state: str = "auto",
                        process_group, model_dir=None, arch_key=None, host_backend=None,
                        plan_only: bool = False) -> ActiveModel:
    optimizer = as_engine_optimizer(optimizer)
    if tp == "auto" or ep == "auto":
        args = dict(locals())
        args.pop("mc")
        tp, ep = choose_layout(mc, args)
    builder = _BLOCK_BUILDERS.get(arch_key) if arch_key else None
    if tp > 1 and ep > 1:
        raise NotImplementedError("tensor and expert parallelism cannot be combined")
    if tp > 1 and type(optimizer).__name__ in ("Muon", "HybridMuonAdamW"):
        raise NotImplementedError("Muon orthogonalises whole weight matrices; a tensor-parallel rank holds a slice of "
                                  "each, and the slice's orthogonalisation is a different update: use AdamW with --tp")
    if (tp > 1 and world_size % tp) or (ep > 1 and world_size % ep):
        raise ValueError(f"world size {world_size} is not a multiple of tp={tp} / ep={ep}")
    embed, layers, head = build_model_parts(mc, dt, lora, head_chunk_size, builder, tp=tp, tp_rank=rank % max(tp, 1))
    if ep > 1:
        # expert parallelism: every rank owns num_experts / ep experts of each MoE layer
        for layer in layers:
            for t in layer.param_spec.tensors:
                if t.shard.ep_dim is not None:
                    t.localize(t.shard.ep_dim, rank % ep, ep)
            if getattr(layer, "moe", None) is not None:
                from .parallel.ep import DEFAULT_CAPACITY_FACTOR
                layer.moe.ep_world, layer.moe.ep_capacity_factor = ep, DEFAULT_CAPACITY_FACTOR
                layer.activation_schema = layer._build_schema()
    hw = _hw_cost(hw_cost, device)
    if ws is None:
        ws = determine_working_set_config(
            layers=layers, embed=embed, head=head, optimizer=optimizer, max_seq_len=max_seq_len,
            max_global_batch_tokens=max_global_batch_tokens, max_gpu_mem_bytes=max_gpu_mem_bytes,
            max_host_mem_bytes=max_host_mem_bytes, leeway_gpu_mem_bytes=leeway_gpu_mem_bytes,
            leeway_host_mem_bytes=leeway_host_mem_bytes, hw=hw, world_size=world_size, tp=tp, ep=ep, shard=dp_shard,
            opt_state=opt_state,
            layers_are_local=True,
            min_chunk_size=min_chunk_size, max_chunk_size=max_chunk_size,
            force_saved_act_level=force_saved_act_level, verbose=verbose)
    ws.resolve_act_slots(layers)          # a hand-built configuration may give the activation ring in bytes only
    if plan_only:
        ws.tp, ws.ep = tp, ep
        return ws
    if getattr(ws, "head_chunk_size", None):
        head.head_chunk_size = min(head.head_chunk_size, ws.head_chunk_size)     # the planner needed the room
    dp = tp_group = ep_group = None
    if world_size > 1:
        from .parallel import build_parallel
        dp, tp_group, ep_group = build_parallel(world_size=world_size, rank=rank, shard=ws.shard, tp=tp, ep=ep,
                                                device=device, process_group=process_group)
    am = ActiveModel(embed=embed, layers=layers, head=head, optimizer=optimizer, ws=ws, device=device, hw_cost=hw,
                     dims=_dims_of(mc), arch=mc.arch, hf_config=mc.hf, force_saved_act_level=force_saved_act_level,
                     verbose=verbose, dp=dp, tp=tp_group, ep=ep_group, model_dir=model_dir, host_backend=host_backend)
    am.model_config = mc
    am.is_causal = mc.is_causal
    am.rank, am.world_size = rank, world_size
    am.tp_degree, am.ep_degree = tp, ep
    mp = tp_group or ep_group
    am.shard_group = getattr(mp, "group_pg", None) if mp is not None else None
    return am


def layout_candidates(mc: ModelConfig, world_size: int, optimizer=None) -> list:
    """``(tp, ep)`` layouts this model can run in on ``world_size`` GPUs, cheapest communication first: data parallel,
    then expert parallel (MoE whose expert count divides), then tensor parallel (head / FFN widths divide, attention
    layers only, element-wise optimizer).  Model-parallel groups span the whole job."""
    out = [(1, 1)]
    if world_size <= 1:
        return out
    if mc.num_experts > 0 and mc.num_experts % world_size == 0:
        out.append((1, world_size))
    muon = type(optimizer).__name__ in ("Muon", "HybridMuonAdamW")
    linear = mc.gdn is not None or any(t == "linear" for t in (mc.layer_types or []))
    if (not muon and not linear and mc.num_experts == 0 and mc.n_heads % world_size == 0
            and mc.n_kv_heads % world_size == 0 and mc.ffn_dim % (world_size * 128) == 0):
        out.append((world_size, 1))
    return out


def choose_layout(mc: ModelConfig, build_args: dict):
    """Plan every candidate layout and return the ``(tp, ep)`` with the lowest estimated step time among those that
    fit the budgets.  Data parallelism wins whenever it fits (no activation traffic between ranks); a model whose
    state does not fit under it (70B-class dense models, large MoE) lands on tensor or expert parallelism."""
    verbose = build_args.get("verbose")
    tried, best = [], None
    for t, e in layout_candidates(mc, build_args["world_size"], build_args.get("optimizer")):
        try:
            ws = _build_active_model(mc, **{**build_args, "tp": t, "ep": e, "plan_only": True, "ws": None,
                                            "verbose": False})
        except (ValueError, NotImplementedError) as err:
            tried.append(f"tp={t} ep={e}: does not fit ({str(err)[:120]})")
            continue
        tried.append(f"tp={t} ep={e}: est {ws.est_step_ms:.0f} ms/step, shard {ws.shard}, "
                     f"{'healthy' if ws.healthy else 'PCIe-exposed'}")
        key = (not ws.healthy, ws.est_step_ms)
        if best is None or key < best[0]:
            best = (key, t, e)
    if verbose:
        for line in tried:
            print(f"[Working Set Log] layout {line}")
    if best is None:
        raise ValueError("no parallel layout fits the budgets: " + "; ".join(tried))
    return best[1], best[2]


def _init_random_weights(am: ActiveModel, seed: int, std: float, on_device: bool = False) -> None:
    """Deterministic init (flextrain/api.py:699-742): names containing ``norm`` → 1, biases → 0, LoRA skipped,
    everything else ``N(0, std)`` drawn in fp32 on a CPU generator in embed → head → layers order."""
    g = torch.Generator().manual_seed(seed)
    dev_gen = None
    if on_device and torch.device(am.device).type == "cuda":
        dev_gen = torch.Generator(device=am.device).manual_seed(seed)
    specs = {}
    for n in am.embed.param_spec.tensors:
        specs[("embed", -1, n.name)] = n
    for n in am.head.param_spec.tensors:
        specs[("head", -1, n.name)] = n
    for l, layer in enumerate(am.layers):
        for n in layer.param_spec.tensors:
            specs[("layer", l, n.name)] = n
    order = {"embed": 0, "head": 1, "layer": 2}
    items = sorted(am.named_master_params(), key=lambda it: (order[it[0]], it[1]))
    for scope, l, name, t in items:
        spec = specs[(scope, l, name)]
        if "_lora_" in name:
            continue
        if spec.init == "ones" or "norm" in name:
            t.fill_(1.0)
        elif spec.init == "zeros" or name.startswith("b_"):
            t.zero_()
        elif dev_gen is not None and t.is_cuda:
            # large models: draw on the GPU (same distribution, different stream of numbers than the CPU generator)
            t.normal_(0.0, std, generator=dev_gen)
        elif spec.is_local_part:
            # same numbers as the unsharded model: draw the whole tensor, keep this rank's part
            dim, a, b = spec.local_slice
            full = torch.randn(spec.global_shape, generator=g, dtype=torch.float32) * std
            t.copy_(full.narrow(dim, a, b - a).to(t.dtype))
        else:
            t.copy_((torch.randn(t.shape, generator=g, dtype=torch.float32) * std).to(t.dtype))
    if am.head.tied:
        am.buffers.head_params()["w_head_proj"].copy_(am.buffers.embed_params()["w_tok_embeddings"])


def _init_lora_params(am: ActiveModel, seed: int, a_std: float) -> None:
    """``A ~ N(0, a_std)``, ``B = 0`` (flextrain/api.py:457-484)."""
    g = torch.Generator().manual_seed(seed)
    for scope, l, name, t in am.named_master_params():
        if name.endswith("_lora_a"):
            spec = am.spec_of(scope, l, name)
            if spec.is_local_part:                             # draw the unsharded tensor, keep this rank's slice
                dim, a, b = spec.local_slice
                full = torch.randn(spec.global_shape, generator=g, dtype=torch.float32) * a_std
                t.copy_(full.narrow(dim, a, b - a).to(t.dtype))
            else:
                t.copy_((torch.randn(t.shape, generator=g, dtype=torch.float32) * a_std).to(t.dtype))
        elif name.endswith("_lora_b"):
            t.zero_()


def from_dims(dims: Mapping, *, arch: str = "llama", optimizer, max_seq_len: int, max_global_batch_tokens: int,
              max_gpu_mem_bytes: int, max_host_mem_bytes: int, hyperparams: Optional[Mapping] = None,
              init_seed: int = 0xF1EC7, init_std: float = 0.02, device: str = "cuda:0",
              leeway_gpu_mem_bytes: int = 3 * (1 << 30), leeway_host_mem_bytes: int = 4 * (1 << 30),
              compute_dtype: torch.dtype = torch.bfloat16, master_dtype: Optional[torch.dtype] = torch.bfloat16,
              grad_dtype: Optional[torch.dtype] = torch.bfloat16, norm_grad_dtype: torch.dtype = torch.float32,
              lora_targets=None, lora_rank: int = 16, lora_alpha: float = 16.0,
              lora_adapter_compute_dtype=torch.bfloat16, lora_adapter_master_dtype=torch.bfloat16,
              lora_adapter_grad_dtype=torch.bfloat16, lora_adapter_opt_state_dtype=torch.bfloat16,
              lora_init_seed: int = 20260424, lora_a_std: float = 0.02, hw_cost: Optional[HardwareCost] = None,
              mem_bw_gbps: Optional[float] = None, fixed_seq_len: bool = False,
              force_saved_act_level: Optional[int] = None, head_chunk_size: int = 4096, verbose: bool = False,
              min_chunk_size: Optional[int] = None, max_chunk_size: Optional[int] = None, moe_backend=None,
              working_set: Optional[WorkingSetConfig] = None, world_size: int = 1, rank: int = 0,
              dp_shard: Optional[str] = None, tp: int = 1, ep: int = 1, process_group=None, host_backend=None,
              opt_state: str = "auto",
              init_weights: bool = True, init_on_device: bool = False, plan_only: bool = False) -> ActiveModel:
    """Build an :class:`ActiveModel` from a dims dict with deterministic random weights; bypasses HF entirely.

    ``plan_only=True`` stops after the working-set planner and returns its :class:`WorkingSetConfig` (nothing is
    allocated, no process group is needed): what the engine WOULD do for this model, budget and parallel layout."""
    mod = select_arch_module(arch)
    hyper = dict(mod.default_hyperparams()) if hasattr(mod, "default_hyperparams") else {}
    hyper.update(hyperparams or {})
    mc = mod.config_from_dims(dims, hyper) if hasattr(mod, "config_from_dims") else config_from_dims(dims, arch, hyper)
    norm_dt = torch.float32 if compute_dtype != torch.float64 else torch.float64
    dt = DTypePolicy(compute_dtype, master_dtype or compute_dtype, grad_dtype or compute_dtype, norm_dt, norm_grad_dtype)
    lora = resolve_lora(lora_targets, lora_rank, lora_alpha, lora_adapter_compute_dtype, lora_adapter_master_dtype,
                        lora_adapter_grad_dtype, lora_adapter_opt_state_dtype)
    am = _build_active_model(mc, optimizer=optimizer, max_seq_len=max_seq_len,
                             max_global_batch_tokens=max_global_batch_tokens, max_gpu_mem_bytes=max_gpu_mem_bytes,
                             max_host_mem_bytes=max_host_mem_bytes, device=device,
                             leeway_gpu_mem_bytes=leeway_gpu_mem_bytes, leeway_host_mem_bytes=leeway_host_mem_bytes,
                             dt=dt, lora=lora, hw_cost=hw_cost, force_saved_act_level=force_saved_act_level,
                             head_chunk_size=head_chunk_size, verbose=verbose, min_chunk_size=min_chunk_size,
                             max_chunk_size=max_chunk_size, ws=working_set, world_size=world_size, rank=rank,
                             dp_shard=dp_shard, tp=tp, ep=ep, opt_state=opt_state, process_group=process_group, arch_key=arch,
                             host_backend=host_backend, plan_only=plan_only)
    if plan_only:
        return am
    am.dims = dict(dims)
    if init_weights:
        _init_random_weights(am, init_seed, init_std, on_device=init_on_device)
    if lora is not None:
        _init_lora_params(am, lora_init_seed, lora_a_std)
    if am.dp is not None:
        am.dp.after_weights_loaded(am)
    return am


def from_pretrained(model_path: str, *, optimizer, max_seq_len: int, max_global_batch_tokens: int,
                    max_gpu_mem_bytes: int, max_host_mem_bytes: int, device: str = "cuda:0",
                    leeway_gpu_mem_bytes: int = 3 * (1 << 30), leeway_host_mem_bytes: int = 4 * (1 << 30),
                    compute_dtype: torch.dtype = torch.bfloat16, master_dtype: Optional[torch.dtype] = torch.bfloat16,
                    grad_dtype: Optional[torch.dtype] = torch.bfloat16, norm_grad_dtype: torch.dtype = torch.float32,
                    lora_targets=None, lora_rank: int = 16, lora_alpha: float = 16.0,
                    lora_adapter_compute_dtype=torch.bfloat16, lora_adapter_master_dtype=torch.bfloat16,
                    lora_adapter_grad_dtype=torch.bfloat16, lora_adapter_opt_state_dtype=torch.bfloat16,
                    lora_init_seed: int = 20260424, lora_a_std: float = 0.02, hw_cost: Optional[HardwareCost] = None,
                    mem_bw_gbps: Optional[float] = None, fixed_seq_len: bool = False,
                    force_saved_act_level: Optional[int] = None, head_chunk_size: int = 4096,
                    load_weights: bool = True, strict: bool = False, verbose: bool = False,
                    min_chunk_size: Optional[int] = None, max_chunk_size: Optional[int] = None, moe_backend=None,
                    enable_multimodal="auto", freeze_modality_encoders: bool = True,
                    working_set: Optional[WorkingSetConfig] = None, world_size: int = 1, rank: int = 0,
                    dp_shard: Optional[str] = None, tp: int = 1, ep: int = 1, process_group=None,
                    opt_state: str = "auto",
                    host_backend=None) -> ActiveModel:
    """Build a configured :class:`ActiveModel` for an HF model directory and load its safetensors weights."""
    with open(os.path.join(model_path, "config.json")) as f:
        hf = json.load(f)
    archs = hf.get("architectures") or [hf.get("model_type", "llama")]
    mod = select_arch_module(archs[0], hf.get("model_type"))
    mc = mod.config_from_hf(hf)
    mc.hf = hf
    norm_dt = torch.float32
    dt = DTypePolicy(compute_dtype, master_dtype or compute_dtype, grad_dtype or compute_dtype, norm_dt, norm_grad_dtype)
    lora = resolve_lora(lora_targets, lora_rank, lora_alpha, lora_adapter_compute_dtype, lora_adapter_master_dtype,
                        lora_adapter_grad_dtype, lora_adapter_opt_state_dtype)
    am = _build_active_model(mc, optimizer=optimizer, max_seq_len=max_seq_len,
                             max_global_batch_tokens=max_global_batch_tokens, max_gpu_mem_bytes=max_gpu_mem_bytes,
                             max_host_mem_bytes=max_host_mem_bytes, device=device,
                             leeway_gpu_mem_bytes=leeway_gpu_mem_bytes, leeway_host_mem_bytes=leeway_host_mem_bytes,
                             dt=dt, lora=lora, hw_cost=hw_cost, force_saved_act_level=force_saved_act_level,
                             head_chunk_size=head_chunk_size, verbose=verbose, min_chunk_size=min_chunk_size,
                             max_chunk_size=max_chunk_size, ws=working_set, world_size=world_size, rank=rank,
                             dp_shard=dp_shard, tp=tp, ep=ep, opt_state=opt_state, process_group=process_group, model_dir=model_path,
                             arch_key=archs[0], host_backend=host_backend)
    if enable_multimodal not in (False, None) and ("vision_config" in hf):
        from .nn.multimodal_input import attach_multimodal_input
        attach_multimodal_input(am, hf, model_path, freeze=freeze_modality_encoders,
                                required=(enable_multimodal is True))
    if load_weights:
        am.load_hf(model_path, strict=strict)
    else:
        _init_random_weights(am, 0xF1EC7, 0.02)
    if lora is not None:
        _init_lora_params(am, lora_init_seed, lora_a_std)
    if am.dp is not None:
        am.dp.after_weights_loaded(am)
    return am
