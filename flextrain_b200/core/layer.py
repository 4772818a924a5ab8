"""Layer contracts: the only surface the engine consumes.

Covers the reference's ``flextrain/core/layer.py`` (TensorSpec / ParamSpec :72-252, ComputeCost
:261-317, ChunkMeta :325-537, LayerContext :599-676, Layer / InputLayer / OutputLayer protocols
:689-1056, LossStats :1059-1138).  Differences that follow from the B200 design: shapes are
concrete (layers are built from a resolved config), weights are ``(out, in)``, and a
``ShardSpec`` says how a tensor is split across data- / tensor- / expert-parallel ranks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Protocol, Sequence, Tuple, runtime_checkable

import torch

_ITEMSIZE = {torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.int32: 4, torch.int64: 8, torch.uint8: 1,
             torch.float64: 8, torch.int8: 1, torch.bool: 1}


def itemsize(dt: torch.dtype) -> int:
    return _ITEMSIZE[dt]


@dataclass(frozen=True)
class ShardSpec:
    """How one tensor is partitioned over a parallel group.

    ``tp_dim``: dimension split across tensor-parallel ranks (None = replicated);
    ``ep_dim``: dimension split across expert-parallel ranks (the expert axis of MoE weights).
    Data-parallel sharding of gradients / optimizer state is flat (by element range) except for
    tensors whose optimizer needs whole matrices (Muon), which are sharded by matrix.
    """
    tp_dim: Optional[int] = None
    ep_dim: Optional[int] = None
    whole_matrix: bool = False


@dataclass
class TensorSpec:
    """One parameter tensor and the dtype of each of its roles (compute / master / grad / opt state)."""
    name: str
    shape: Tuple[int, ...]
    compute_dtype: torch.dtype = torch.bfloat16
    master_dtype: Optional[torch.dtype] = None
    grad_dtype: Optional[torch.dtype] = None
    opt_state_dtype: Optional[torch.dtype] = None
    optimizer: Optional[str] = None        # explicit "adamw" / "muon" hint; None = rule-based
    frozen: bool = False
    init: str = "normal"                   # "normal" | "ones" | "zeros"
    shard: ShardSpec = field(default_factory=ShardSpec)
    global_shape: Optional[Tuple[int, ...]] = None          # set by localize(): the unsharded shape
    local_slice: Optional[Tuple[int, int, int]] = None      # (dim, start, stop) of this rank's part

    def __post_init__(self):
        self.shape = tuple(int(s) for s in self.shape)
        if self.master_dtype is None:
            self.master_dtype = self.compute_dtype
        if self.grad_dtype is None:
            self.grad_dtype = self.compute_dtype

    @property
    def numel(self) -> int:
        return int(math.prod(self.shape))

    def localize(self, dim: int, index: int, count: int) -> "TensorSpec":
        """Keep only part ``index`` of ``count`` along ``dim`` (tensor- or expert-parallel ownership).  Buffers,
        gradients and optimizer state are then sized for the local part; loaders slice, exporters gather."""
        g = self.global_shape or self.shape
        if g[dim] % count:
            raise ValueError(f"{self.name}: dim {dim} of {g} is not divisible by {count}")
        n = g[dim] // count
        self.global_shape = tuple(g)
        self.local_slice = (dim, index * n, (index + 1) * n)
        self.shape = tuple(g[:dim]) + (n,) + tuple(g[dim + 1:])
        return self

    def mark_local(self, dim: int, index: int, count: int) -> "TensorSpec":
        """Like :meth:`localize` for a spec that was already built with its LOCAL shape (tensor parallelism builds
        the blocks with ``heads / tp`` and ``ffn / tp``): records the global shape and this rank's slice."""
        n = self.shape[dim]
        self.global_shape = tuple(self.shape[:dim]) + (n * count,) + tuple(self.shape[dim + 1:])
        self.local_slice = (dim, index * n, (index + 1) * n)
        return self

    @property
    def is_local_part(self) -> bool:
        return self.local_slice is not None

    @property
    def grad_name(self) -> str:
        """``w_q -> g_q``, ``b_q -> g_b_q`` (flextrain/engine/buffers.py:282-285)."""
        return "g_" + self.name[2:] if self.name.startswith("w_") else "g_" + self.name

    def bytes(self, role: str) -> int:
        if role == "compute":
            return self.numel * itemsize(self.compute_dtype)
        if role == "master":
            return self.numel * itemsize(self.master_dtype)
        if self.frozen:
            return 0
        if role == "grad":
            return self.numel * itemsize(self.grad_dtype)
        raise KeyError(role)


@dataclass
class ParamSpec:
    tensors: List[TensorSpec]

    def __iter__(self):
        return iter(self.tensors)

    def names(self) -> List[str]:
        return [t.name for t in self.tensors]

    def get(self, name: str) -> TensorSpec:
        for t in self.tensors:
            if t.name == name:
                return t
        raise KeyError(name)

    def trainable(self) -> List[TensorSpec]:
        return [t for t in self.tensors if not t.frozen]

    def byte_size(self, role: str) -> int:
        return sum(_align(t.bytes(role)) for t in self.tensors)

    def numel(self, trainable_only: bool = False) -> int:
        return sum(t.numel for t in self.tensors if not (trainable_only and t.frozen))


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


@dataclass
class ComputeCost:
    """Forward FLOPs of one (layer, chunk) and the FLOPs *not* recomputed when saving at tier ``i``.

    ``avoided_recompute_flops`` must be non-decreasing in the tier
    (flextrain/core/layer.py:261-317).
    """
    total_fwd_flops: float
    avoided_recompute_flops: Tuple[float, ...]
    attn_fwd_flops: float = 0.0

    def __post_init__(self):
        a = self.avoided_recompute_flops
        if any(a[i] > a[i + 1] + 1e-6 for i in range(len(a) - 1)):
            raise ValueError(f"avoided_recompute_flops must be monotone, got {a}")


@dataclass
class ChunkMeta:
    """Packing metadata of one training chunk (several short sequences, or one slice of a long one).

    ``cu_seqlens_q`` / ``cu_seqlens_k`` are int32 device tensors; queries of a sequence are the last
    ``len_q`` positions of its ``len_k`` keys (``len_k = prior_len + len_q``).
    """
    chunk_id: int
    num_tokens: int
    seq_ids: List[int]
    seq_lens: List[int]                 # tokens of each packed sequence inside this chunk
    prior_lens: List[int]               # tokens of the same sequence in earlier chunks
    seq_offsets: List[int]              # offset of this chunk's tokens inside their sequence (== prior_lens)
    has_more_chunks: List[bool]
    cu_seqlens_q: torch.Tensor
    cu_seqlens_k: torch.Tensor
    max_seqlen_q: int
    max_seqlen_k: int
    positions: torch.Tensor             # (T,) int32, or (T,3) for MRoPE
    tokens: Optional[torch.Tensor] = None
    targets: Optional[torch.Tensor] = None
    loss_mask: Optional[torch.Tensor] = None
    seq_group: int = 0
    extra: Dict[str, Any] = field(default_factory=dict)

    @property
    def total_k(self) -> int:
        return sum(self.seq_lens) + sum(self.prior_lens)

    @property
    def has_prior(self) -> bool:
        return any(p > 0 for p in self.prior_lens)

    @staticmethod
    def build(chunk_id: int, seq_ids: Sequence[int], seq_lens: Sequence[int], prior_lens: Sequence[int],
              has_more: Sequence[bool], device, *, tokens=None, targets=None, loss_mask=None, seq_group: int = 0,
              positions: Optional[torch.Tensor] = None) -> "ChunkMeta":
        cu_q, cu_k, pos = [0], [0], []
        for L, P in zip(seq_lens, prior_lens):
            cu_q.append(cu_q[-1] + L)
            cu_k.append(cu_k[-1] + L + P)
            pos.append(torch.arange(P, P + L, dtype=torch.int32))
        T = cu_q[-1]
        if positions is None:
            positions = torch.cat(pos) if pos else torch.zeros(0, dtype=torch.int32)
        return ChunkMeta(
            chunk_id=chunk_id, num_tokens=T, seq_ids=list(seq_ids), seq_lens=list(seq_lens),
            prior_lens=list(prior_lens), seq_offsets=list(prior_lens), has_more_chunks=list(has_more),
            cu_seqlens_q=torch.tensor(cu_q, dtype=torch.int32, device=device),
            cu_seqlens_k=torch.tensor(cu_k, dtype=torch.int32, device=device),
            max_seqlen_q=max(seq_lens) if len(seq_lens) else 0,
            max_seqlen_k=max((l + p for l, p in zip(seq_lens, prior_lens)), default=0),
            positions=positions.to(device), tokens=tokens, targets=targets, loss_mask=loss_mask, seq_group=seq_group)


@dataclass
class KVContextWindow:
    """Rolling K/V (and dK/dV) window shared by all layers; see flextrain/engine/buffers.py:57-98."""
    k: torch.Tensor
    v: torch.Tensor
    dk: Optional[torch.Tensor] = None
    dv: Optional[torch.Tensor] = None


@dataclass
class LayerContext:
    """Per-call services the engine hands to a layer (flextrain/core/layer.py:599-676)."""
    kv_window: Optional[KVContextWindow] = None
    lin_state_in: Optional[torch.Tensor] = None       # (Nseq, HV, dk, dv) fp32 state carried into this chunk
    lin_conv_in: Optional[torch.Tensor] = None        # (Nseq, conv_dim, W-1)
    lin_dstate_in: Optional[torch.Tensor] = None      # gradient of the state flowing back from the next chunk
    lin_dconv_in: Optional[torch.Tensor] = None
    lin_attn_recompute_only: bool = False
    secondary_stream: Any = None
    total_tokens_per_step: int = 0
    training: bool = True
    tp: Any = None                                     # TensorParallel group handle, or None
    ep: Any = None                                     # ExpertParallel group handle, or None
    param_gather: Any = None                           # data parallel with deferred parameter all-gather: callable
                                                       # (layer_id, x, w) -> x @ w.T or None (see parallel/dp.py)
    out: Dict[str, Any] = field(default_factory=dict)  # values a layer hands back (state gradients, ...)


@dataclass
class LossStats:
    total_loss: float = 0.0
    active_tokens: int = 0
    per_token_loss: Optional[torch.Tensor] = None
    argmax: Optional[torch.Tensor] = None
    argmax_prob: Optional[torch.Tensor] = None


@runtime_checkable
class Layer(Protocol):
    param_spec: ParamSpec
    activation_schema: Any

    def forward(self, x, meta: ChunkMeta, params: Dict[str, torch.Tensor], slot, ctx: LayerContext): ...
    def forward_recompute(self, meta: ChunkMeta, params, slot, ctx: LayerContext) -> None: ...
    def backward(self, dx, meta: ChunkMeta, params, grads, slot, ctx: LayerContext): ...
    def compute_cost(self, num_tokens: int, avg_ctx: float) -> ComputeCost: ...


@runtime_checkable
class InputLayer(Protocol):
    param_spec: ParamSpec

    def forward(self, meta: ChunkMeta, params) -> torch.Tensor: ...
    def backward(self, dx, meta: ChunkMeta, params, grads) -> None: ...


@runtime_checkable
class OutputLayer(Protocol):
    param_spec: ParamSpec

    def forward_backward(self, x, meta: ChunkMeta, params, grads, loss_fn, loss_scale: float) -> LossStats: ...


@runtime_checkable
class ModalityEncoder(Protocol):
    def encode(self, inputs) -> torch.Tensor: ...
