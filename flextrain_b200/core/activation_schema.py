"""Activation schema: which tensors a layer saves for backward, at which save tier, and where.

Reference behaviour kept (flextrain/core/activation_schema.py:73-519): fields are packed in
declaration order, each field and each slot end aligned to 256 B; a slot saved at level ``L``
holds exactly the fields with ``tier <= L``; ``slot.has(name)`` is *tier-aware* (a stale
higher-tier view left in a reused ring slot must never read as present).

A slot is either *dynamic* (fields are ordinary tensors, used when everything stays in HBM) or
*buffer-backed* (typed views into one ``uint8`` ring slot or pinned host slot).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from .layer import itemsize

ALIGN = 256
ON_DEVICE = -1          # SaveLevel: slot never leaves the GPU ring, every field kept


def align_up(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


@dataclass(frozen=True)
class ActivationField:
    name: str
    shape_fn: Callable[[int], Tuple[int, ...]]     # num_tokens -> shape
    dtype: torch.dtype
    tier: int                                       # 0 = always saved ... 3 = cheapest to recompute
    per_seq: bool = False                           # first dim is "sequences in chunk", not tokens

    def nbytes(self, num_tokens: int) -> int:
        n = 1
        for s in self.shape_fn(num_tokens):
            n *= int(s)
        return n * itemsize(self.dtype)


@dataclass
class ActivationSchema:
    fields: List[ActivationField]
    max_tier: int = 3

    def by_name(self, name: str) -> ActivationField:
        for f in self.fields:
            if f.name == name:
                return f
        raise KeyError(name)

    def fields_at(self, level: int) -> List[ActivationField]:
        lv = self.max_tier if level == ON_DEVICE else level
        return [f for f in self.fields if f.tier <= lv]

    def home_size_bytes(self, num_tokens: int, level: int) -> int:
        """Bytes of a slot saved at ``level`` (what travels to the host when offloaded)."""
        return align_up(sum(align_up(f.nbytes(num_tokens)) for f in self.fields_at(level)))

    def device_size_bytes(self, num_tokens: int) -> int:
        return self.home_size_bytes(num_tokens, self.max_tier)

    def offsets(self, num_tokens: int, level: int) -> Dict[str, Tuple[int, int]]:
        out, off = {}, 0
        for f in self.fields_at(level):
            nb = f.nbytes(num_tokens)
            out[f.name] = (off, nb)
            off += align_up(nb)
        return out


class ActivationSlot:
    """Named saved tensors of one (layer, chunk) at a save level."""

    def __init__(self, schema: ActivationSchema, num_tokens: int, level: int = ON_DEVICE,
                 buffer: Optional[torch.Tensor] = None):
        self.schema = schema
        self.num_tokens = num_tokens
        self.level = level
        self.buffer = buffer
        self._t: Dict[str, torch.Tensor] = {}
        if buffer is not None:
            self._build_views()

    # -- construction -------------------------------------------------------------
    @classmethod
    def from_buffer(cls, schema, buffer: torch.Tensor, num_tokens: int, level: int) -> "ActivationSlot":
        return cls(schema, num_tokens, level, buffer)

    def _build_views(self) -> None:
        self._t.clear()
        # a device ring slot is always laid out at full tier so forward can write every field
        layout_level = self.schema.max_tier if self.buffer.is_cuda else self.level
        for name, (off, nb) in self.schema.offsets(self.num_tokens, layout_level).items():
            f = self.schema.by_name(name)
            if off + nb > self.buffer.numel():
                raise ValueError(f"slot buffer too small for field {name}: need {off + nb}, have {self.buffer.numel()}")
            self._t[name] = self.buffer[off:off + nb].view(f.dtype).view(f.shape_fn(self.num_tokens))

    # -- access -------------------------------------------------------------------
    def _visible(self, name: str) -> bool:
        lv = self.schema.max_tier if self.level == ON_DEVICE else self.level
        return self.schema.by_name(name).tier <= lv

    def has(self, name: str) -> bool:
        """True only if ``name`` is populated *and* belongs to the slot's current save level."""
        return name in self._t and self._visible(name) and self._t[name] is not None

    def get(self, name: str) -> torch.Tensor:
        if not self.has(name):
            raise KeyError(f"activation field {name!r} not present at level {self.level}")
        return self._t[name]

    def __getitem__(self, name: str) -> torch.Tensor:
        return self.get(name)

    def put(self, name: str, value: torch.Tensor) -> torch.Tensor:
        """Store a field. Buffer-backed slots copy into their view; dynamic slots keep the tensor."""
        f = self.schema.by_name(name)
        if self.buffer is not None and name in self._t:
            dst = self._t[name]
            if dst.data_ptr() != value.data_ptr():
                dst.copy_(value.reshape(dst.shape))
            return dst
        self._t[name] = value
        return value

    def out(self, name: str, device, like_shape=None) -> torch.Tensor:
        """Tensor to write field ``name`` into (a ring view, or a fresh tensor for dynamic slots)."""
        if self.buffer is not None and name in self._t:
            return self._t[name]
        f = self.schema.by_name(name)
        t = torch.empty(f.shape_fn(self.num_tokens), dtype=f.dtype, device=device)
        self._t[name] = t
        return t

    def raise_level(self, level: int) -> None:
        """After recompute the slot again holds higher tiers."""
        self.level = level

    def demote(self, level: int) -> None:
        """Drop fields above ``level`` (frees dynamic tensors; buffer views just become invisible)."""
        self.level = level
        if self.buffer is None and level != ON_DEVICE:
            for f in self.schema.fields:
                if f.tier > level:
                    self._t.pop(f.name, None)

    def names(self) -> List[str]:
        return [n for n in self._t if self.has(n)]


def send_home(slot: ActivationSlot, host_buffer: torch.Tensor, level: int, copy_fn=None) -> ActivationSlot:
    """Copy the fields with ``tier <= level`` into a host slot laid out at ``level``; returns the host slot.

    ``copy_fn(dst, src)`` lets the caller route the copies through the copy engine / a stream
    (flextrain/core/activation_schema.py:483-519 issues one ``copy_`` per field).
    """
    host = ActivationSlot(slot.schema, slot.num_tokens, level, None)
    for name, (off, nb) in slot.schema.offsets(slot.num_tokens, level).items():
        f = slot.schema.by_name(name)
        dst = host_buffer[off:off + nb].view(f.dtype).view(f.shape_fn(slot.num_tokens))
        src = slot.get(name)
        (copy_fn or (lambda d, s: d.copy_(s, non_blocking=True)))(dst, src)
        host._t[name] = dst
    host.buffer = host_buffer
    return host


def fetch_home(host_slot: ActivationSlot, device_buffer: Optional[torch.Tensor], device, copy_fn=None) -> ActivationSlot:
    """Bring a host slot back to the GPU at its saved level (the slot is rebuilt at the *saved* level so stale
    higher-tier bytes in a reused ring slot stay invisible)."""
    dev = ActivationSlot(host_slot.schema, host_slot.num_tokens, host_slot.level, device_buffer)
    for f in host_slot.schema.fields_at(host_slot.level):
        src = host_slot._t[f.name]
        dst = dev.out(f.name, device)
        (copy_fn or (lambda d, s: d.copy_(s, non_blocking=True)))(dst, src)
    return dev
