"""All long-lived memory of one engine (flextrain/engine/buffers.py:497-1330).

Per layer there are three flat byte buffers — parameters, gradients, optimizer state — each packed
in spec order with 256 B alignment and exposed as typed views.  A class of state is either
*resident* (one GPU buffer per layer; the normal case with 180 GB of HBM) or *ringed*: the master
copy lives in pinned host memory and ``n`` GPU slots are recycled layer by layer (layer ``l`` uses
slot ``l % n``), moved by one coalesced copy per layer instead of one per tensor.  Embedding and
head parameters, gradients and optimizer state always stay on the GPU
(flextrain/engine/buffers.py:547-556, 824-860).  Frozen tensors (LoRA base weights) have no
gradient / state bytes and are skipped when a layer is written back.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..core.activation_schema import align_up
from ..core.layer import KVContextWindow, ParamSpec, itemsize
from .host_memory import HostMemoryBackend, default_backend


def _layout(entries: List[Tuple[str, Tuple[int, ...], torch.dtype]]):
    """[(name, shape, dtype)] -> ({name: (offset, nbytes, shape, dtype)}, total_bytes)."""
    out, off = {}, 0
    for name, shape, dt in entries:
        n = 1
        for s in shape:
            n *= s
        nb = n * itemsize(dt)
        out[name] = (off, nb, shape, dt)
        off += align_up(nb)
    return out, off


def _views(buf: torch.Tensor, layout) -> Dict[str, torch.Tensor]:
    return {name: buf[off:off + nb].view(dt).view(shape) for name, (off, nb, shape, dt) in layout.items()}


class LayerBuffers:
    """Layouts of one layer's three state classes (device dtype view and host/master dtype view)."""

    def __init__(self, spec: ParamSpec, optimizer):
        self.spec = spec
        self.p_layout, self.p_bytes = _layout([(t.name, t.shape, t.compute_dtype) for t in spec])
        self.m_layout, self.m_bytes = _layout([(t.name, t.shape, t.master_dtype) for t in spec])
        self.g_layout, self.g_bytes = _layout([(t.grad_name, t.shape, t.grad_dtype) for t in spec.trainable()])
        st = optimizer.state_specs(spec) if optimizer is not None else []
        self.o_layout, self.o_bytes = _layout([(s.key, s.shape, s.dtype) for s in st])
        self.same_master = all(t.master_dtype == t.compute_dtype for t in spec)


class BufferManager:
    def __init__(self, layer_specs: List[ParamSpec], embed_spec: ParamSpec, head_spec: ParamSpec, optimizer, device,
                 *, n_gpu_layers: Optional[int] = None, n_gpu_grads: Optional[int] = None,
                 n_gpu_opt_layers: Optional[int] = None, host_backend: Optional[HostMemoryBackend] = None,
                 kv_window_tokens: int = 0, kv_heads: int = 0, head_dim: int = 0, act_dtype=torch.bfloat16,
                 host_act_bytes: int = 0, verbose: bool = False, device_alloc=None, shard_opt: bool = False):
        self.device = torch.device(device)
        self.host = host_backend or default_backend(device)
        L = len(layer_specs)
        self.n_layers = L
        self.n_p = L if n_gpu_layers is None else max(1, min(L, n_gpu_layers))
        self.n_g = L if n_gpu_grads is None else max(1, min(L, n_gpu_grads))
        self.n_o = L if n_gpu_opt_layers is None else max(0, min(L, n_gpu_opt_layers))
        self.layers = [LayerBuffers(s, optimizer) for s in layer_specs]
        self.embed = LayerBuffers(embed_spec, optimizer)
        self.head = LayerBuffers(head_spec, optimizer)
        dev = self.device
        u8 = lambda n: torch.zeros(max(n, 1), dtype=torch.uint8, device=dev)
        self.params_resident = self.n_p >= L
        self.grads_resident = self.n_g >= L
        self.opt_resident = self.n_o >= L
        maxp = max(lb.p_bytes for lb in self.layers)
        maxg = max(lb.g_bytes for lb in self.layers)
        maxo = max(lb.o_bytes for lb in self.layers)
        # ---- parameters / gradients: one arena each when a data-parallel group needs them peer-mapped
        #      (unit order: embed, layer 0..L-1, head), else one buffer per unit
        self.param_arena = self.grad_arena = None
        self.p_off: Dict[object, int] = {}
        self.g_off: Dict[object, int] = {}
        if device_alloc is not None:
            if not (self.params_resident and self.grads_resident):
                raise ValueError("peer-mapped parameter / gradient arenas need resident parameters and gradients")
            units = [("embed", self.embed)] + [(i, lb) for i, lb in enumerate(self.layers)] + [("head", self.head)]
            po = go = 0
            for key, lb in units:
                self.p_off[key], self.g_off[key] = po, go
                po += align_up(max(lb.p_bytes, 1)); go += align_up(max(lb.g_bytes, 1))
            self.param_arena, self.grad_arena = device_alloc(po, "params"), device_alloc(go, "grads")
            pa, ga = self.param_arena.local, self.grad_arena.local
            cut = lambda arena, off, n: arena[off:off + max(n, 1)]
            self.embed_p, self.embed_g = cut(pa, self.p_off["embed"], self.embed.p_bytes), cut(ga, self.g_off["embed"], self.embed.g_bytes)
            self.head_p, self.head_g = cut(pa, self.p_off["head"], self.head.p_bytes), cut(ga, self.g_off["head"], self.head.g_bytes)
            self.gpu_p = [cut(pa, self.p_off[i], lb.p_bytes) for i, lb in enumerate(self.layers)]
            self.gpu_g = [cut(ga, self.g_off[i], lb.g_bytes) for i, lb in enumerate(self.layers)]
            self.embed_o, self.head_o = u8(0 if shard_opt else self.embed.o_bytes), u8(0 if shard_opt else self.head.o_bytes)
        else:
            # ---- resident embed / head (params + grads + opt state)
            self.embed_p, self.embed_g, self.embed_o = u8(self.embed.p_bytes), u8(self.embed.g_bytes), u8(self.embed.o_bytes)
            self.head_p, self.head_g, self.head_o = u8(self.head.p_bytes), u8(self.head.g_bytes), u8(self.head.o_bytes)
            # ---- per-layer state: resident buffers or rings + pinned host masters
            self.gpu_p = [u8(lb.p_bytes) for lb in self.layers] if self.params_resident else [u8(maxp) for _ in range(self.n_p)]
            self.gpu_g = [u8(lb.g_bytes) for lb in self.layers] if self.grads_resident else [u8(maxg) for _ in range(self.n_g)]
        if shard_opt:
            # optimizer state lives in the data-parallel group's shards, not here
            self.gpu_o = [u8(0) for _ in self.layers]
            self.opt_resident = True
            self.host_p = self.host_g = self.host_o = None
            self._finish_init(kv_window_tokens, kv_heads, head_dim, act_dtype, host_act_bytes)
            return
        if self.opt_resident:
            self.gpu_o = [u8(lb.o_bytes) for lb in self.layers]
        else:
            self.gpu_o = [u8(maxo) for _ in range(max(self.n_o, 2))]
        self.host_p = None if self.params_resident else [self.host.alloc(lb.m_bytes) for lb in self.layers]
        self.host_g = None if self.grads_resident else [self.host.alloc(lb.g_bytes) for lb in self.layers]
        self.host_o = None if self.opt_resident else [self.host.alloc(lb.o_bytes) for lb in self.layers]
        self._finish_init(kv_window_tokens, kv_heads, head_dim, act_dtype, host_act_bytes)

    def _finish_init(self, kv_window_tokens, kv_heads, head_dim, act_dtype, host_act_bytes) -> None:
        dev = self.device
        self._view_cache: Dict[Tuple[str, int], Dict[str, torch.Tensor]] = {}
        # ---- context windows
        self.kv_window = None
        if kv_window_tokens > 0 and kv_heads > 0:
            mk = lambda: torch.zeros(kv_window_tokens, kv_heads, head_dim, dtype=act_dtype, device=dev)
            self.kv_window = KVContextWindow(mk(), mk(), mk(), mk())
        # ---- host activation arena (bump allocated per round)
        self.host_act = self.host.alloc(host_act_bytes) if host_act_bytes > 0 else None
        self._host_act_off = 0

    # ------------------------------------------------------------------------ views
    def _slot(self, kind: str, layer: int) -> int:
        n = {"p": self.n_p, "g": self.n_g, "o": max(self.n_o, 2) if not self.opt_resident else self.n_o}[kind]
        res = {"p": self.params_resident, "g": self.grads_resident, "o": self.opt_resident}[kind]
        return layer if res else layer % n

    def params(self, layer: int) -> Dict[str, torch.Tensor]:
        key = ("p", layer)
        if key not in self._view_cache:
            self._view_cache[key] = _views(self.gpu_p[self._slot("p", layer)], self.layers[layer].p_layout)
        return self._view_cache[key]

    def grads(self, layer: int) -> Dict[str, torch.Tensor]:
        key = ("g", layer)
        if key not in self._view_cache:
            self._view_cache[key] = _views(self.gpu_g[self._slot("g", layer)], self.layers[layer].g_layout)
        return self._view_cache[key]

    def opt_state(self, layer: int) -> Dict[str, torch.Tensor]:
        key = ("o", layer)
        if key not in self._view_cache:
            self._view_cache[key] = _views(self.gpu_o[self._slot("o", layer)], self.layers[layer].o_layout)
        return self._view_cache[key]

    def grad_buffer(self, layer: int) -> torch.Tensor:
        return self.gpu_g[self._slot("g", layer)][: self.layers[layer].g_bytes]

    def param_buffer(self, layer: int) -> torch.Tensor:
        return self.gpu_p[self._slot("p", layer)][: self.layers[layer].p_bytes]

    def opt_buffer(self, layer: int) -> torch.Tensor:
        return self.gpu_o[self._slot("o", layer)][: self.layers[layer].o_bytes]

    def embed_params(self): return self._cached("ep", self.embed_p, self.embed.p_layout)
    def embed_grads(self): return self._cached("eg", self.embed_g, self.embed.g_layout)
    def embed_opt(self): return self._cached("eo", self.embed_o, self.embed.o_layout)
    def head_params(self): return self._cached("hp", self.head_p, self.head.p_layout)
    def head_grads(self): return self._cached("hg", self.head_g, self.head.g_layout)
    def head_opt(self): return self._cached("ho", self.head_o, self.head.o_layout)

    def _cached(self, key, buf, layout):
        k = (key, -1)
        if k not in self._view_cache:
            self._view_cache[k] = _views(buf, layout)
        return self._view_cache[k]

    def host_params(self, layer: int) -> Dict[str, torch.Tensor]:
        """Master copy of a layer (host views when ringed, the GPU views when resident)."""
        if self.params_resident:
            return self.params(layer)
        return _views(self.host_p[layer], self.layers[layer].m_layout)

    def master_opt_state(self, layer: int) -> Dict[str, torch.Tensor]:
        """Optimizer state of a layer where it lives between steps (host views when ringed, GPU views when resident)."""
        if self.opt_resident or self.host_o is None:
            return self.opt_state(layer)
        return _views(self.host_o[layer], self.layers[layer].o_layout)

    # ------------------------------------------------------------------ fetch / offload
    def _copy(self, dst: torch.Tensor, src: torch.Tensor, copier=None):
        if copier is not None:
            copier(dst, src)
        else:
            dst.copy_(src, non_blocking=True)

    def fetch_layer_params(self, layer: int, copier=None) -> None:
        if self.params_resident:
            return
        lb = self.layers[layer]
        if lb.same_master:
            self._copy(self.param_buffer(layer), self.host_p[layer][: lb.p_bytes], copier)
        else:
            dst, src = self.params(layer), _views(self.host_p[layer], lb.m_layout)
            for n in dst:
                dst[n].copy_(src[n], non_blocking=True)

    def offload_layer_params(self, layer: int, copier=None, skip_frozen: bool = True) -> None:
        if self.params_resident:
            return
        lb = self.layers[layer]
        if lb.same_master and not (skip_frozen and any(t.frozen for t in lb.spec)):
            self._copy(self.host_p[layer][: lb.p_bytes], self.param_buffer(layer), copier)
            return
        src, dst = self.params(layer), _views(self.host_p[layer], lb.m_layout)
        for t in lb.spec:
            if skip_frozen and t.frozen:
                continue
            dst[t.name].copy_(src[t.name], non_blocking=True)

    def fetch_layer_grads(self, layer: int, copier=None) -> None:
        if not self.grads_resident:
            self._copy(self.grad_buffer(layer), self.host_g[layer], copier)

    def offload_layer_grads(self, layer: int, copier=None) -> None:
        if not self.grads_resident:
            self._copy(self.host_g[layer], self.grad_buffer(layer), copier)

    def zero_layer_grads(self, layer: int) -> None:
        self.grad_buffer(layer).zero_()

    def fetch_layer_opt(self, layer: int, copier=None) -> None:
        if not self.opt_resident:
            self._copy(self.opt_buffer(layer), self.host_o[layer], copier)

    def offload_layer_opt(self, layer: int, copier=None) -> None:
        if not self.opt_resident:
            self._copy(self.host_o[layer], self.opt_buffer(layer), copier)

    # ------------------------------------------------------------------ host activations
    def reset_host_act(self) -> None:
        self._host_act_off = 0

    def host_act_slot(self, nbytes: int) -> torch.Tensor:
        nbytes = align_up(nbytes)
        if self.host_act is None or self._host_act_off + nbytes > self.host_act.numel():
            raise MemoryError(f"host activation arena exhausted: need {nbytes} more bytes at offset "
                              f"{self._host_act_off} of {0 if self.host_act is None else self.host_act.numel()}")
        s = self.host_act[self._host_act_off:self._host_act_off + nbytes]
        self._host_act_off += nbytes
        return s

    # ------------------------------------------------------------------------ sizes
    def gpu_bytes(self) -> int:
        n = sum(b.numel() for b in self.gpu_p + self.gpu_g + self.gpu_o)
        n += sum(b.numel() for b in (self.embed_p, self.embed_g, self.embed_o, self.head_p, self.head_g, self.head_o))
        if self.kv_window is not None:
            n += 4 * self.kv_window.k.numel() * self.kv_window.k.element_size()
        return n

    def host_bytes(self) -> int:
        n = 0
        for lst in (self.host_p, self.host_g, self.host_o):
            if lst is not None:
                n += sum(b.numel() for b in lst)
        if self.host_act is not None:
            n += self.host_act.numel()
        return n

    def destroy(self) -> None:
        for lst in (self.host_p, self.host_g, self.host_o):
            if lst is not None:
                for b in lst:
                    self.host.free(b)
        if self.host_act is not None:
            self.host.free(self.host_act)
        self._view_cache.clear()
