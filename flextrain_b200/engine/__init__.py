"""Engine layer: the ActiveModel driver, buffers and rings, round / chunk schedule, streams and events, host memory
(the names the reference exports from ``flextrain.engine``, flextrain/engine/__init__.py)."""
from .buffers import BufferManager, LayerBuffers
from .host_memory import (HostMemoryBackend, LocalPinnedHostBackend, UnpinnedHostBackend, default_backend,
                          default_host_backend, unregister_all_process_pinned_memory)
from .schedule import ChunkPlan, ChunkPolicy, pack_sequences, prepare_training_chunks, split_sequences
from .streams import EventBook, EventMap, LayerChunkEventMap, LayerEventMap, SlotEventMap, StreamBundle

__all__ = ["BufferManager", "LayerBuffers", "HostMemoryBackend", "LocalPinnedHostBackend", "UnpinnedHostBackend",
           "default_backend", "default_host_backend", "unregister_all_process_pinned_memory", "ChunkPlan", "ChunkPolicy",
           "pack_sequences", "prepare_training_chunks", "split_sequences", "EventBook", "EventMap", "LayerChunkEventMap",
           "LayerEventMap", "SlotEventMap", "StreamBundle"]
