"""IO layer: HuggingFace safetensors, training-state checkpoints, token sources, image pre-processing.

HuggingFace is a config + weights + tokenizer source here, not a compute path: a checkpoint's ``config.json`` becomes a
:class:`ModelConfig` and its shards are copied into the engine's buffers through one weight-name map per architecture
(``io/arch``).  The token-ingestion adapters are called *sources* (``io/sources.py``); "stream" is kept for CUDA streams.
The names below are the ones the reference exports from its ``flextrain.io`` (flextrain/io/__init__.py:17-34), plus
this package's additional adapters.
"""
from .sequence import Sequence
from .sources import (CustomSchemaTokenSource, HFTokenSource, JsonSFTTokenSource, MultimodalJsonSource, RankStridedSource,
                      RawTokenSource, ShardTokenSource, SyntheticTokenSource, TokenSource)

__all__ = ["CustomSchemaTokenSource", "HFTokenSource", "JsonSFTTokenSource", "MultimodalJsonSource", "RankStridedSource",
           "RawTokenSource", "Sequence", "ShardTokenSource", "SyntheticTokenSource", "TokenSource"]
