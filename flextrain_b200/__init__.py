"""flextrain_b200: a Blackwell-native working-set training engine.

Public surface (mirrors flextrain/__init__.py:7-32):
``from_pretrained``, ``from_dims``, ``register_block_builder``, ``BuildContext``, ``ActiveModel``,
``StepStats``, the optimizers, ``Sequence`` and the token sources, ``HardwareCost``,
``WorkingSetConfig``.
"""
from .api import BlockBuilder, BuildContext, from_dims, from_pretrained, register_block_builder
from .core.save_level import HardwareCost, SaveLevelPlan
from .core.working_set import WorkingSetConfig, determine_working_set_config
from .engine.active_model import ActiveModel, StepStats
from .io.sequence import Sequence
from .io.sources import (CustomSchemaTokenSource, HFTokenSource, JsonSFTTokenSource, MultimodalJsonSource, RankStridedSource, RawTokenSource,
                         ShardTokenSource, SyntheticTokenSource, TokenSource)
from .optim import AdamW, HybridMuonAdamW, Muon
from . import export  # noqa: E402  (``flextrain_b200.export.save_hf_full`` / ``save_lora_adapter`` / ``save_hf_merged``)

__version__ = "0.1.0"

__all__ = [
    "from_pretrained", "from_dims", "register_block_builder", "BlockBuilder", "BuildContext", "ActiveModel", "StepStats",
    "AdamW", "Muon", "HybridMuonAdamW", "Sequence", "TokenSource", "SyntheticTokenSource", "RawTokenSource",
    "ShardTokenSource", "JsonSFTTokenSource", "CustomSchemaTokenSource", "HFTokenSource", "RankStridedSource", "MultimodalJsonSource",
    "HardwareCost",
    "SaveLevelPlan", "WorkingSetConfig", "determine_working_set_config",
]
