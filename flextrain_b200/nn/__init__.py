"""Model layer: blocks, the config-driven decoder layer, embedding, head, losses (the names the reference exports
from ``flextrain.nn``, flextrain/nn/__init__.py)."""
from .embed import TokenEmbedLayer
from .head import LMHead
from .loss import CrossEntropyLoss, GRPOLoss, LossFn, MSELoss, TokenContext, TokenSlice, apply_loss

IGNORE_INDEX = -100          # target value of a position that carries no loss

__all__ = ["TokenEmbedLayer", "LMHead", "CrossEntropyLoss", "GRPOLoss", "LossFn", "MSELoss", "TokenContext", "TokenSlice", "apply_loss",
           "IGNORE_INDEX"]
