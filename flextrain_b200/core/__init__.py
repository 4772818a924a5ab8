"""Core layer: layer contracts, activation schema and slots, save tiers and the DP solver binding, the working-set
planner, sizing, memory probes, hardware probe, FLOP accounting, modality records (the names the reference exports
from ``flextrain.core``, flextrain/core/__init__.py)."""
from .activation_schema import ActivationField, ActivationSchema, ActivationSlot
from .hw_probe import probe_hardware
from .layer import (ChunkMeta, ComputeCost, InputLayer, Layer, LayerContext, ModalityEncoder, OutputLayer, ParamSpec,
                    TensorSpec)
from .modality import ImageEmbeddings, ImageGradInputs, ImageInputCPU, ImageInputs, InputsSummary
from .save_level import DPTables, HardwareCost, SaveLevelPlan, build_dp_tables
from .working_set import WorkingSetConfig, determine_working_set_config

__all__ = ["ActivationField", "ActivationSchema", "ActivationSlot", "probe_hardware", "ChunkMeta", "ComputeCost",
           "InputLayer", "Layer", "LayerContext", "ModalityEncoder", "OutputLayer", "ParamSpec", "TensorSpec",
           "ImageEmbeddings", "ImageGradInputs", "ImageInputCPU", "ImageInputs", "InputsSummary", "DPTables",
           "HardwareCost", "SaveLevelPlan", "build_dp_tables", "WorkingSetConfig", "determine_working_set_config"]
