"""Checkpoint exports (flextrain/export/__init__.py:42-51): full HF directory, PEFT LoRA adapter, merged."""
from ._common import write_sharded_safetensors
from ._hf_full import save_hf_full
from ._lora_adapter import save_lora_adapter
from ._merged import merge_lora_into_base, save_hf_merged

__all__ = ["save_hf_full", "save_lora_adapter", "save_hf_merged", "merge_lora_into_base", "write_sharded_safetensors"]
