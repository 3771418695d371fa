"""Quantized ``nn.Linear`` replacements over the B200 kernels (mirrors ``engine/quantization``)."""

from .checkpoint import load_w4a16_checkpoint, save_w4a16_checkpoint
from .fused_qkv import FusedProjections, install_fused_qkv, uninstall_fused_qkv
from .int8 import Int8Linear, model_storage_bytes, quantize_linear_modules
from .w4a16 import (
    W4A16Linear, W4A16Report, describe, install_w4a16, load_w4a16_model, reference_mode,
    reserve_workspace, w4a16_modules,
)

__all__ = [
    "Int8Linear", "model_storage_bytes", "quantize_linear_modules",
    "W4A16Linear", "W4A16Report", "describe", "install_w4a16", "load_w4a16_model",
    "reference_mode", "reserve_workspace", "w4a16_modules", "save_w4a16_checkpoint", "load_w4a16_checkpoint",
    "FusedProjections", "install_fused_qkv", "uninstall_fused_qkv",
]
