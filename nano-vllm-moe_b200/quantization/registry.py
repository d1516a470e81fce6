"""Config lookup and the post-load hook (reference: nanovllm/quantization/registry.py:9-19)."""
from __future__ import annotations

from torch import nn

from .base_config import QuantizationConfig
from .fp8 import Fp8Config, is_fp8_config


def get_quant_config(hf_config) -> QuantizationConfig | None:
    """``hf_config.quantization_type`` in {fp8_w8a16, fp8_w8a8_static} -> Fp8Config, else None."""
    if is_fp8_config(hf_config):
        return Fp8Config(hf_config.quantization_type)
    return None


def process_weights_after_loading(model: nn.Module) -> None:
    """Prepack every module that carries a ``quant_method`` (called once after the checkpoint is loaded)."""
    for module in model.modules():
        method = getattr(module, "quant_method", None)
        if method is not None:
            method.process_weights_after_loading(module)
