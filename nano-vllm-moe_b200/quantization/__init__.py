from .base_config import QuantizationConfig, QuantizeMethodBase
from .fp8 import Fp8Config, Fp8LinearMethod, is_fp8_config
from .registry import get_quant_config, process_weights_after_loading

__all__ = [
    "Fp8Config", "Fp8LinearMethod", "QuantizationConfig", "QuantizeMethodBase",
    "get_quant_config", "is_fp8_config", "process_weights_after_loading",
]
