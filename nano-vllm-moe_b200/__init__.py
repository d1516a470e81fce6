"""B200-native FP8 quantized-linear engine, drop-in for nano-vllm-moe's
``nanovllm/quantization`` linear backend and ``nanovllm/layers/linear.py`` layers.

The arithmetic lives in ``libfp8lin.so`` (hand-written CUDA for sm_100a behind a
plain C ABI, ``include/fp8lin.h``); this package is the thin Python host side
that mirrors the reference's interface.  There is no CPU or library fallback:
calling a linear without the CUDA library raises.
"""
from . import _lib  # noqa: F401
from .quantization import (  # noqa: F401
    Fp8Config,
    Fp8LinearMethod,
    QuantizationConfig,
    QuantizeMethodBase,
    get_quant_config,
    is_fp8_config,
    process_weights_after_loading,
)
from .layers.linear import (  # noqa: F401
    ColumnParallelLinear,
    LinearBase,
    MergedColumnParallelLinear,
    QKVParallelLinear,
    ReplicatedLinear,
    RowParallelLinear,
)

from .layers.mlp import FusedFp8MLP  # noqa: F401,E402
from .layers.layernorm import QuantizedActivation, RMSNorm  # noqa: F401,E402

__all__ = [
    "FusedFp8MLP", "RMSNorm", "QuantizedActivation",
    "Fp8Config", "Fp8LinearMethod", "QuantizationConfig", "QuantizeMethodBase", "get_quant_config",
    "is_fp8_config", "process_weights_after_loading", "LinearBase", "ReplicatedLinear", "ColumnParallelLinear",
    "MergedColumnParallelLinear", "QKVParallelLinear", "RowParallelLinear",
]
