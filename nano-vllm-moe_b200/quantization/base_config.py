"""Linear-backend interface; same contract as the reference's
nanovllm/quantization/base_config.py:9-38 so layers written against it work
unchanged."""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch
from torch import nn


class QuantizeMethodBase(ABC):
    """What a linear layer delegates to: buffer creation, post-load packing, forward."""

    @abstractmethod
    def create_weights(self, layer: nn.Module, *, input_size_per_partition: int,
                       output_partition_sizes: list[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype) -> None:
        ...

    def process_weights_after_loading(self, layer: nn.Module) -> None:
        return None

    @abstractmethod
    def apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        ...


class QuantizationConfig(ABC):
    @abstractmethod
    def get_name(self) -> str:
        ...

    @abstractmethod
    def get_quant_method(self, layer: nn.Module, prefix: str = "") -> QuantizeMethodBase | None:
        ...
