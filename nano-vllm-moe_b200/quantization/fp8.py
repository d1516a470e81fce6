"""FP8 linear method: W8A16 and W8A8-static behind ``QuantizeMethodBase``.

Same buffers, loader behaviour and ``apply`` contract as the reference's
``Fp8LinearMethod`` (nanovllm/quantization/fp8.py:63-249), so checkpoints
exported by scripts/quantization/quantize.py load unchanged:

* ``qweight``      uint8  [K_part, N_part]   e4m3 codes, filled shard by shard
* ``weight_scale`` float32 [N_part]
* ``input_scale``  float32 scalar            (fp8_w8a8_static only)

Differences, all deliberate:
* one backend (libfp8lin.so); no NANOVLLM_FP8_W8A8_RUNTIME_BACKEND dispatch;
* per-output-channel weight scales are kept for W8A8 too (the reference folds
  them into one per-tensor scale and re-rounds the weights, fp8.py:100-105);
* after loading, the weight is repacked once into 128 x 128-byte tiles (the
  layout every kernel streams, ``qweight_packed``) and the [K, N] copy is released.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from .. import _lib
from . import kernels
from .base_config import QuantizationConfig, QuantizeMethodBase

FP8_W8A16 = "fp8_w8a16"
FP8_W8A8_STATIC = "fp8_w8a8_static"
_SCHEMES = (FP8_W8A16, FP8_W8A8_STATIC)


def is_fp8_config(config: Any) -> bool:
    return getattr(config, "quantization_type", None) in _SCHEMES


@dataclass(frozen=True)
class Fp8Config(QuantizationConfig):
    quantization_type: str = FP8_W8A16
    keep_checkpoint_layout: bool = False   # keep the [K, N] ``qweight`` copy after prepacking

    def __post_init__(self) -> None:
        if self.quantization_type not in _SCHEMES:
            raise ValueError(f"Unsupported FP8 quantization_type={self.quantization_type!r}")

    def get_name(self) -> str:
        return "fp8"

    def get_quant_method(self, layer: nn.Module, prefix: str = "") -> "Fp8LinearMethod":
        return Fp8LinearMethod(self, prefix)


def _tp_slice(layer: nn.Module, tensor: torch.Tensor, dim_for: dict[int, int]) -> torch.Tensor:
    """Cut this rank's share out of a full checkpoint tensor.

    ``dim_for`` maps the layer's ``tp_dim`` (0 = column parallel, 1 = row
    parallel) to the tensor dimension that is split; a missing entry means the
    tensor is replicated for that kind of layer."""
    dim = dim_for.get(getattr(layer, "tp_dim", None))
    if dim is None:
        return tensor
    per_rank = tensor.shape[dim] // layer.tp_size
    return tensor.narrow(dim, layer.tp_rank * per_rank, per_rank)


def _dest_range(layer: nn.Module, shard_id, loaded_size: int) -> tuple[int, int]:
    """Column range of the fused buffer that ``shard_id`` (q/k/v, 0/1) fills."""
    if shard_id is not None and hasattr(layer, "get_quant_output_offset_size"):
        return layer.get_quant_output_offset_size(shard_id)
    return 0, loaded_size


class Fp8LinearMethod(QuantizeMethodBase):
    def __init__(self, quant_config: Fp8Config, prefix: str = "") -> None:
        self.quant_config = quant_config
        self.prefix = prefix

    @property
    def is_w8a8(self) -> bool:
        return self.quant_config.quantization_type == FP8_W8A8_STATIC

    # ---- buffers + loaders -----------------------------------------------------
    def create_weights(self, layer: nn.Module, *, input_size_per_partition: int,
                       output_partition_sizes: list[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype) -> None:
        n_part = sum(output_partition_sizes)
        layer.register_buffer("qweight", torch.empty((input_size_per_partition, n_part), dtype=torch.uint8))
        layer.register_buffer("weight_scale", torch.empty((n_part,), dtype=torch.float32))
        layer.qweight.weight_loader = self._qweight_loader(layer)
        layer.weight_scale.weight_loader = self._weight_scale_loader(layer)
        if self.is_w8a8:
            layer.register_buffer("input_scale", torch.empty((), dtype=torch.float32))
            layer.input_scale.weight_loader = self._input_scale_loader()
        layer._fp8_kn_shape = (input_size_per_partition, n_part)

    def _qweight_loader(self, layer: nn.Module):
        def load(param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
            # checkpoint tensor is [N, K]: column layers split N (dim 0), row layers split K (dim 1)
            mine = _tp_slice(layer, loaded, {0: 0, 1: 1})
            start, size = _dest_range(layer, shard_id, mine.shape[0])
            param.data[:, start:start + size].copy_(mine.t())
        return load

    def _weight_scale_loader(self, layer: nn.Module):
        def load(param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
            flat = loaded.reshape(-1).to(torch.float32)
            if flat.numel() > 1:
                flat = _tp_slice(layer, flat, {0: 0})      # row layers keep every channel's scale
            if flat.numel() == 1 and shard_id is None:
                # one scale for the whole tensor: broadcast it to every channel (the
                # reference writes only element 0 here and leaves the rest unset)
                param.data.fill_(float(flat))
                return
            start, size = _dest_range(layer, shard_id, flat.numel())
            dest = param.data[start:start + size]
            if flat.numel() == 1:
                dest.fill_(float(flat))
            else:
                dest.copy_(flat)
        return load

    @staticmethod
    def _input_scale_loader():
        def load(param: torch.Tensor, loaded: torch.Tensor, shard_id=None) -> None:
            param.data.copy_(loaded.reshape(()).to(torch.float32))
        return load

    # ---- prepack ---------------------------------------------------------------------
    def process_weights_after_loading(self, layer: nn.Module) -> None:
        if not layer.qweight.is_cuda:
            return  # same as the reference: nothing to do for a CPU-resident layer
        major, _ = torch.cuda.get_device_capability(layer.qweight.device)
        if major != 10:
            raise RuntimeError("the fp8lin kernels are built for sm_100a (B200) only")
        _lib.load()  # fail here, loudly, if the CUDA library was not built
        layer.register_buffer("qweight_packed", kernels.prepack_weight(layer.qweight), persistent=False)
        layer.weight_scale.data = layer.weight_scale.data.to(torch.float32).contiguous()
        if self.is_w8a8:
            layer.input_scale.data = layer.input_scale.data.to(torch.float32).reshape(())
        if not self.quant_config.keep_checkpoint_layout:
            layer.qweight = torch.empty((0, 0), dtype=torch.uint8, device=layer.qweight_packed.device)
        layer._fp8_backend = "fp8lin_w8a8" if self.is_w8a8 else "fp8lin_w8a16"

    # ---- forward ---------------------------------------------------------------------
    def apply(self, layer: nn.Module, x: torch.Tensor, bias: torch.Tensor | None = None,
              out: torch.Tensor | None = None) -> torch.Tensor:
        """``out`` (optional, bf16 [M, N], row stride a multiple of 8) receives the result in place;
        the row-parallel layer uses it to compute M in chunks into one buffer."""
        backend = getattr(layer, "_fp8_backend", None)
        codes = getattr(x, "codes", None)
        if codes is not None:
            # activations already quantised by the producer (layers/layernorm.py RMSNorm.forward_quant)
            if not self.is_w8a8:
                raise ValueError("pre-quantised activations need the fp8_w8a8_static scheme")
            if backend is None:
                raise RuntimeError("FP8 backend is not initialized: call process_weights_after_loading first")
            if (x.scale.data_ptr() != layer.input_scale.data_ptr() and not torch.cuda.is_current_stream_capturing()
                    and not torch.equal(x.scale.reshape(()), layer.input_scale.reshape(()))):
                raise ValueError("the activations were quantised with a scale other than this layer's input_scale")
            if bias is not None and bias.dtype != torch.bfloat16:
                bias = bias.to(torch.bfloat16)
            y = kernels.launch_w8a8_preq(codes.reshape(-1, codes.shape[-1]), layer.qweight_packed, layer.input_scale,
                                         layer.weight_scale, bias, out=out)
            return out if out is not None else y.view(*codes.shape[:-1], y.shape[-1])
        if not x.is_cuda:
            scheme = "FP8 W8A8 static" if self.is_w8a8 else "FP8 W8A16"
            raise RuntimeError(f"{scheme} requires CUDA")
        if backend is None:
            raise RuntimeError("FP8 backend is not initialized: call process_weights_after_loading first")
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if x2.dtype != torch.bfloat16:
            x2 = x2.to(torch.bfloat16)
        if bias is not None and bias.dtype != torch.bfloat16:
            bias = bias.to(torch.bfloat16)
        if self.is_w8a8:
            y = kernels.launch_w8a8_gemm(x2, layer.qweight_packed, layer.input_scale, layer.weight_scale, bias, out=out)
        else:
            y = kernels.launch_w8a16_gemm(x2, layer.qweight_packed, layer.weight_scale, bias, out=out)
        if out is not None:
            return out
        return y.view(*x.shape[:-1], y.shape[-1]).to(x.dtype)
