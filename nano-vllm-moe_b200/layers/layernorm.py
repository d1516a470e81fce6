"""RMSNorm with the W8A8 activation quantiser folded in.

Same constructor, parameter and ``forward(x, residual=None)`` contract as the reference's
``nanovllm/layers/layernorm.py:5-49`` (one result, or ``(result, new_residual)`` when a residual is
given).  ``forward_quant`` is the fused form for a norm whose only consumer is a W8A8-static linear
(``input_layernorm`` -> ``qkv_proj`` and ``post_attention_layernorm`` -> ``gate_up_proj`` in the
reference's decoder layer, nanovllm/models/qwen2.py:148-160): it returns the e4m3 codes that linear
would have produced from the norm's bf16 output, so the bf16 tensor is never written and the linear
runs without its quantiser pass (``Fp8LinearMethod.apply`` accepts the codes directly).

Arithmetic: the reference's compiled methods -- fp32 throughout, one rounding to bf16 on the product
with the weight; the residual stream is bf16(x + residual).
"""
from __future__ import annotations

import torch
from torch import nn

from ..quantization import kernels


class QuantizedActivation:
    """e4m3 codes [.., K] (uint8) of an activation together with the static scale they were made with."""

    __slots__ = ("codes", "scale")

    def __init__(self, codes: torch.Tensor, scale: torch.Tensor):
        self.codes = codes
        self.scale = scale

    @property
    def shape(self):
        return self.codes.shape


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6) -> None:
        super().__init__()
        self.hidden_size = hidden_size
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def _weight_bf16(self, device) -> torch.Tensor:
        w = self.weight.data
        if w.dtype != torch.bfloat16 or w.device != device:
            w = w.to(device=device, dtype=torch.bfloat16)
        return w.contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        if not x.is_cuda:
            raise RuntimeError("fp8lin RMSNorm requires CUDA")
        x2 = x.reshape(-1, x.shape[-1])
        if residual is None:
            _, y = kernels.rmsnorm_quant(x2, self._weight_bf16(x.device), self.eps)
            return y.view(x.shape)
        res = residual.reshape(-1, x.shape[-1]).clone()       # the reference returns a new residual tensor
        _, y = kernels.rmsnorm_quant(x2, self._weight_bf16(x.device), self.eps, residual=res)
        return y.view(x.shape), res.view(x.shape)

    def forward_quant(self, x: torch.Tensor, input_scale: torch.Tensor, residual: torch.Tensor | None = None,
                      inplace_residual: bool = True):
        """-> (QuantizedActivation, new_residual or None).  With ``inplace_residual`` (default) the
        residual tensor is updated in place, as a decode loop replayed from a CUDA graph needs."""
        if not x.is_cuda:
            raise RuntimeError("fp8lin RMSNorm requires CUDA")
        x2 = x.reshape(-1, x.shape[-1])
        res = None
        if residual is not None:
            res = residual.reshape(-1, x.shape[-1])
            if not inplace_residual:
                res = res.clone()
        xq, _ = kernels.rmsnorm_quant(x2, self._weight_bf16(x.device), self.eps, input_scale=input_scale, residual=res)
        return QuantizedActivation(xq.view(*x.shape[:-1], x.shape[-1]), input_scale), (res.view(x.shape) if res is not None else None)
