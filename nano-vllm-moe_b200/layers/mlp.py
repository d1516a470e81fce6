"""The MLP block of the reference's dense models as one fused call.

``Qwen2MLP.forward`` (nanovllm/models/qwen2.py:110-114) runs ``gate_up_proj`` ->
``SiluAndMul`` (nanovllm/layers/activation.py:11-14) -> ``down_proj``.  With both projections
on the W8A8-static scheme this module replaces the three steps by ``fp8lin_mlp_w8a8``: the
gate_up GEMM's epilogue computes ``silu(gate) * up`` and quantises it for the down projection,
so the bf16 gate_up tensor is neither written nor read back (more than 64 rows), and the down
GEMM starts from e4m3 rows.  Results carry the same roundings as the three separate steps.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from ..quantization import kernels
from .linear import MergedColumnParallelLinear, RowParallelLinear


class FusedFp8MLP(nn.Module):
    """Wraps an already loaded and processed (gate_up_proj, down_proj) pair.

    ``release_unfused=True`` drops the gate_up layer's own packed weight after the interleaved copy
    is made (the layer can then no longer be called on its own).
    """

    def __init__(self, gate_up_proj: MergedColumnParallelLinear, down_proj: RowParallelLinear, release_unfused: bool = False):
        super().__init__()
        if getattr(gate_up_proj, "_fp8_backend", None) != "fp8lin_w8a8" or getattr(down_proj, "_fp8_backend", None) != "fp8lin_w8a8":
            raise ValueError("FusedFp8MLP needs both projections on the fp8_w8a8_static scheme, after process_weights_after_loading")
        if len(gate_up_proj.output_sizes) != 2 or gate_up_proj.output_sizes[0] != gate_up_proj.output_sizes[1]:
            raise ValueError("gate_up_proj must merge two equally sized projections")
        inter = gate_up_proj.output_size_per_partition // 2
        if inter != down_proj.input_size_per_partition:
            raise ValueError("gate_up_proj and down_proj disagree on the intermediate size")
        if inter % 128:
            raise ValueError(f"the per-rank intermediate size must be a multiple of 128 (got {inter})")
        self.gate_up_proj = gate_up_proj
        self.down_proj = down_proj
        self.inter = inter
        gu_bias = getattr(gate_up_proj, "bias", None)
        w, s, b = kernels.interleave_gate_up(gate_up_proj.qweight_packed, gate_up_proj.weight_scale,
                                             gu_bias.detach().to(torch.bfloat16) if gu_bias is not None else None, inter)
        self.register_buffer("gate_up_packed", w, persistent=False)
        self.register_buffer("gate_up_scale", s, persistent=False)
        self.gate_up_bias = b
        if release_unfused:
            gate_up_proj.qweight_packed = torch.empty((0,), dtype=torch.uint8, device=w.device)

    def forward(self, x) -> torch.Tensor:
        """``x``: bfloat16 [.., H], or a ``QuantizedActivation`` made with gate_up_proj's input scale."""
        codes = getattr(x, "codes", None)
        if codes is not None:
            x = codes
        if not x.is_cuda:
            raise RuntimeError("FP8 W8A8 static requires CUDA")
        down = self.down_proj
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        bias = down.bias if (getattr(down, "bias", None) is not None and down.tp_rank == 0) else None   # as layers/linear.py:259
        y = kernels.launch_mlp_w8a8(x2, self.gate_up_packed, self.gate_up_scale, self.gate_up_proj.input_scale, self.gate_up_bias,
                                    down.qweight_packed, down.weight_scale, down.input_scale, bias)
        if down.tp_size > 1 and down.reduce_results:
            dist.all_reduce(y, group=down.tp_group)
        return y.reshape(*lead, y.shape[-1])
