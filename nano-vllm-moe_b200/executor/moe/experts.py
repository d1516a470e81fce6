"""Local expert FFN on FP8 weights: one grouped tcgen05 GEMM per projection.

Counterpart of the reference's ``MoEExpertsKernel`` implementations
(experts/eager_experts.py, experts/optimized.py), which are bf16-only and ignore the
``w13_weight_scale`` / ``w2_weight_scale`` arguments; here the scales are used.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ... import _lib
from ...quantization import kernels


@dataclass
class Fp8ExpertWeights:
    """Packed expert weights of one MoE layer (this rank's experts)."""
    w13_packed: torch.Tensor        # uint8, E x packed(K=H, N=2I); rows [0,I) gate, [I,2I) up
    w13_scale: torch.Tensor         # float32 [E, 2I]
    w13_input_scale: torch.Tensor   # float32 scalar
    w2_packed: torch.Tensor         # uint8, E x packed(K=I, N=H)
    w2_scale: torch.Tensor          # float32 [E, H]
    w2_input_scale: torch.Tensor    # float32 scalar
    num_experts: int
    hidden_size: int
    inter_size: int

    @classmethod
    def from_checkpoint_layout(cls, w13_q: torch.Tensor, w13_scale: torch.Tensor, w13_input_scale: torch.Tensor,
                               w2_q: torch.Tensor, w2_scale: torch.Tensor, w2_input_scale: torch.Tensor,
                               tp_rank: int = 0, tp_size: int = 1) -> "Fp8ExpertWeights":
        """w13_q uint8 [E, 2I, H], w2_q uint8 [E, H, I] (the reference's stacked layout, blocks/base.py:58-63).
        With ``tp_size`` > 1 this rank keeps slice ``tp_rank`` of the intermediate dimension: gate rows and up rows
        [tp_rank * I/tp, (tp_rank + 1) * I/tp) of w13 with their scales, the matching columns of w2 (all of its
        output-channel scales), as the reference shards its expert weights (blocks/base.py:66-93,
        local_inter_size = I / tp); the ranks' outputs are summed by the TP all-reduce of ``finalize``."""
        e, two_i, h = w13_q.shape
        i = two_i // 2
        if tp_size > 1:
            if i % tp_size or (i // tp_size) % 16:
                raise ValueError(f"the intermediate size {i} must split into {tp_size} slices that are multiples of 16")
            il = i // tp_size
            lo, hi = tp_rank * il, (tp_rank + 1) * il
            w13_q = torch.cat([w13_q[:, lo:hi], w13_q[:, i + lo:i + hi]], dim=1).contiguous()
            w13_scale = torch.cat([w13_scale[:, lo:hi], w13_scale[:, i + lo:i + hi]], dim=1).contiguous()
            w2_q = w2_q[:, :, lo:hi].contiguous()
            i = il
        if w2_q.shape != (e, h, i):
            raise ValueError(f"w2 must be [E, H, I] = {(e, h, i)}, got {tuple(w2_q.shape)}")
        w13_p = torch.cat([kernels.pack_weight_nk(w13_q[x]) for x in range(e)])
        w2_p = torch.cat([kernels.pack_weight_nk(w2_q[x]) for x in range(e)])
        dev = w13_q.device
        return cls(w13_p, w13_scale.to(dev, torch.float32).contiguous(), w13_input_scale.to(dev, torch.float32).reshape(()),
                   w2_p, w2_scale.to(dev, torch.float32).contiguous(), w2_input_scale.to(dev, torch.float32).reshape(()),
                   e, h, i)


class Fp8Experts:
    """``apply`` keeps the reference's argument order (experts/base.py) with the packed weights
    in place of the dense w13 / w2 tensors."""

    def apply(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, weights: Fp8ExpertWeights,
              *, x_div: int = 1) -> torch.Tensor:
        """x [rows / x_div, H] bf16; topk_ids [rows] local expert per routed row; topk_weights [rows].
        Returns bf16 [rows, H]: routed row r = W2[e](silu_mul(W13[e](x[r // x_div]))) * weight."""
        if not x.is_cuda:
            raise ValueError("the expert kernels need CUDA tensors (there is no CPU path)")
        if x.dtype != torch.bfloat16:
            x = x.to(torch.bfloat16)
        if x.stride(1) != 1:
            x = x.contiguous()
        rows = topk_ids.numel()
        ids = topk_ids.reshape(-1).to(torch.int32).contiguous()
        w = topk_weights.reshape(-1).to(torch.float32).contiguous()
        wt = weights
        out = torch.zeros((rows, wt.hidden_size), dtype=torch.bfloat16, device=x.device)
        lib = _lib.load()
        with torch.cuda.device(x.device):
            need = int(lib.fp8lin_moe_workspace_bytes(rows, wt.num_experts, wt.hidden_size, wt.inter_size))
            ws = kernels.workspace(x.device, need)
            rc = lib.fp8lin_moe_experts_w8a8(
                x.data_ptr(), x.stride(0), x_div, ids.data_ptr(), w.data_ptr(), rows,
                wt.w13_packed.data_ptr(), wt.w13_scale.data_ptr(), wt.w13_input_scale.data_ptr(),
                wt.w2_packed.data_ptr(), wt.w2_scale.data_ptr(), wt.w2_input_scale.data_ptr(),
                wt.num_experts, wt.hidden_size, wt.inter_size, out.data_ptr(), out.stride(0),
                ws.data_ptr(), ws.numel(), kernels._stream_ptr(x.device))
        _lib.raise_for(rc, "fp8lin_moe_experts_w8a8")
        return out
