"""prepare -> experts -> finalize (reference: executor/moe/kernel.py:14-78)."""
from __future__ import annotations

import torch

from .config import MoEParallelConfig
from .experts import Fp8Experts, Fp8ExpertWeights


class MoEKernel:
    def __init__(self, *, prepare_finalize, experts: Fp8Experts, parallel_config: MoEParallelConfig) -> None:
        self.prepare_finalize = prepare_finalize
        self.experts = experts
        self.parallel_config = parallel_config

    def __call__(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, weights: Fp8ExpertWeights,
                 *, model_dtype: torch.dtype, reduce_tp: bool = True) -> torch.Tensor:
        prepared = self.prepare_finalize.prepare(x, topk_weights, topk_ids)
        local = self.experts.apply(prepared.hidden_states, prepared.topk_ids, prepared.topk_weights, weights,
                                   x_div=prepared.ctx.get("x_div", 1))
        return self.prepare_finalize.finalize(local, prepared, output_shape=(x.shape[0], x.shape[1]),
                                              model_dtype=model_dtype, reduce_tp=reduce_tp)
