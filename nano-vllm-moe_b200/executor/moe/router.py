"""Softmax top-k router (reference: executor/moe/router.py:9-34), on the CUDA router kernel."""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch

from ... import _lib
from ...quantization.kernels import _stream_ptr


class MoERouter(ABC):
    @abstractmethod
    def select_experts(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        ...


class SoftmaxTopKRouter(MoERouter):
    def __init__(self, top_k: int, renormalize: bool) -> None:
        self.top_k = top_k
        self.renormalize = renormalize

    def select_experts(self, hidden_states, router_logits):
        """-> (weights float32 [T, k], expert ids int64 [T, k]); softmax in fp32 over all experts, then top-k."""
        del hidden_states
        if not router_logits.is_cuda:
            raise ValueError("the router kernel needs CUDA tensors (there is no CPU path)")
        if router_logits.dim() != 2 or router_logits.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("router_logits must be [T, E] float32 or bfloat16")
        logits = router_logits if router_logits.stride(1) == 1 else router_logits.contiguous()
        t, e = logits.shape
        w = torch.empty((t, self.top_k), dtype=torch.float32, device=logits.device)
        ids = torch.empty((t, self.top_k), dtype=torch.int32, device=logits.device)
        with torch.cuda.device(logits.device):
            rc = _lib.load().fp8lin_moe_route(logits.data_ptr(), 1 if logits.dtype == torch.bfloat16 else 0,
                                              logits.stride(0), t, e, self.top_k, int(self.renormalize),
                                              w.data_ptr(), ids.data_ptr(), _stream_ptr(logits.device))
        _lib.raise_for(rc, "fp8lin_moe_route")
        return w, ids.to(torch.int64)
