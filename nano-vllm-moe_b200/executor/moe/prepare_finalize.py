"""Dispatch of routed rows to the ranks that own their experts, and the combine on the way back
(reference: executor/moe/prepare_finalize/{base,no_ep,torch_alltoall}.py)."""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from .config import MoEParallelConfig


@dataclass
class PrepareResult:
    hidden_states: torch.Tensor     # rows the local experts will process
    topk_ids: torch.Tensor          # LOCAL expert id per row
    topk_weights: torch.Tensor      # routing weight per row
    ctx: dict = field(default_factory=dict)


def _sum_over_slots(rows: torch.Tensor, tokens: int, top_k: int, hidden: int, dtype: torch.dtype) -> torch.Tensor:
    """[T*k, H] in routed-row order -> [T, H]; CUDA bf16 goes through the combine kernel."""
    if rows.is_cuda and dtype == torch.bfloat16 and hidden % 8 == 0:
        from ... import _lib
        from ...quantization.kernels import _stream_ptr
        rows = rows.to(torch.bfloat16).contiguous()
        y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=rows.device)
        with torch.cuda.device(rows.device):
            rc = _lib.load().fp8lin_moe_combine(rows.data_ptr(), y.data_ptr(), tokens, top_k, hidden, _stream_ptr(rows.device))
        _lib.raise_for(rc, "fp8lin_moe_combine")
        return y
    return rows.to(dtype).view(tokens, top_k, hidden).sum(dim=1)


class NoEPPrepareFinalize:
    """All experts are local: nothing moves.  Unlike the reference (no_ep.py:27) the token rows are
    not expanded k times; the experts kernel reads row ``r // k`` of x for routed row r."""
    supports_cuda_graph = True
    uses_dynamic_alltoall = False

    def __init__(self, parallel_config: MoEParallelConfig) -> None:
        if parallel_config.ep_size != 1:
            raise ValueError("NoEPPrepareFinalize requires ep_size == 1")
        self.parallel_config = parallel_config

    def prepare(self, x, topk_weights, topk_ids) -> PrepareResult:
        top_k = topk_ids.shape[-1]
        return PrepareResult(x, topk_ids.reshape(-1), topk_weights.reshape(-1), {"top_k": top_k, "x_div": top_k})

    def finalize(self, expert_out, prepared, *, output_shape, model_dtype, reduce_tp=True):
        tokens, hidden = output_shape
        out = _sum_over_slots(expert_out, tokens, prepared.ctx["top_k"], hidden, model_dtype)
        if reduce_tp and self.parallel_config.tp_size > 1:
            dist.all_reduce(out, group=self.parallel_config.tp_group)
        return out


class TorchAllToAllPrepareFinalize:
    """Expert parallel: routed rows are sorted by owning rank (expert id // experts per rank),
    exchanged with variable-split all-to-alls (counts first, then rows, local ids and weights),
    processed by the local experts, sent back and summed over the k slots
    (reference: prepare_finalize/torch_alltoall.py:19-93; the sort here is stable)."""
    supports_cuda_graph = False
    uses_dynamic_alltoall = True

    def __init__(self, parallel_config: MoEParallelConfig) -> None:
        if parallel_config.ep_size <= 1:
            raise ValueError("TorchAllToAllPrepareFinalize requires ep_size > 1")
        self.parallel_config = parallel_config

    def prepare(self, x, topk_weights, topk_ids) -> PrepareResult:
        cfg = self.parallel_config
        top_k = topk_ids.shape[-1]
        flat_ids = topk_ids.reshape(-1).to(torch.long)
        target = torch.div(flat_ids, cfg.local_num_experts, rounding_mode="floor").clamp_(0, cfg.ep_size - 1)
        perm = torch.argsort(target, stable=True)
        send_x = x.repeat_interleave(top_k, dim=0)[perm]
        send_ids = (flat_ids % cfg.local_num_experts)[perm]
        send_w = topk_weights.reshape(-1).to(torch.float32)[perm]
        send_counts = torch.bincount(target, minlength=cfg.ep_size).to(torch.long)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=cfg.ep_group)
        s_list, r_list = send_counts.tolist(), recv_counts.tolist()
        n_recv = int(sum(r_list))
        recv_x = torch.empty((n_recv, x.shape[1]), dtype=x.dtype, device=x.device)
        recv_ids = torch.empty((n_recv,), dtype=torch.long, device=x.device)
        recv_w = torch.empty((n_recv,), dtype=torch.float32, device=x.device)
        dist.all_to_all_single(recv_x, send_x, r_list, s_list, group=cfg.ep_group)
        dist.all_to_all_single(recv_ids, send_ids, r_list, s_list, group=cfg.ep_group)
        dist.all_to_all_single(recv_w, send_w, r_list, s_list, group=cfg.ep_group)
        return PrepareResult(recv_x, recv_ids, recv_w,
                             {"top_k": top_k, "x_div": 1, "perm": perm, "s_list": s_list, "r_list": r_list})

    def finalize(self, expert_out, prepared, *, output_shape, model_dtype, reduce_tp=True):
        cfg = self.parallel_config
        tokens, hidden = output_shape
        ctx = prepared.ctx
        back = torch.empty((tokens * ctx["top_k"], hidden), dtype=model_dtype, device=expert_out.device)
        dist.all_to_all_single(back, expert_out.to(model_dtype).contiguous(), ctx["s_list"], ctx["r_list"], group=cfg.ep_group)
        routed = torch.empty_like(back)
        routed[ctx["perm"]] = back
        out = _sum_over_slots(routed, tokens, ctx["top_k"], hidden, model_dtype)
        if reduce_tp and cfg.tp_size > 1:
            dist.all_reduce(out, group=cfg.tp_group)
        return out
