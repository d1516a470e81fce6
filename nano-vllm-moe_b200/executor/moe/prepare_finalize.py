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


class FixedCapacityAllToAllPrepareFinalize:
    """Expert parallel without host round trips: every rank sends every other rank a block of exactly
    ``capacity`` row slots (rows for that rank first, padding after), so all split sizes are known
    when the call is made, nothing is read back to the host, and the whole dispatch -> experts ->
    combine sequence can be captured in a CUDA graph.  This is the step the reference leaves open
    (todo.md:48; torch_alltoall.py:11-12 marks its own exchange as not graph-capturable because of the
    ``.tolist()`` split sizes).

    Padding slots carry local expert id -1: the expert kernels skip ids outside the local range and
    leave those output rows zero.  ``capacity`` defaults to all ``T * k`` routed rows of the sending
    rank, which can never overflow; a smaller ``capacity_factor`` (slots = factor * T * k / ep_size,
    rounded up) moves fewer bytes, and rows that do not fit are dropped (they add zero); the number of
    dropped rows of the last call is kept on the device in ``last_overflow`` for the caller to inspect
    outside the hot path.
    """
    supports_cuda_graph = True
    uses_dynamic_alltoall = False

    def __init__(self, parallel_config: MoEParallelConfig, capacity_factor: float | None = None) -> None:
        if parallel_config.ep_size <= 1:
            raise ValueError("FixedCapacityAllToAllPrepareFinalize requires ep_size > 1")
        if capacity_factor is not None and capacity_factor <= 0:
            raise ValueError("capacity_factor must be positive")
        self.parallel_config = parallel_config
        self.capacity_factor = capacity_factor
        self.last_overflow: torch.Tensor | None = None

    def capacity(self, routed_rows: int) -> int:
        if self.capacity_factor is None:
            return routed_rows
        ep = self.parallel_config.ep_size
        return max(1, min(routed_rows, -(-int(self.capacity_factor * routed_rows) // ep)))

    def prepare(self, x, topk_weights, topk_ids) -> PrepareResult:
        cfg = self.parallel_config
        ep, dev = cfg.ep_size, x.device
        top_k = topk_ids.shape[-1]
        rows = topk_ids.numel()
        cap = self.capacity(rows)
        flat_ids = topk_ids.reshape(-1).to(torch.long)
        target = torch.div(flat_ids, cfg.local_num_experts, rounding_mode="floor").clamp_(0, ep - 1)
        perm = torch.argsort(target, stable=True)                       # routed rows grouped by destination rank
        tgt_sorted = target[perm]
        counts = (tgt_sorted[:, None] == torch.arange(ep, device=dev)[None, :]).sum(dim=0)      # no host sync
        starts = torch.cumsum(counts, 0) - counts
        pos = torch.arange(rows, device=dev) - starts[tgt_sorted]       # position inside the destination's block
        fits = pos < cap
        self.last_overflow = (~fits).sum()
        slot = torch.where(fits, tgt_sorted * cap + pos, torch.full_like(pos, ep * cap))      # overflow -> spill row
        send_x = torch.zeros((ep * cap + 1, x.shape[1]), dtype=x.dtype, device=dev)
        send_ids = torch.full((ep * cap + 1,), -1, dtype=torch.long, device=dev)
        send_w = torch.zeros((ep * cap + 1,), dtype=torch.float32, device=dev)
        send_x[slot] = x[torch.div(perm, top_k, rounding_mode="floor")]
        send_ids[slot] = (flat_ids % cfg.local_num_experts)[perm]
        send_w[slot] = topk_weights.reshape(-1).to(torch.float32)[perm]
        send_ids[ep * cap:].fill_(-1)                                    # whatever overflowed into the spill row is padding
        recv_x = torch.empty((ep * cap, x.shape[1]), dtype=x.dtype, device=dev)
        recv_ids = torch.empty((ep * cap,), dtype=torch.long, device=dev)
        recv_w = torch.empty((ep * cap,), dtype=torch.float32, device=dev)
        dist.all_to_all_single(recv_x, send_x[: ep * cap], group=cfg.ep_group)           # equal splits: cap rows per rank
        dist.all_to_all_single(recv_ids, send_ids[: ep * cap], group=cfg.ep_group)
        dist.all_to_all_single(recv_w, send_w[: ep * cap], group=cfg.ep_group)
        return PrepareResult(recv_x, recv_ids, recv_w, {"top_k": top_k, "x_div": 1, "perm": perm, "slot": slot, "fits": fits,
                                                         "cap": cap})

    def finalize(self, expert_out, prepared, *, output_shape, model_dtype, reduce_tp=True):
        cfg = self.parallel_config
        tokens, hidden = output_shape
        ctx = prepared.ctx
        ep, cap = cfg.ep_size, ctx["cap"]
        back = torch.zeros((ep * cap + 1, hidden), dtype=model_dtype, device=expert_out.device)     # last row: zeros for dropped rows
        dist.all_to_all_single(back[: ep * cap], expert_out.to(model_dtype).contiguous(), group=cfg.ep_group)
        routed = torch.empty((tokens * ctx["top_k"], hidden), dtype=model_dtype, device=expert_out.device)
        routed[ctx["perm"]] = back[ctx["slot"]]
        out = _sum_over_slots(routed, tokens, ctx["top_k"], hidden, model_dtype)
        if reduce_tp and cfg.tp_size > 1:
            dist.all_reduce(out, group=cfg.tp_group)
        return out
