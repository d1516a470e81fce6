"""Expert/tensor-parallel layout of one MoE layer (reference: executor/moe/config.py:9-53)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch.distributed as dist


@dataclass(frozen=True)
class MoEParallelConfig:
    tp_group: Optional[dist.ProcessGroup]
    ep_group: Optional[dist.ProcessGroup]
    tp_size: int
    tp_rank: int
    ep_size: int
    ep_rank: int
    global_num_experts: int
    local_num_experts: int
    intermediate_size: int
    local_inter_size: int


def _size_rank(group) -> tuple[int, int]:
    return (dist.get_world_size(group), dist.get_rank(group)) if group is not None else (1, 0)


def make_moe_parallel_config(*, tp_group, ep_group, global_num_experts: int, intermediate_size: int) -> MoEParallelConfig:
    """Experts are split contiguously over the EP group, the intermediate dimension over the TP group."""
    tp_size, tp_rank = _size_rank(tp_group)
    ep_size, ep_rank = _size_rank(ep_group)
    if global_num_experts % ep_size:
        raise ValueError(f"global_num_experts={global_num_experts} must be divisible by ep_size={ep_size}")
    if intermediate_size % tp_size:
        raise ValueError(f"intermediate_size={intermediate_size} must be divisible by tp_size={tp_size}")
    return MoEParallelConfig(tp_group, ep_group, tp_size, tp_rank, ep_size, ep_rank, global_num_experts,
                             global_num_experts // ep_size, intermediate_size, intermediate_size // tp_size)


def make_ep_tp_groups(tp_size: int):
    """Process groups of an EP x TP layout over the default group: rank = ep_rank * tp_size + tp_rank, so the
    ranks that split one expert's intermediate dimension are neighbours and each EP group holds the ranks with the
    same tp_rank (the 8-GPU layout of 60 experts: EP 4 x TP 2, executor/moe/config.py:34-53 of the reference
    accepts it because 60 % 4 == 0 and 1408 % 2 == 0).  Every rank must call this (new_group is collective).
    Returns (tp_group, ep_group) of the calling rank; a group of size 1 is returned as None."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if tp_size < 1 or world % tp_size:
        raise ValueError(f"world size {world} is not a multiple of tp_size={tp_size}")
    ep_size = world // tp_size
    my_tp = my_ep = None
    for e in range(ep_size):
        ranks = [e * tp_size + t for t in range(tp_size)]
        g = dist.new_group(ranks) if tp_size > 1 else None
        if rank in ranks:
            my_tp = g
    for t in range(tp_size):
        ranks = [e * tp_size + t for e in range(ep_size)]
        g = dist.new_group(ranks) if ep_size > 1 else None
        if rank in ranks:
            my_ep = g
    return my_tp, my_ep
