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
