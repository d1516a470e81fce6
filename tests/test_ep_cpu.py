"""Expert-parallel dispatch/combine on CPU ranks (gloo, world size 2), checked against a closed
form, the way the reference's own microbench does it
(scripts/moe/ep_prepare_finalize_microbench.py:73-96): the expert computation is replaced by
out = x * (local_id + 1) + rank_offset so the expected combined result can be written down."""
import importlib
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, routing, result_dir, flavour="dynamic"):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    moe = importlib.import_module("nano-vllm-moe_b200.executor.moe")
    E, k, T, H = 8, 2, 12, 16
    cfg = moe.make_moe_parallel_config(tp_group=None, ep_group=dist.group.WORLD, global_num_experts=E, intermediate_size=32)
    assert cfg.local_num_experts == E // world and cfg.ep_rank == rank
    if flavour == "dynamic":
        pf = moe.TorchAllToAllPrepareFinalize(cfg)
    elif flavour == "fixed":
        pf = moe.FixedCapacityAllToAllPrepareFinalize(cfg)
    else:                                                  # tight capacity: rows that do not fit are dropped
        pf = moe.FixedCapacityAllToAllPrepareFinalize(cfg, capacity_factor=1.0)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn((T, H), generator=g)
    if routing == "balanced":
        ids = (torch.arange(T * k) % E).view(T, k)
    elif routing == "skewed":
        ids = torch.zeros((T, k), dtype=torch.long); ids[:, 1] = 1          # everything goes to rank 0
    else:
        ids = torch.randint(0, E, (T, k), generator=g)
    w = torch.rand((T, k), generator=g)
    prep = pf.prepare(x, w, ids)
    # every received row must belong to one of this rank's experts
    assert prep.topk_ids.numel() == prep.hidden_states.shape[0] == prep.topk_weights.numel()
    valid = prep.topk_ids >= 0
    if flavour == "dynamic":
        assert valid.all()
    else:
        assert prep.hidden_states.shape[0] == world * pf.capacity(T * k)           # fixed shapes, padding marked -1
        assert (prep.topk_ids[~valid] == -1).all()
    assert (prep.topk_ids[valid] < cfg.local_num_experts).all()
    local_out = prep.hidden_states * (prep.topk_ids[:, None].float() + 1.0) * prep.topk_weights[:, None] + 100.0 * rank
    local_out = torch.where(valid[:, None], local_out, torch.zeros_like(local_out))   # what the expert kernels do with id -1
    y = pf.finalize(local_out, prep, output_shape=(T, H), model_dtype=torch.float32, reduce_tp=False)
    owner = ids // cfg.local_num_experts
    local = ids % cfg.local_num_experts
    terms = x[:, None, :] * (local[..., None].float() + 1.0) * w[..., None] + 100.0 * owner[..., None].float()
    dropped = 0
    if flavour == "tight":
        # a routed row is kept iff fewer than `capacity` earlier routed rows of this rank go to the same owner
        cap = pf.capacity(T * k)
        flat_owner = owner.reshape(-1)
        seen = torch.zeros(world, dtype=torch.long)
        keep = torch.zeros(T * k, dtype=torch.bool)
        for r in range(T * k):
            keep[r] = seen[flat_owner[r]] < cap
            seen[flat_owner[r]] += 1
        terms = terms * keep.view(T, k, 1)
        dropped = int((~keep).sum())
        assert int(pf.last_overflow) == dropped
    elif flavour == "fixed":
        assert int(pf.last_overflow) == 0
    want = terms.sum(dim=1)
    np.save(Path(result_dir) / f"ok_{routing}_{rank}.npy", np.array([float((y - want).abs().max()), float(dropped)]))
    dist.destroy_process_group()


@pytest.mark.parametrize("flavour", ["dynamic", "fixed", "tight"])
@pytest.mark.parametrize("routing", ["balanced", "skewed", "random"])
def test_alltoall_dispatch_combine_closed_form(tmp_path, routing, flavour):
    """dynamic = variable splits with host-side counts (the reference's exchange); fixed = fixed-capacity
    blocks, no host round trip; tight = the same with capacity for a balanced load only (skewed routing
    overflows and the dropped rows must be exactly the late ones)."""
    port = _free_port()
    mp.spawn(_worker, args=(2, port, routing, str(tmp_path), flavour), nprocs=2, join=True)
    dropped = 0.0
    for rank in range(2):
        err, d = np.load(tmp_path / f"ok_{routing}_{rank}.npy")
        assert err < 1e-5, (routing, flavour, rank, err)
        dropped += d
    if flavour == "tight" and routing == "skewed":
        assert dropped > 0


def _row_parallel_worker(rank, world, port, result_dir):
    """Row-parallel layer wiring on CPU ranks: shard shapes, bias on rank 0 only, all-reduce."""
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = importlib.import_module("nano-vllm-moe_b200")

    class Probe(pkg.QuantizeMethodBase):                    # stands in for the CUDA kernels on CPU
        def create_weights(self, layer, *, input_size_per_partition, output_partition_sizes, **kw):
            layer.register_buffer("w", torch.zeros(sum(output_partition_sizes), input_size_per_partition))

        def apply(self, layer, x, bias=None):
            y = x @ layer.w.t()
            return y + bias if bias is not None else y

    torch.manual_seed(0)
    full_w = torch.randn(6, 8); full_b = torch.randn(6); x = torch.randn(3, 8)
    row = pkg.RowParallelLinear(8, 6, bias=True, quant_method=Probe())
    assert (row.tp_size, row.tp_rank, row.input_size_per_partition) == (world, rank, 8 // world)
    row.w.copy_(full_w[:, rank * 4:(rank + 1) * 4])
    row.bias.weight_loader(row.bias, full_b)
    y = row(x[:, rank * 4:(rank + 1) * 4])
    col = pkg.ColumnParallelLinear(8, 6, bias=True, quant_method=Probe())
    col.w.copy_(full_w[rank * 3:(rank + 1) * 3]); col.bias.weight_loader(col.bias, full_b)
    yc = col(x)
    want = x @ full_w.t() + full_b
    np.save(Path(result_dir) / f"tp_{rank}.npy", np.array([float((y - want).abs().max()),
                                                            float((yc - want[:, rank * 3:(rank + 1) * 3]).abs().max())]))
    dist.destroy_process_group()


def test_row_and_column_parallel_on_two_cpu_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_row_parallel_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        errs = np.load(tmp_path / f"tp_{rank}.npy")
        assert errs.max() < 1e-5, (rank, errs)
