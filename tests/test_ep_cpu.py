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


def _ep_tp_worker(rank, world, port, result_dir):
    """EP 2 x TP 2 on four CPU ranks: the two ranks of a TP group hold the same tokens and the same experts, each
    contributes a share of every expert's output (standing in for its slice of the intermediate dimension), and
    finalize adds the shares with the TP all-reduce (prepare_finalize/torch_alltoall.py:92 of the reference)."""
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    moe = importlib.import_module("nano-vllm-moe_b200.executor.moe")
    tp_group, ep_group = moe.make_ep_tp_groups(2)
    E, k, T, H = 6, 2, 10, 8
    cfg = moe.make_moe_parallel_config(tp_group=tp_group, ep_group=ep_group, global_num_experts=E, intermediate_size=1408)
    assert (cfg.tp_size, cfg.ep_size, cfg.local_num_experts, cfg.local_inter_size) == (2, 2, 3, 704)
    assert (cfg.ep_rank, cfg.tp_rank) == (rank // 2, rank % 2)
    errs = []
    for pf in (moe.TorchAllToAllPrepareFinalize(cfg), moe.FixedCapacityAllToAllPrepareFinalize(cfg)):
        g = torch.Generator().manual_seed(500 + cfg.ep_rank)           # the ranks of a TP group see the same tokens
        x = torch.randn((T, H), generator=g)
        ids = torch.randint(0, E, (T, k), generator=g)
        w = torch.rand((T, k), generator=g)
        prep = pf.prepare(x, w, ids)
        valid = prep.topk_ids >= 0
        share = 0.25 if cfg.tp_rank == 0 else 0.75                     # this TP rank's part of the expert output
        local_out = prep.hidden_states * (prep.topk_ids[:, None].float() + 1.0) * prep.topk_weights[:, None] * share
        local_out = torch.where(valid[:, None], local_out, torch.zeros_like(local_out))
        y = pf.finalize(local_out, prep, output_shape=(T, H), model_dtype=torch.float32, reduce_tp=True)
        local = ids % cfg.local_num_experts
        want = (x[:, None, :] * (local[..., None].float() + 1.0) * w[..., None]).sum(dim=1)
        errs.append(float((y - want).abs().max()))
        y_half = pf.finalize(local_out, prep, output_shape=(T, H), model_dtype=torch.float32, reduce_tp=False)
        errs.append(float((y_half - want * share).abs().max()))
    np.save(Path(result_dir) / f"eptp_{rank}.npy", np.array(errs))
    dist.destroy_process_group()


def test_expert_parallel_times_tensor_parallel_on_four_cpu_ranks(tmp_path):
    mp.spawn(_ep_tp_worker, args=(4, _free_port(), str(tmp_path)), nprocs=4, join=True)
    for rank in range(4):
        assert np.load(tmp_path / f"eptp_{rank}.npy").max() < 1e-5, rank


def test_expert_weights_are_sliced_along_the_intermediate_dimension():
    """Fp8ExpertWeights.from_checkpoint_layout with a TP slice keeps gate and up rows of the slice and the matching
    columns of the down weight (checked through the slicing arithmetic alone: packing needs a GPU)."""
    exp = importlib.import_module("nano-vllm-moe_b200.executor.moe.experts")
    E, I, H = 2, 64, 32
    w13 = torch.arange(E * 2 * I * H, dtype=torch.int64).remainder(251).to(torch.uint8).view(E, 2 * I, H)
    s13 = torch.arange(E * 2 * I, dtype=torch.float32).view(E, 2 * I)
    w2 = torch.arange(E * H * I, dtype=torch.int64).remainder(241).to(torch.uint8).view(E, H, I)
    seen = {}

    def fake_pack(q):
        seen.setdefault("shapes", []).append(tuple(q.shape))
        seen.setdefault("first", []).append(q.clone())
        return q.reshape(-1)
    orig = exp.kernels.pack_weight_nk
    exp.kernels.pack_weight_nk = fake_pack
    try:
        wt = exp.Fp8ExpertWeights.from_checkpoint_layout(w13, s13, torch.tensor(1.0), w2, torch.ones(E, H), torch.tensor(1.0),
                                                         tp_rank=1, tp_size=2)
    finally:
        exp.kernels.pack_weight_nk = orig
    assert wt.inter_size == 32 and seen["shapes"] == [(64, H), (64, H), (H, 32), (H, 32)]
    assert torch.equal(seen["first"][0], torch.cat([w13[0, 32:64], w13[0, 96:128]]))
    assert torch.equal(seen["first"][2], w2[0, :, 32:64])
    assert torch.equal(wt.w13_scale[1], torch.cat([s13[1, 32:64], s13[1, 96:128]]))
    with pytest.raises(ValueError):
        exp.Fp8ExpertWeights.from_checkpoint_layout(w13, s13, torch.tensor(1.0), w2, torch.ones(E, H), torch.tensor(1.0), tp_rank=0, tp_size=8)


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
