"""Two- and four-GPU tensor-parallel checks (skipped on boxes with fewer GPUs): a row-parallel W8A8 layer through
the NCCL all-reduce and through the peer-memory epilogue reduction, both against the oracle's
row-parallel restatement (bias on rank 0, per-rank bf16 partials, fp32 sum in rank order)."""
import importlib
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    from datetime import timedelta
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(seconds=90))
    from oracle import fp8_oracle as O
    pkg = importlib.import_module("nano-vllm-moe_b200")
    m, k, n = 650, 1024, 512            # ragged: the last rank's band of rows is shorter than the others'
    c = O.make_case(2468, m, k, n)
    with torch.device(dev):
        lay = pkg.RowParallelLinear(k, n, bias=True, quant_method=pkg.Fp8Config("fp8_w8a8_static").get_quant_method(None, "down"))
    lay.qweight.weight_loader(lay.qweight, torch.from_numpy(c["wq"]).to(dev))
    lay.weight_scale.weight_loader(lay.weight_scale, torch.from_numpy(c["w_scale"]).to(dev))
    lay.input_scale.weight_loader(lay.input_scale, torch.tensor(float(c["input_scale"])))
    lay.bias.data = torch.from_numpy(c["bias"]).to(dev, torch.bfloat16)
    pkg.process_weights_after_loading(lay)
    ks = k // world
    x = torch.from_numpy(np.ascontiguousarray(c["x"][:, rank * ks:(rank + 1) * ks])).to(dev, torch.bfloat16)
    lay.peer_reduce = False
    y_nccl = lay(x).float().cpu().numpy()
    lay.peer_reduce = True
    lay.peer_reduce_min_rows = 1
    y_peer1 = lay(x).float().cpu().numpy()
    y_peer2 = lay(x).float().cpu().numpy()          # second call reuses the slots
    lay.peer_reduce = "rs"                          # reduce-scatter in the epilogue + sum + all-gather by peer stores
    lay.peer_scatter = "epilogue"
    y_rs1 = lay(x).float().cpu().numpy()
    y_rs2 = lay(x).float().cpu().numpy()
    lay.defer_gather = True                         # sum + all-gather on a side stream; the caller joins before reading
    y_def = lay(x)
    lay.wait_reduce()
    y_def1 = y_def.float().cpu().numpy()
    y_def = lay(x)                                  # (the next call waits for the previous gather by itself)
    lay.wait_reduce()
    y_def2 = y_def.float().cpu().numpy()
    lay.peer_scatter = "copy"                       # the bands travel by copy engine instead of the GEMM's stores
    y_cp = lay(x)
    lay.wait_reduce()
    y_cp1 = y_cp.float().cpu().numpy()
    lay.defer_gather = False
    y_cp2 = lay(x).float().cpu().numpy()
    lay.peer_scatter = "epilogue"
    lay.reduce_results = "scatter"                  # ... stopping after the sum: this rank's band of rows only
    y_band = lay(x).float().cpu().numpy()
    lay.reduce_results = True
    band = -(-(-(-m // world)) // 32) * 32
    torch.cuda.synchronize()
    ref = O.row_parallel(c["x"], c["wq"], c["w_scale"], c["input_scale"], c["bias"], world, "fp8_w8a8_static")
    np.savez(Path(out_dir) / f"r{rank}.npz", nccl=y_nccl, peer1=y_peer1, peer2=y_peer2, rs1=y_rs1, rs2=y_rs2, def1=y_def1, def2=y_def2, cp1=y_cp1, cp2=y_cp2, band=y_band,
             band_ref=ref[rank * band:(rank + 1) * band], ref=ref)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_row_parallel_nccl_and_peer_reduce(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    from oracle import fp8_oracle as O
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    outs = [np.load(tmp_path / f"r{rank}.npz") for rank in range(world)]
    for rank, d in enumerate(outs):
        for key in ("nccl", "peer1", "peer2", "rs1", "rs2"):
            ok, worst = O.check_close(d[key], d["ref"], ulps=float(world))     # one bf16 rounding per rank's partial
            assert ok, (rank, key, worst)
        np.testing.assert_array_equal(d["peer1"], d["peer2"])
        np.testing.assert_array_equal(d["rs1"], d["rs2"])
        np.testing.assert_array_equal(d["rs1"], d["peer1"])                    # same partials, same order of the sum
        np.testing.assert_array_equal(d["def1"], d["rs1"])
        np.testing.assert_array_equal(d["def2"], d["rs1"])
        np.testing.assert_array_equal(d["cp1"], d["cp2"])
        ok, worst = O.check_close(d["cp1"], d["ref"], ulps=float(world))       # (another GEMM route: same values to the accumulation order)
        assert ok, (rank, "copy", worst)
        assert d["band"].shape == d["band_ref"].shape
        ok, worst = O.check_close(d["band"], d["band_ref"], ulps=float(world))
        assert ok, (rank, "band", worst)
        np.testing.assert_array_equal(outs[0]["peer1"], d["peer1"])            # every rank ends with the same bits


def _ep_worker(rank, world, port, out_dir):
    """Expert parallel on real kernels: the variable-split exchange, the fixed-capacity exchange (eager and
    replayed from a CUDA graph) and, on the same tokens, one rank holding every expert must agree bit for bit
    (a routed row's arithmetic does not depend on which rank or position it is computed at)."""
    import torch.distributed as dist
    from datetime import timedelta
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(seconds=90))
    moe = importlib.import_module("nano-vllm-moe_b200.executor.moe")
    E, K, T, H, I = 8, 2, 96, 256, 128
    g = torch.Generator(device=dev).manual_seed(77)                      # the same full expert set on every rank
    def codes(*shape):
        w = torch.randn(shape, generator=g, device=dev) * 0.05
        s = w.abs().amax(dim=-1).clamp(min=1e-8) / 448.0
        return (w / s[..., None]).to(torch.float8_e4m3fn).view(torch.uint8), s
    q13, s13 = codes(E, 2 * I, H)
    q2, s2 = codes(E, H, I)
    in13, in2 = torch.tensor(4.0 / 448.0), torch.tensor(2.0 / 448.0)
    gr = torch.Generator(device=dev).manual_seed(1000 + rank)            # every rank brings its own tokens
    x = torch.randn((T, H), generator=gr, device=dev).to(torch.bfloat16)
    ids = torch.randint(0, E, (T, K), generator=gr, device=dev)
    w = torch.rand((T, K), generator=gr, device=dev)
    full_cfg = moe.make_moe_parallel_config(tp_group=None, ep_group=None, global_num_experts=E, intermediate_size=I)
    full = moe.MoEKernel(prepare_finalize=moe.NoEPPrepareFinalize(full_cfg), experts=moe.Fp8Experts(), parallel_config=full_cfg)
    y_full = full(x, w, ids, moe.Fp8ExpertWeights.from_checkpoint_layout(q13, s13, in13, q2, s2, in2), model_dtype=torch.bfloat16)
    cfg = moe.make_moe_parallel_config(tp_group=None, ep_group=dist.group.WORLD, global_num_experts=E, intermediate_size=I)
    el = cfg.local_num_experts
    mine = slice(rank * el, (rank + 1) * el)
    wts = moe.Fp8ExpertWeights.from_checkpoint_layout(q13[mine], s13[mine], in13, q2[mine], s2[mine], in2)
    outs = {"full": y_full}
    for name, pf in (("dynamic", moe.TorchAllToAllPrepareFinalize(cfg)), ("fixed", moe.FixedCapacityAllToAllPrepareFinalize(cfg))):
        kern = moe.MoEKernel(prepare_finalize=pf, experts=moe.Fp8Experts(), parallel_config=cfg)
        outs[name] = kern(x, w, ids, wts, model_dtype=torch.bfloat16)
        if name == "fixed":
            torch.cuda.synchronize()
            side = torch.cuda.Stream(dev)
            gph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                kern(x, w, ids, wts, model_dtype=torch.bfloat16)
                torch.cuda.synchronize()
                with torch.cuda.graph(gph, stream=side):
                    y_graph = kern(x, w, ids, wts, model_dtype=torch.bfloat16)
            gph.replay()
            torch.cuda.synchronize()
            outs["fixed_graph"] = y_graph.clone()
            assert int(pf.last_overflow) == 0
            del gph
    torch.cuda.synchronize()
    np.savez(Path(out_dir) / f"ep{rank}.npz", **{k: v.float().cpu().numpy() for k, v in outs.items()})
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_exchanges_agree_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_ep_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        d = np.load(tmp_path / f"ep{rank}.npz")
        assert np.abs(d["full"]).max() > 0
        for key in ("dynamic", "fixed", "fixed_graph"):
            np.testing.assert_array_equal(d[key], d["full"], err_msg=f"rank {rank} {key}")


def _ep_tp_worker(rank, world, port, out_dir):
    """EP 2 x TP 2 on four GPUs: experts split over the EP group, every expert's intermediate dimension over the TP
    group; a single rank holding everything is the comparison (different roundings: each TP rank rounds its own
    partial down projection, so the bound is looser than bit equality)."""
    import torch.distributed as dist
    from datetime import timedelta
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(seconds=90))
    moe = importlib.import_module("nano-vllm-moe_b200.executor.moe")
    tp_group, ep_group = moe.make_ep_tp_groups(2)
    E, K, T, H, I = 6, 2, 80, 256, 1408                                  # I / 2 = 704: not a multiple of 128
    g = torch.Generator(device=dev).manual_seed(78)                      # the same full expert set on every rank
    def codes(*shape):
        w = torch.randn(shape, generator=g, device=dev) * 0.05
        s = w.abs().amax(dim=-1).clamp(min=1e-8) / 448.0
        return (w / s[..., None]).to(torch.float8_e4m3fn).view(torch.uint8), s
    q13, s13 = codes(E, 2 * I, H)
    q2, s2 = codes(E, H, I)
    in13, in2 = torch.tensor(4.0 / 448.0), torch.tensor(2.0 / 448.0)
    cfg = moe.make_moe_parallel_config(tp_group=tp_group, ep_group=ep_group, global_num_experts=E, intermediate_size=I)
    gr = torch.Generator(device=dev).manual_seed(2000 + cfg.ep_rank)     # the ranks of a TP group share their tokens
    x = torch.randn((T, H), generator=gr, device=dev).to(torch.bfloat16)
    ids = torch.randint(0, E, (T, K), generator=gr, device=dev)
    w = torch.rand((T, K), generator=gr, device=dev)
    full_cfg = moe.make_moe_parallel_config(tp_group=None, ep_group=None, global_num_experts=E, intermediate_size=I)
    full = moe.MoEKernel(prepare_finalize=moe.NoEPPrepareFinalize(full_cfg), experts=moe.Fp8Experts(), parallel_config=full_cfg)
    y_full = full(x, w, ids, moe.Fp8ExpertWeights.from_checkpoint_layout(q13, s13, in13, q2, s2, in2), model_dtype=torch.bfloat16)
    el = cfg.local_num_experts
    mine = slice(cfg.ep_rank * el, (cfg.ep_rank + 1) * el)
    wts = moe.Fp8ExpertWeights.from_checkpoint_layout(q13[mine], s13[mine], in13, q2[mine], s2[mine], in2,
                                                      tp_rank=cfg.tp_rank, tp_size=cfg.tp_size)
    assert wts.inter_size == I // 2
    outs = {"full": y_full}
    for name, pf in (("dynamic", moe.TorchAllToAllPrepareFinalize(cfg)), ("fixed", moe.FixedCapacityAllToAllPrepareFinalize(cfg))):
        kern = moe.MoEKernel(prepare_finalize=pf, experts=moe.Fp8Experts(), parallel_config=cfg)
        outs[name] = kern(x, w, ids, wts, model_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    np.savez(Path(out_dir) / f"eptp{rank}.npz", **{k: v.float().cpu().numpy() for k, v in outs.items()})
    dist.barrier()
    dist.destroy_process_group()


def test_expert_parallel_times_tensor_parallel_on_four_gpus(tmp_path):
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    import torch.multiprocessing as mp
    from oracle import fp8_oracle as O
    mp.spawn(_ep_tp_worker, args=(4, _free_port(), str(tmp_path)), nprocs=4, join=True)
    outs = [np.load(tmp_path / f"eptp{rank}.npz") for rank in range(4)]
    for rank, d in enumerate(outs):
        assert np.abs(d["full"]).max() > 0
        np.testing.assert_array_equal(d["dynamic"], d["fixed"])
        ok, worst = O.check_close(d["fixed"], d["full"], ulps=4.0)      # two partial down projections, each rounded, then summed
        assert ok and O.cosine(d["fixed"], d["full"]) > 0.9999, (rank, worst)
    np.testing.assert_array_equal(outs[0]["fixed"], outs[1]["fixed"])    # the two ranks of a TP group end with the same bits
    np.testing.assert_array_equal(outs[2]["fixed"], outs[3]["fixed"])
