"""The reference's own check formula, as a timed CPU baseline.  TEST INFRASTRUCTURE ONLY.

``torch.mm(x_bf16, Wq.to(bf16) * weight_scale.to(bf16))`` is what the
reference's microbenchmarks call the "BF16 dequant" path and compare every
FP8 kernel against (scripts/quantization/w8a16_linear_microbench.py:47-53,
scripts/quantization/fp8_linear_microbench.py:67,77).  It is executed here on
the host CPU with all cores; only ``bench.py`` (CPU-baseline leg and
``--impl reference``) and the tests use it.  Parity: pinned — the formula's
output on seeded inputs is stored in tests/golden/linear.npz (``rand_*_oref``)
and checked against the numpy oracle in tests/test_oracle_golden.py.
"""
from __future__ import annotations

import os
import time

import torch


def dequant_matmul(x_bf16: torch.Tensor, q_nk_u8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """x [M,K] bf16, q [N,K] uint8 e4m3 codes, scale [N] f32 -> [M,N] bf16 (dequantisation inside the call)."""
    w = q_nk_u8.view(torch.float8_e4m3fn).to(torch.bfloat16) * scale.to(torch.bfloat16).unsqueeze(1)
    return torch.mm(x_bf16, w.t())


def time_linears(ops, steps: int, warmup: int, budget_s: float, rows_cap: int = 256):
    """Time the reference's CPU formula on a bounded sample of a list of linears.

    ops = [(x [M,K] bf16, q_nk [N,K] uint8, scale [N] f32, full_rows)]: every x holds at most
    ``rows_cap`` of the ``full_rows`` rows the workload has; a linear's time is scaled by
    full_rows / M (a matmul's time is linear in its rows) and the scaled times are summed to one pass.
    Two figures per pass, as the reference's microbenchmarks report them: ``cached`` multiplies by a
    bf16 weight dequantised once outside the timed region (fp8_linear_microbench.py:67,77 -- weights
    as [K,N]), ``dequant`` dequantises inside every call (w8a16_linear_microbench.py:47-53).
    Returns {"cached": [seconds per pass], "dequant": [...], "threads": n}."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    prepared = []
    for x, q_nk, scale, full_rows in ops:
        q_kn = q_nk.t().contiguous()                                   # the reference's runtime layout [K,N]
        w_bf16 = q_kn.view(torch.float8_e4m3fn).to(torch.bfloat16) * scale.to(torch.bfloat16).unsqueeze(0)
        prepared.append((x, q_kn, scale, w_bf16, full_rows / max(x.shape[0], 1)))

    def one_pass(cached: bool) -> float:
        total = 0.0
        for x, q_kn, scale, w_bf16, factor in prepared:
            t0 = time.perf_counter()
            if cached:
                torch.mm(x, w_bf16)
            else:
                torch.mm(x, q_kn.view(torch.float8_e4m3fn).to(torch.bfloat16) * scale.to(torch.bfloat16).unsqueeze(0))
            total += (time.perf_counter() - t0) * factor
        return total

    out = {"cached": [], "dequant": [], "threads": torch.get_num_threads()}
    for _ in range(warmup):
        one_pass(True); one_pass(False)
    t_start = time.perf_counter()
    for _ in range(steps):
        out["cached"].append(one_pass(True))
        out["dequant"].append(one_pass(False))
        if time.perf_counter() - t_start > budget_s:
            break
    return out


def time_passes(tensors, steps: int, warmup: int, budget_s: float) -> tuple[list[float], int]:
    """Time ``steps`` passes over ``tensors`` = [(x, q_nk, scale), ...]; stops early when the
    wall-clock budget is spent.  Returns (seconds per pass, threads used)."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    for _ in range(warmup):
        for x, q, s in tensors:
            dequant_matmul(x, q, s)
    out = []
    t_start = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        for x, q, s in tensors:
            dequant_matmul(x, q, s)
        out.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    return out, torch.get_num_threads()


def eager_experts(x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """The reference's expert FFN as it runs it (bf16 dense experts, one python loop over experts;
    nanovllm/executor/moe/experts/eager_experts.py:26-35 + prepare_finalize/no_ep.py:19-45), on CPU.
    x [T,H] bf16; topk_ids/topk_w [T,k]; w13 [E,2I,H] bf16; w2 [E,H,I] bf16 -> [T,H] bf16."""
    import torch.nn.functional as F
    t, k = topk_ids.shape
    xe = x.repeat_interleave(k, dim=0)
    ids = topk_ids.reshape(-1)
    w = topk_w.reshape(-1)
    out = torch.zeros(xe.shape[0], w2.shape[1], dtype=x.dtype)
    for e in range(w13.shape[0]):
        idx = torch.nonzero(ids == e, as_tuple=False).flatten()
        if idx.numel() == 0:
            continue
        gate, up = F.linear(xe[idx], w13[e]).chunk(2, dim=-1)
        out[idx] = F.linear(F.silu(gate) * up, w2[e]) * w[idx, None].to(x.dtype)
    return out.view(t, k, -1).sum(dim=1)
