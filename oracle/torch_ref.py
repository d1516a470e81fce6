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
