"""Shared pieces of the GPU parity tests: seeded cases, device upload, comparison."""
import importlib

import numpy as np
import torch

from oracle import fp8_oracle as O

K = None


def kernels():
    global K
    if K is None:
        K = importlib.import_module("nano-vllm-moe_b200.quantization.kernels")
    return K


def to_bf16_cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).cuda()


def from_bf16(t):
    return t.detach().float().cpu().numpy()


def upload_case(c):
    d = {
        "x": to_bf16_cuda(c["x"]),
        "w_nk": kernels().pack_weight_nk(torch.from_numpy(c["wq"]).cuda()),
        "w_scale": torch.from_numpy(c["w_scale"]).cuda(),
        "bias": to_bf16_cuda(c["bias"]) if c.get("bias") is not None else None,
        "input_scale": torch.tensor(float(c["input_scale"]), dtype=torch.float32, device="cuda"),
    }
    return d


def run_linear(scheme, d, bias=True):
    Kn = kernels()
    b = d["bias"] if bias else None
    if scheme == "fp8_w8a16":
        return from_bf16(Kn.launch_w8a16_gemm(d["x"], d["w_nk"], d["w_scale"], b))
    return from_bf16(Kn.launch_w8a8_gemm(d["x"], d["w_nk"], d["input_scale"], d["w_scale"], b))


def oracle_linear(scheme, c, bias=True, rows=None, exact=False):
    x = c["x"] if rows is None else c["x"][rows]
    b = c["bias"] if bias else None
    if scheme == "fp8_w8a16":
        return O.linear_w8a16(x, c["wq"], c["w_scale"], b, exact=exact)
    return O.linear_w8a8(x, c["wq"], c["w_scale"], c["input_scale"], b, exact=exact)


def assert_parity(y, ref, what, ulps=1.0, min_cos=0.99999):
    assert y.shape == ref.shape, (what, y.shape, ref.shape)
    assert np.isfinite(y).all(), what
    ok, worst = O.check_close(y, ref, ulps=ulps)
    cos = O.cosine(y, ref)
    assert ok and cos >= min_cos, f"{what}: worst tolerance ratio {worst:.3f}, cosine {cos:.7f}"
