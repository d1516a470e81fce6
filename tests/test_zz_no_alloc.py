"""fp8lin_linear_static_scratch: the entry point for callers that cannot allocate
device memory (a server whose KV-cache pool already owns all free HBM, or a
latency-critical loop that must not wait on an allocation).  It keeps its
split-K scratch in a fixed array inside the library instead of a caller's
workspace.  The test calls it through the C ABI, twice in a row on the same
shared array, and compares with the workspace-taking entry points and with the
CPU oracle (the first alone would be a weak check where both entry points run
the same kernel on different scratch).

This file is named so that pytest collects it last."""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as O
from helpers import assert_parity, from_bf16, kernels, oracle_linear, run_linear, upload_case

pytestmark = pytest.mark.gpu

# (M, K, N): a split-K shape, a no-split shape, a ragged one
SHAPES = [(16, 3584, 3584), (4, 2048, 11008), (33, 704, 72), (64, 18944, 3584)]


def _call(pkg, scheme_id, d, m, k, n, bias=True):
    lib = pkg._lib.load()
    y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    b = d["bias"] if bias else None
    rc = lib.fp8lin_linear_static_scratch(
        scheme_id, d["x"].data_ptr(), d["x"].stride(0), d["w_nk"].data_ptr(), d["w_scale"].data_ptr(),
        d["input_scale"].data_ptr(), b.data_ptr() if b is not None else None, y.data_ptr(), y.stride(0),
        m, k, n, torch.cuda.current_stream().cuda_stream)
    pkg._lib.raise_for(rc, "fp8lin_linear_static_scratch")
    torch.cuda.synchronize()
    return from_bf16(y)


@pytest.mark.parametrize("scheme", ["fp8_w8a8_static", "fp8_w8a16"])
def test_static_scratch_matches_workspace_entry_point(pkg, scheme):
    scheme_id = pkg._lib.W8A8_STATIC if scheme == "fp8_w8a8_static" else pkg._lib.W8A16
    for m, k, n in SHAPES:
        c = O.make_case(555 + m + n, m, k, n)
        d = upload_case(c)
        want = run_linear(scheme, d)                       # existing entry point, caller-owned workspace
        first = _call(pkg, scheme_id, d, m, k, n)
        second = _call(pkg, scheme_id, d, m, k, n)         # same array again, straight after
        assert_parity(first, want, f"static scratch {scheme} {m}x{k}x{n} (1st call)")
        assert_parity(second, want, f"static scratch {scheme} {m}x{k}x{n} (2nd call)")
        np.testing.assert_array_equal(first, second)
        assert_parity(first, oracle_linear(scheme, c), f"static scratch {scheme} {m}x{k}x{n} vs the oracle")
        del d


def test_static_scratch_refuses_what_does_not_fit(pkg):
    lib = pkg._lib.load()
    L = pkg._lib
    c = O.make_case(1, 2, 64, 16)
    d = upload_case(c)
    y = torch.empty((2, 16), dtype=torch.bfloat16, device="cuda")
    args = (d["x"].data_ptr(), 64, d["w_nk"].data_ptr(), d["w_scale"].data_ptr(), d["input_scale"].data_ptr(), None,
            y.data_ptr(), 16)
    assert lib.fp8lin_linear_static_scratch(L.W8A8_STATIC, *args, 65, 64, 16, None) == L.ERR_WORKSPACE
    assert "64 rows" in L.last_error()
    assert lib.fp8lin_linear_static_scratch(7, *args, 2, 64, 16, None) == L.ERR_ARG
    assert lib.fp8lin_linear_static_scratch(L.W8A8_STATIC, *args, 2, 40, 16, None) == L.ERR_SHAPE
    assert lib.fp8lin_linear_static_scratch(L.W8A8_STATIC, *args, 0, 64, 16, None) == L.OK
