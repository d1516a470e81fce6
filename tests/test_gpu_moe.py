"""MoE expert FFN on FP8 operands: router, grouped GEMMs, activation, combine -- against the oracle.

The reference's experts are bf16-only (its scale arguments are discarded,
experts/eager_experts.py:25), so the FP8 expert arithmetic is checked against this build's own
restatement (oracle.moe_experts_w8a8); router and combine are additionally pinned by the
reference-generated fixture.  Tolerance: each stage rounds to bf16, so the end-to-end bound is
3 x T1 (three roundings: gu, h, routed output) and cosine >= 0.9999.
"""
import importlib

import numpy as np
import pytest
import torch

from oracle import fp8_oracle as O
from helpers import assert_parity, from_bf16, kernels, to_bf16_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def moe():
    return importlib.import_module("nano-vllm-moe_b200.executor.moe")


def make_moe_case(seed, T, H, I, E, k):
    rng = np.random.default_rng(seed)
    x = O.bf16_round(rng.standard_normal((T, H), dtype=np.float32))
    logits = rng.standard_normal((T, E), dtype=np.float32)
    w13 = (rng.standard_normal((E, 2 * I, H), dtype=np.float32) * 0.02).astype(np.float32)
    w2 = (rng.standard_normal((E, H, I), dtype=np.float32) * 0.02).astype(np.float32)
    w13_q = np.empty(w13.shape, np.uint8); w13_s = np.empty((E, 2 * I), np.float32)
    w2_q = np.empty(w2.shape, np.uint8); w2_s = np.empty((E, H), np.float32)
    for e in range(E):
        w13_q[e], w13_s[e] = O.quantize_weight_per_channel(w13[e])
        w2_q[e], w2_s[e] = O.quantize_weight_per_channel(w2[e])
    in13 = O.input_scale_from_amax(np.abs(O.bf16_round(rng.standard_normal((512, H), dtype=np.float32))).max())
    in2 = np.float32(0.25 / 448.0 * 4)     # silu(g)*u of N(0,~0.9)-ish values: amax of a few units
    return dict(x=x, logits=logits, w13_q=w13_q, w13_s=w13_s, w2_q=w2_q, w2_s=w2_s, in13=in13, in2=in2)


def upload_weights(moe, c):
    T = lambda a: torch.from_numpy(a).cuda()
    return moe.Fp8ExpertWeights.from_checkpoint_layout(
        T(c["w13_q"]), T(c["w13_s"]), torch.tensor(float(c["in13"])), T(c["w2_q"]), T(c["w2_s"]), torch.tensor(float(c["in2"])))


def test_router_matches_reference_fixture(moe, golden):
    g = golden("moe")
    for ren in (0, 1):
        router = moe.SoftmaxTopKRouter(4, bool(ren))
        for dtype in (torch.float32,):
            w, ids = router.select_experts(None, torch.from_numpy(g["logits"]).cuda().to(dtype))
            assert ids.dtype == torch.int64 and w.dtype == torch.float32
            np.testing.assert_array_equal(ids.cpu().numpy(), g[f"topk_ids_ren{ren}"])
            np.testing.assert_allclose(w.cpu().numpy(), g[f"topk_w_ren{ren}"], rtol=1e-5, atol=1e-8)


def test_router_large_and_bf16(moe):
    rng = np.random.default_rng(3)
    for T, E, k in [(1, 60, 4), (257, 60, 4), (64, 128, 8), (5, 7, 2), (33, 64, 6), (40, 300, 5), (9, 1000, 3)]:
        logits = rng.standard_normal((T, E), dtype=np.float32)
        w_ref, ids_ref = O.softmax_topk(logits, k, False)
        w, ids = moe.SoftmaxTopKRouter(k, False).select_experts(None, torch.from_numpy(logits).cuda())
        np.testing.assert_array_equal(ids.cpu().numpy(), ids_ref)
        np.testing.assert_allclose(w.cpu().numpy(), w_ref, rtol=1e-5)
        lb = O.bf16_round(logits)
        w_ref, ids_ref = O.softmax_topk(lb, k, True)
        w, ids = moe.SoftmaxTopKRouter(k, True).select_experts(None, to_bf16_cuda(lb))
        np.testing.assert_array_equal(ids.cpu().numpy(), ids_ref)
        np.testing.assert_allclose(w.cpu().numpy(), w_ref, rtol=1e-5)


@pytest.mark.parametrize("T,H,I,E,k", [(1, 256, 128, 8, 2), (16, 512, 256, 12, 4), (64, 2048, 1408, 60, 4),
                                       (300, 256, 128, 6, 2), (1024, 512, 384, 8, 4),
                                       (48, 2048, 704, 15, 4), (700, 512, 704, 5, 2)])     # 704 = a TP-2 slice of 1408
def test_expert_ffn_matches_oracle(moe, T, H, I, E, k):
    c = make_moe_case(100 + T + E, T, H, I, E, k)
    wts = upload_weights(moe, c)
    w_ref, ids_ref = O.softmax_topk(c["logits"], k, False)
    ref = O.moe_experts_w8a8(c["x"], ids_ref, w_ref, c["w13_q"], c["w13_s"], c["in13"], c["w2_q"], c["w2_s"], c["in2"])
    cfg = moe.make_moe_parallel_config(tp_group=None, ep_group=None, global_num_experts=E, intermediate_size=I)
    kern = moe.MoEKernel(prepare_finalize=moe.NoEPPrepareFinalize(cfg), experts=moe.Fp8Experts(), parallel_config=cfg)
    w, ids = moe.SoftmaxTopKRouter(k, False).select_experts(None, torch.from_numpy(c["logits"]).cuda())
    y1 = from_bf16(kern(to_bf16_cuda(c["x"]), w, ids, wts, model_dtype=torch.bfloat16))
    y2 = from_bf16(kern(to_bf16_cuda(c["x"]), w, ids, wts, model_dtype=torch.bfloat16))
    np.testing.assert_array_equal(y1, y2)              # row grouping order must not change a bit
    assert_parity(y1, ref, f"moe T={T} E={E}", ulps=3.0, min_cos=0.9999)
    assert kernels().read_status(torch.device("cuda", 0)) == 0


@pytest.mark.parametrize("T,H,I,E,k", [(1024, 512, 384, 8, 4), (600, 2048, 1408, 60, 4), (4096, 256, 128, 6, 2), (900, 512, 256, 60, 1),
                                       (2100, 272, 128, 5, 3), (3000, 2048, 1408, 60, 4)])     # H = 272: a lone last weight tile
def test_fused_activation_epilogue_equals_the_separate_pass(moe, T, H, I, E, k):
    """Prefill-sized batches: the gate_up grouped GEMM's epilogue applies silu * up and quantises for the down
    projection.  Same values, same roundings as the separate pass: bit-identical outputs (chunks of 32, 64 and 128 rows,
    experts with no rows, ragged last chunks)."""
    Kn = kernels()
    c = make_moe_case(300 + T + E, T, H, I, E, k)
    wts = upload_weights(moe, c)
    cfg = moe.make_moe_parallel_config(tp_group=None, ep_group=None, global_num_experts=E, intermediate_size=I)
    kern = moe.MoEKernel(prepare_finalize=moe.NoEPPrepareFinalize(cfg), experts=moe.Fp8Experts(), parallel_config=cfg)
    w, ids = moe.SoftmaxTopKRouter(k, False).select_experts(None, torch.from_numpy(c["logits"]).cuda())
    x = to_bf16_cuda(c["x"])
    try:
        y_rows = kern(x, w, ids, wts, model_dtype=torch.bfloat16)          # default: rows as the MMA M dimension where chunks are 128 rows
        Kn.set_tuning("moe_rows_major", 0)                                 # the channel-major grouped kernel, activation fused ...
        y_fused = kern(x, w, ids, wts, model_dtype=torch.bfloat16)
        Kn.set_tuning("moe_fused", 0)                                      # ... and with the separate activation pass
        y_plain = kern(x, w, ids, wts, model_dtype=torch.bfloat16)
    finally:
        Kn.set_tuning("moe_fused", -1)
        Kn.set_tuning("moe_rows_major", -1)
    assert torch.equal(y_fused, y_plain)
    assert y_fused.float().abs().max() > 0
    # the other orientation multiplies the same codes; only the accumulation order inside the MMA may differ
    assert_parity(from_bf16(y_rows), from_bf16(y_plain), "rows-major vs channel-major grouped GEMM", ulps=2.0, min_cos=0.99999)
    w_ref, ids_ref = O.softmax_topk(c["logits"], k, False)
    if T * k * H * I <= 2e9:
        ref = O.moe_experts_w8a8(c["x"], ids_ref, w_ref, c["w13_q"], c["w13_s"], c["in13"], c["w2_q"], c["w2_s"], c["in2"])
        assert_parity(from_bf16(y_rows), ref, f"rows-major moe T={T} E={E}", ulps=3.0, min_cos=0.9999)
    assert Kn.read_status(torch.device("cuda", 0)) == 0


def test_expert_rows_outside_local_range_are_skipped(moe):
    """Expert-parallel ranks see ids of other ranks' experts as out of range: those rows stay zero."""
    c = make_moe_case(7, 32, 256, 128, 4, 2)
    wts = upload_weights(moe, c)
    ids = torch.tensor([0, 1, 2, 3, -1, 4, 9, 2] * 8, dtype=torch.int64, device="cuda")
    w = torch.ones(64, dtype=torch.float32, device="cuda")
    out = from_bf16(moe.Fp8Experts().apply(to_bf16_cuda(c["x"]), ids, w, wts, x_div=2))
    bad = np.isin(ids.cpu().numpy(), [-1, 4, 9])
    assert (out[bad] == 0).all() and (np.abs(out[~bad]).sum(axis=1) > 0).all()
