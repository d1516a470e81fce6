"""Pin the CPU oracle against what the reference's own code produced
(fixtures in tests/golden/, generator tests/golden/make_golden.py)."""
import numpy as np
import pytest

from oracle import fp8_oracle as O


def test_e4m3_decode_all_codes(golden):
    g = golden("e4m3_codec")
    dec = O.e4m3_decode(np.arange(256, dtype=np.uint8))
    np.testing.assert_array_equal(np.isnan(dec), np.isnan(g["decoded"]))
    m = ~np.isnan(dec)
    np.testing.assert_array_equal(dec[m], g["decoded"][m])


def test_e4m3_encode_matches_torch(golden):
    g = golden("e4m3_codec")
    np.testing.assert_array_equal(O.e4m3_encode(g["values"]), g["encoded"])


def test_e4m3_roundtrip():
    codes = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)
    np.testing.assert_array_equal(O.e4m3_encode(O.e4m3_decode(codes)), codes)


def test_activation_quant_matches_reference(golden):
    g = golden("act_quant")
    for s, want in zip(g["scales"], g["codes"]):
        np.testing.assert_array_equal(O.quantize_activation(g["x"], s), want)


def test_weight_quant_matches_reference(golden):
    g = golden("weight_quant")
    q, s = O.quantize_weight_per_channel(g["w"])
    np.testing.assert_array_equal(s, g["scale"])
    np.testing.assert_array_equal(q, g["codes"])


def _bf16_ulps(a, b):
    return np.abs(O.bf16_bits(a).astype(np.int64) - O.bf16_bits(b).astype(np.int64))


def test_known_answer_patterns_match_reference_gemm(golden):
    g = golden("linear")
    for si, (m, n, k) in enumerate(g["kat_shapes"]):
        for p in ["ones", "identity", "xones_wramp", "xramp_wones", "ramp"]:
            x, wq, s_in, s_w = O.known_answer_case(p, m, n, k)
            got = O.debug_reference_gemm(x, wq, s_in, s_w)
            want = g[f"kat_{si}_{p}"]
            assert got.shape == want.shape
            # same bf16 operands, fp32 accumulation in a different order: <= 1 bf16 ulp
            assert O.cosine(got, want) > 0.999999, (p, m, n, k)
            same_sign = np.sign(got) == np.sign(want)
            assert _bf16_ulps(got, want)[same_sign].max() <= 1, (p, m, n, k)


def test_known_answer_exact_values():
    # ones: every output is K (exactly representable while K <= 256)
    x, wq, s_in, s_w = O.known_answer_case("ones", 4, 8, 64)
    y = O.linear_w8a8(x, wq, np.full(8, s_w, np.float32), s_in)
    np.testing.assert_array_equal(y, np.full((4, 8), 64.0, np.float32))
    # identity: y[i, i] = 1
    x, wq, s_in, s_w = O.known_answer_case("identity", 8, 8, 32)
    y = O.linear_w8a8(x, wq, np.full(8, s_w, np.float32), s_in)
    np.testing.assert_array_equal(y, np.eye(8, dtype=np.float32))


def test_random_cases_match_torch_epilogue(golden):
    g = golden("linear")
    for ci, (m, k, n) in enumerate(g["rand_shapes"]):
        c = O.make_case(1000 + ci, m, k, n, calib_rows=64)
        np.testing.assert_array_equal(O.quantize_activation(c["x"], c["input_scale"]), g[f"rand_{ci}_xq"])
        for got, key in (
            (O.linear_w8a16(c["x"], c["wq"], c["w_scale"], c["bias"]), "w8a16"),
            (O.linear_w8a16(c["x"], c["wq"], c["w_scale"], None), "w8a16_nobias"),
            (O.linear_w8a8(c["x"], c["wq"], c["w_scale"], c["input_scale"], c["bias"]), "w8a8"),
            (O.linear_dequant_matmul(c["x"], c["wq"], c["w_scale"]), "oref"),
        ):
            want = g[f"rand_{ci}_{key}"]
            ok, worst = O.check_close(got, want, ulps=1.0)
            assert ok, (key, m, k, n, worst)
            assert (O.bf16_bits(got) != O.bf16_bits(want)).mean() < 0.02, key


def test_exact_oracle_is_close_to_dequant_matmul():
    # tolerance T2: how far the quantised paths sit from the reference's bf16
    # dequant-then-matmul check on the benchmark's distributions
    c = O.make_case(7, 16, 2048, 512)
    oref = O.linear_dequant_matmul(c["x"], c["wq"], c["w_scale"])
    y16 = O.linear_w8a16(c["x"], c["wq"], c["w_scale"], None)
    y8 = O.linear_w8a8(c["x"], c["wq"], c["w_scale"], c["input_scale"], None)
    assert O.cosine(y16, oref) >= 0.9999
    assert O.cosine(y8, oref) >= 0.999


def test_router_matches_reference(golden):
    g = golden("moe")
    for ren in (0, 1):
        w, ids = O.softmax_topk(g["logits"], 4, bool(ren))
        np.testing.assert_array_equal(ids, g[f"topk_ids_ren{ren}"])
        np.testing.assert_allclose(w, g[f"topk_w_ren{ren}"], rtol=2e-6, atol=1e-8)


def test_moe_ffn_algebra_matches_reference(golden):
    g = golden("moe")
    y = O.moe_experts_dense(g["x"], g["topk_ids_ren0"], g["topk_w_ren0"], g["w13"], g["w2"])
    ok, worst = O.check_close(y, g["moe_out"], ulps=2.0)
    assert ok, worst


def test_row_parallel_sums_to_full():
    c = O.make_case(11, 8, 256, 64)
    full = O.linear_w8a8(c["x"], c["wq"], c["w_scale"], c["input_scale"], c["bias"])
    for tp in (2, 4):
        y = O.row_parallel(c["x"], c["wq"], c["w_scale"], c["input_scale"], c["bias"], tp, "fp8_w8a8_static")
        ok, worst = O.check_close(y, full, ulps=tp)
        assert ok, (tp, worst)
    ycol = O.column_parallel(c["x"], c["wq"], c["w_scale"], c["input_scale"], c["bias"], 4, "fp8_w8a8_static")
    np.testing.assert_array_equal(ycol, full)


def test_silu_and_mul_both_forms_match_reference(golden):
    """The activation as the reference runs it (compiled: one rounding) and as the same Python runs
    eagerly (two roundings) -- the dense MLP uses the first, the expert FFN the second."""
    g = golden("activation")
    fused, eager = O.silu_mul(g["x"]), O.silu_mul_unfused(g["x"])
    # exp() differs in the last fp32 bit between libraries: at most a handful of bf16 results move by one ulp
    for got, want in ((fused, g["compiled"]), (eager, g["eager"])):
        diff = O.bf16_bits(got) != O.bf16_bits(want)
        assert diff.mean() < 1e-3 and _bf16_ulps(got, want).max() <= 1
    # the two forms are really different functions on these inputs, so the fixture tells them apart
    assert (O.bf16_bits(fused) != O.bf16_bits(g["eager"])).mean() > 0.1
    assert (O.bf16_bits(eager) != O.bf16_bits(g["compiled"])).mean() > 0.1


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_rmsnorm_matches_reference(golden, tag):
    g = golden("rmsnorm")
    x, res, w, eps = g[f"{tag}_x"], g[f"{tag}_residual"], g[f"{tag}_weight"], g[f"{tag}_eps"]
    for compiled, key in ((True, "compiled"), (False, "eager")):
        y = O.rmsnorm(x, w, eps, compiled=compiled)
        y2, r2 = O.rmsnorm(x, w, eps, res, compiled=compiled)
        # the fp32 mean of squares is summed in another order here: at most one bf16 ulp, almost never
        for got, want in ((y, g[f"{tag}_{key}"]), (y2, g[f"{tag}_add_{key}"])):
            assert (O.bf16_bits(got) != O.bf16_bits(want)).mean() < 1e-3 and _bf16_ulps(got, want).max() <= 1
        np.testing.assert_array_equal(r2, g[f"{tag}_add_residual_{key}"])
    assert (O.bf16_bits(O.rmsnorm(x, w, eps)) != O.bf16_bits(g[f"{tag}_eager"])).mean() > 0.05


def test_moe_row_grouping_matches_reference_alignment(golden):
    """moe_align_block_size (nanovllm/utils/moe.py) on the fixture's routing: every block holds rows of one
    expert only, each expert's rows appear exactly once, padding uses the sentinel T*k."""
    g = golden("moe")
    ids = g["topk_ids_ren0"].reshape(-1)
    st, eids, nb = g["align_sorted_weight_idx"], g["align_expert_ids"], int(g["align_total_blocks"])
    tok = g["align_sorted_token_ids"]
    np.testing.assert_array_equal(tok[st < ids.size], st[st < ids.size] // 4)      # token of a routed row (k = 4)
    block = 8
    assert st.size >= nb * block
    for b in range(nb):
        rows = st[b * block:(b + 1) * block]
        real = rows[rows < ids.size]
        assert (ids[real] == eids[b]).all()
    real = st[: nb * block]
    real = real[real < ids.size]
    np.testing.assert_array_equal(np.sort(real), np.arange(ids.size))
    perm, counts, _ = O.ep_dispatch_plan(g["topk_ids_ren0"], 12, 1)
    assert counts.sum() == ids.size
