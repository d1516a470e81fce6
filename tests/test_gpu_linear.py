"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle.

Tolerance T1 (vs the exact oracle): |y - o| <= 2^-7 |o| + 2^-7 rms(o) per
element and cosine >= 0.99999 -- one bf16 ulp plus cancellation slack, because
fp32 accumulation order differs between the tensor cores and the CPU.
Tolerance T2 (vs the reference's bf16 dequant-then-matmul check): cosine >=
0.9999 for W8A16 and >= 0.999 for W8A8 (activation quantisation noise).
Integer/byte results (prepack, activation codes) are compared bit for bit.
"""
import numpy as np
import pytest
import torch

from oracle import fp8_oracle as O
from helpers import (assert_parity, from_bf16, kernels, oracle_linear, run_linear, to_bf16_cuda, upload_case)

pytestmark = pytest.mark.gpu
SCHEMES = ["fp8_w8a16", "fp8_w8a8_static"]


@pytest.fixture(autouse=True)
def _clean_tuning_and_status():
    Kn = kernels()
    yield
    for knob in ("stream_splits", "stream_max_m", "umma_bn", "umma_splits", "swap_splits", "swap_enable", "swap_min_m", "swap_preq_min_m", "w8a16_swap_enable",
                 "w8a16_swap_min_m", "w8a16_umma_min_m", "w8a16_chunk_mb", "umma_pair"):
        Kn.set_tuning(knob, -1)
    torch.cuda.synchronize()
    assert Kn.read_status(torch.device("cuda", 0)) == 0


def test_library_is_loaded_from_the_tree(pkg):
    lib = pkg._lib.load()
    assert "libfp8lin.so" in str(pkg._lib.LIB_PATH) and lib.fp8lin_version() == 1
    assert torch.cuda.get_device_capability(0)[0] == 10


def test_prepack_layout_is_exact():
    Kn = kernels()
    g = torch.Generator().manual_seed(0)
    for k, n in [(64, 48), (448, 576), (2048, 2048), (1408, 72), (16, 8)]:
        q_nk = torch.randint(0, 256, (n, k), dtype=torch.uint8, generator=g)
        want = O.pack_tiles(q_nk.numpy())
        assert want.size == Kn.packed_bytes(k, n)
        from_nk = Kn.pack_weight_nk(q_nk.cuda()).cpu().numpy()
        from_kn = Kn.prepack_weight(q_nk.t().contiguous().cuda()).cpu().numpy()
        np.testing.assert_array_equal(from_nk, want)
        np.testing.assert_array_equal(from_kn, want)


def test_activation_codes_match_reference_bit_for_bit(golden):
    Kn = kernels()
    g = golden("act_quant")
    n = (g["x"].size // 16) * 16
    x = g["x"][:n].reshape(-1, 16)
    for s, want in zip(g["scales"], g["codes"]):
        got = Kn.quantize_activation(to_bf16_cuda(x), torch.tensor(float(s), device="cuda")).cpu().numpy()
        np.testing.assert_array_equal(got.reshape(-1), want[:n])
    # a strided view (row stride > K)
    rng = np.random.default_rng(9)
    wide = to_bf16_cuda(rng.standard_normal((37, 96), dtype=np.float32))
    view = wide[:, :64]
    got = Kn.quantize_activation(view, torch.tensor(0.0121, device="cuda")).cpu().numpy()
    np.testing.assert_array_equal(got, O.quantize_activation(from_bf16(view), np.float32(0.0121)))


def test_activation_quantiser_exhaustive_over_bf16():
    """Every finite bf16 value x a set of scales (calibration-like, powers of two, all-ones
    mantissa, the 1e-12 clamp): the device codes equal true-division codes bit for bit."""
    Kn = kernels()
    bits = np.arange(65536, dtype=np.uint32)
    x = (bits << 16).view(np.float32).reshape(4096, 16)
    finite = np.isfinite(x)
    xt = torch.from_numpy(bits.astype(np.int32).astype(np.int16).reshape(4096, 16)).view(torch.bfloat16).cuda()
    scales = [0.0121, 0.011764526, 1.0, 16.0, 0.5, 3.1e-3, np.float32(1.9999999), np.float32(0.012499999),
              1e-13, 7.3, 1.0e-5, 2.5e4]
    rng = np.random.default_rng(12)
    scales += list(np.exp(rng.uniform(np.log(1e-4), np.log(10.0), 20)).astype(np.float32))
    for s in scales:
        s = np.float32(s)
        got = Kn.quantize_activation(xt, torch.tensor(float(s), dtype=torch.float32, device="cuda")).cpu().numpy()
        with np.errstate(over="ignore", invalid="ignore"):
            want = O.quantize_activation(np.where(finite, x, 0), s)
        np.testing.assert_array_equal(got[finite], want[finite], err_msg=f"scale {s}")
        inf = np.isinf(x)
        assert ((got[inf] & 0x7F) == 0x7E).all()              # +-inf saturates to +-448 like clamp()
        nan = np.isnan(x)
        assert ((got[nan] & 0x7F) == 0x7F).all()


@pytest.mark.parametrize("scheme", SCHEMES)
def test_golden_random_cases(golden, scheme):
    g = golden("linear")
    key = "w8a16" if scheme == "fp8_w8a16" else "w8a8"
    for ci, (m, k, n) in enumerate(g["rand_shapes"]):
        if k % 16:
            continue
        c = O.make_case(1000 + ci, int(m), int(k), int(n), calib_rows=64)
        y = run_linear(scheme, upload_case(c))
        assert_parity(y, g[f"rand_{ci}_{key}"], f"golden {key} {m}x{k}x{n}")


@pytest.mark.parametrize("pattern", ["ones", "identity", "xones_wramp", "xramp_wones", "ramp"])
def test_known_answer_patterns(golden, pattern):
    g = golden("linear")
    Kn = kernels()
    for si, (m, n, k) in enumerate(g["kat_shapes"]):
        m, n, k = int(m), int(n), int(k)
        x, wq, s_in, s_w = O.known_answer_case(pattern, m, n, k)
        d = {"x": to_bf16_cuda(x), "w_nk": Kn.pack_weight_nk(torch.from_numpy(wq).cuda()),
             "w_scale": torch.full((n,), float(s_w), device="cuda"),
             "input_scale": torch.tensor(float(s_in), device="cuda"), "bias": None}
        y = run_linear("fp8_w8a8_static", d, bias=False)
        ref = O.linear_w8a8(x, wq, np.full(n, s_w, np.float32), s_in)
        if pattern in ("ones", "identity"):
            np.testing.assert_array_equal(y, ref)             # exactly representable sums
        else:
            assert_parity(y, ref, f"{pattern} {m}x{n}x{k}")
        # the reference's own gate: cosine > 0.999 against its quant-aware bf16 check
        want = g[f"kat_{si}_{pattern}"]
        if np.abs(want).max() > 0:
            assert O.cosine(y, want) > 0.999


STREAM_SHAPES = [
    (1, 2048, 2048), (16, 2048, 11008), (3, 448, 576), (4, 3584, 4608), (17, 704, 72), (8, 256, 16),
    (64, 3584, 3584), (33, 2368, 1000), (1, 18944, 3584), (2, 64, 8), (7, 16, 24), (40, 1408, 2048),
]


@pytest.mark.parametrize("scheme", SCHEMES + ["fp8_w8a8_static/mma_sync", "fp8_w8a16/mma_sync"])
@pytest.mark.parametrize("m,k,n", STREAM_SHAPES)
def test_streaming_kernel_parity(scheme, m, k, n):
    """Decode-sized shapes: W8A16 on the mma.sync streaming kernel, W8A8 on the swapped-operand
    tcgen05 kernel, and W8A8 on the mma.sync streaming kernel (kept for shapes the tcgen05 path
    does not take)."""
    if scheme.endswith("/mma_sync"):
        kernels().set_tuning("swap_enable", 0)
        kernels().set_tuning("w8a16_swap_enable", 0)
        scheme = scheme.split("/")[0]
        assert kernels().variant_name(1 if "a8" in scheme[-10:] else 0, m, k, n).startswith("stream_mma_")
    elif scheme == "fp8_w8a16":
        kernels().set_tuning("w8a16_swap_min_m", 1)  # by default M <= 8 stays on the mma.sync kernel
        assert kernels().variant_name(0, m, k, n).startswith("umma_swap_w8a16")
    elif scheme == "fp8_w8a8_static":
        kernels().set_tuning("swap_min_m", 1)        # by default M <= 8 goes to the mma.sync kernel
        assert kernels().variant_name(1, m, k, n).startswith("umma_swap_w8a8")
    c = O.make_case(20260519 + m * 7 + k + n, m, k, n)
    d = upload_case(c)
    y = run_linear(scheme, d)
    assert_parity(y, oracle_linear(scheme, c), f"{scheme} {m}x{k}x{n}")
    y_nb = run_linear(scheme, d, bias=False)
    assert_parity(y_nb, oracle_linear(scheme, c, bias=False), f"{scheme} no-bias {m}x{k}x{n}")
    oref = O.linear_dequant_matmul(c["x"], c["wq"], c["w_scale"])
    if k >= 256:
        assert O.cosine(y_nb, oref) >= (0.9999 if scheme == "fp8_w8a16" else 0.999)


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("m", [1, 16, 17, 33, 64])
def test_swapped_w8a16_kernel_split_variants(m, splits):
    Kn = kernels()
    Kn.set_tuning("w8a16_swap_min_m", 1)
    Kn.set_tuning("swap_splits", splits)
    c = O.make_case(1900 + m + splits, m, 2048, 640)
    d = upload_case(c)
    assert Kn.variant_name(0, m, 2048, 640).startswith("umma_swap_w8a16")
    y1 = run_linear("fp8_w8a16", d)
    y2 = run_linear("fp8_w8a16", d)
    np.testing.assert_array_equal(y1, y2)
    assert_parity(y1, oracle_linear("fp8_w8a16", c), f"swap w8a16 m={m} splits={splits}")


@pytest.mark.parametrize("scheme", SCHEMES)
def test_streaming_split_k_is_deterministic_and_equal(scheme):
    Kn = kernels()
    Kn.set_tuning("w8a16_swap_enable", 0)
    c = O.make_case(77, 16, 3584, 512)
    d = upload_case(c)
    ref = oracle_linear(scheme, c)
    outs = []
    Kn.set_tuning("swap_enable", 0)
    for splits in (1, 2, 7, 14):
        Kn.set_tuning("stream_splits", splits)
        y1 = run_linear(scheme, d)
        y2 = run_linear(scheme, d)
        np.testing.assert_array_equal(y1, y2)
        assert_parity(y1, ref, f"{scheme} splits={splits}")
        outs.append(y1)
        if 1 < splits <= 8:
            # up to eight slices hand their sums over inside a cluster; through scratch and the arrival counter instead:
            # the same additions in the same order, so the same bits
            Kn.set_tuning("stream_push", 0)
            try:
                np.testing.assert_array_equal(y1, run_linear(scheme, d))
            finally:
                Kn.set_tuning("stream_push", 1)


@pytest.mark.parametrize("scheme", SCHEMES)
def test_wide_m_passes_through_streaming_kernel(scheme):
    # the mma.sync kernel walks M > 64 in 64-row passes (W8A16: 65..255 rows by default)
    Kn = kernels()
    Kn.set_tuning("stream_max_m", 1 << 20)
    Kn.set_tuning("w8a16_umma_min_m", 0)
    c = O.make_case(5, 150, 512, 264)
    y = run_linear(scheme, upload_case(c))
    assert_parity(y, oracle_linear(scheme, c), f"{scheme} 150 rows")


def test_strided_x_and_empty_batch():
    Kn = kernels()
    c = O.make_case(3, 6, 128, 80)
    d = upload_case(c)
    wide = torch.zeros((6, 160), dtype=torch.bfloat16, device="cuda")
    wide[:, :128] = d["x"]
    y = from_bf16(Kn.launch_w8a8_gemm(wide[:, :128], d["w_nk"], d["input_scale"], d["w_scale"], d["bias"]))
    assert_parity(y, oracle_linear("fp8_w8a8_static", c), "strided x")
    empty = torch.zeros((0, 128), dtype=torch.bfloat16, device="cuda")
    assert Kn.launch_w8a8_gemm(empty, d["w_nk"], d["input_scale"], d["w_scale"], d["bias"]).shape == (0, 80)
    assert Kn.launch_w8a16_gemm(empty, d["w_nk"], d["w_scale"], None).shape == (0, 80)
    with pytest.raises(ValueError):
        Kn.launch_w8a16_gemm(torch.zeros((6, 256), dtype=torch.bfloat16, device="cuda"), d["w_nk"], d["w_scale"])  # K mismatch


UMMA_SHAPES = [
    (256, 11008, 2048), (1024, 2048, 11008), (130, 448, 576), (65, 128, 8), (300, 2368, 1000),
    (128, 3584, 4608), (513, 704, 72), (200, 16, 264),
]


@pytest.mark.parametrize("m,k,n", UMMA_SHAPES)
def test_tcgen05_gemm_parity(m, k, n):
    c = O.make_case(4242 + m + k + n, m, k, n)
    d = upload_case(c)
    assert kernels().variant_name(1, m, k, n).startswith("umma_w8a8")
    y = run_linear("fp8_w8a8_static", d)
    assert_parity(y, oracle_linear("fp8_w8a8_static", c), f"umma {m}x{k}x{n}")
    y2 = run_linear("fp8_w8a8_static", d)
    np.testing.assert_array_equal(y, y2)


@pytest.mark.parametrize("m,k,n", [(1280, 256, 4000), (1024, 2048, 11008), (2500, 144, 2056)])
def test_tcgen05_half_width_tail_items(m, k, n):
    """When the tile count leaves a short last round, its tiles run as two 128-column halves each
    (ragged N: the second half of the last column block is partly or wholly past N)."""
    Kn = kernels()
    c = O.make_case(808 + m + n, m, k, n)
    d = upload_case(c)
    assert "+half" in Kn.variant_name(1, m, k, n)
    y = run_linear("fp8_w8a8_static", d)
    assert_parity(y, oracle_linear("fp8_w8a8_static", c), f"umma half-width tail {m}x{k}x{n}")
    Kn.set_tuning("umma_bn", 128)                       # same arithmetic on whole 128-wide tiles
    np.testing.assert_array_equal(y, run_linear("fp8_w8a8_static", d))


PAIR_SHAPES = [(256, 256, 256), (130, 448, 576), (300, 2368, 1000), (1024, 2048, 11008), (4096, 3584, 4608), (65, 16, 8)]


@pytest.mark.parametrize("m,k,n", PAIR_SHAPES)
def test_tcgen05_cta_pair_gemm_parity(m, k, n):
    """256 x 256 tiles on CTA pairs (one MMA across two SMs): ragged M (the second CTA's rows partly or
    wholly past M), ragged N and K, against the oracle and the one-CTA kernel."""
    Kn = kernels()
    c = O.make_case(6060 + m + k + n, m, k, n)
    d = upload_case(c)
    y1 = run_linear("fp8_w8a8_static", d)
    Kn.set_tuning("umma_pair", 1)
    assert Kn.variant_name(1, m, k, n).startswith("umma_pair_w8a8")
    y = run_linear("fp8_w8a8_static", d)
    assert_parity(y, oracle_linear("fp8_w8a8_static", c), f"cta pair {m}x{k}x{n}")
    np.testing.assert_array_equal(y, run_linear("fp8_w8a8_static", d))
    assert_parity(y, y1, "cta pair vs one-CTA kernel", ulps=1.0)


def test_w8a16_large_m_on_cta_pairs():
    Kn = kernels()
    Kn.set_tuning("umma_pair", 1)
    Kn.set_tuning("w8a16_chunk_mb", 1)
    m, k, n = 520, 1408, 1928
    c = O.make_case(6161, m, k, n)
    y = run_linear("fp8_w8a16", upload_case(c))
    assert_parity(y, oracle_linear("fp8_w8a16", c), "w8a16 f16 gemm on cta pairs")


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("splits", [1, 3])
def test_tcgen05_tile_and_split_variants(bn, splits):
    Kn = kernels()
    Kn.set_tuning("umma_bn", bn)
    Kn.set_tuning("umma_splits", splits)
    c = O.make_case(99, 260, 1408, 520)
    y = run_linear("fp8_w8a8_static", upload_case(c))
    assert_parity(y, oracle_linear("fp8_w8a8_static", c), f"umma bn={bn} splits={splits}")


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("m", [1, 16, 17, 33, 64])
def test_swapped_tcgen05_kernel_split_variants(m, splits):
    Kn = kernels()
    Kn.set_tuning("swap_min_m", 1)
    Kn.set_tuning("swap_splits", splits)
    c = O.make_case(900 + m + splits, m, 2048, 640)
    d = upload_case(c)
    y1 = run_linear("fp8_w8a8_static", d)
    y2 = run_linear("fp8_w8a8_static", d)
    np.testing.assert_array_equal(y1, y2)
    assert_parity(y1, oracle_linear("fp8_w8a8_static", c), f"swap m={m} splits={splits}")


@pytest.mark.parametrize("preq_min", [1, 65])
@pytest.mark.parametrize("m", [12, 33, 64])
def test_swapped_kernel_with_and_without_prequantised_rows(m, preq_min):
    """The swapped-operand kernel either quantises the rows itself or takes them pre-quantised
    (default from 17 rows); both must give the same bits."""
    Kn = kernels()
    Kn.set_tuning("swap_preq_min_m", preq_min)
    c = O.make_case(4000 + m, m, 1408, 1000)
    d = upload_case(c)
    y = run_linear("fp8_w8a8_static", d)
    assert ("_preq" in Kn.variant_name(1, m, 1408, 1000)) == (m >= preq_min)
    assert_parity(y, oracle_linear("fp8_w8a8_static", c), f"swap preq_min={preq_min} m={m}")
    Kn.set_tuning("swap_preq_min_m", 65 if preq_min == 1 else 1)
    np.testing.assert_array_equal(y, run_linear("fp8_w8a8_static", d))


W8A16_UMMA_SHAPES = [(129, 448, 576), (256, 3584, 4608), (300, 2368, 1000), (513, 704, 72), (1024, 2048, 11008), (200, 16, 264)]


@pytest.mark.parametrize("m,k,n", W8A16_UMMA_SHAPES)
def test_w8a16_large_m_f16_gemm_parity(m, k, n):
    """Large M (by default from 256 rows): weights widened to f16 chunk by chunk, tcgen05 f16 GEMM; against the oracle and the
    mma.sync passes (same operand values, so only the accumulation order differs)."""
    Kn = kernels()
    c = O.make_case(5150 + m + k + n, m, k, n)
    d = upload_case(c)
    assert Kn.variant_name(0, m, k, n).startswith("umma_w8a16_f16") == (m >= 256)     # default threshold
    Kn.set_tuning("w8a16_umma_min_m", 1)
    assert Kn.variant_name(0, m, k, n).startswith("umma_w8a16_f16")
    y = run_linear("fp8_w8a16", d)
    assert_parity(y, oracle_linear("fp8_w8a16", c), f"w8a16 f16 gemm {m}x{k}x{n}")
    np.testing.assert_array_equal(y, run_linear("fp8_w8a16", d))
    Kn.set_tuning("w8a16_umma_min_m", 0)
    assert Kn.variant_name(0, m, k, n).startswith("stream_mma_w8a16")
    assert_parity(y, run_linear("fp8_w8a16", d), "f16 gemm vs mma.sync passes")


@pytest.mark.parametrize("chunk_mb,bn,splits", [(1, -1, -1), (1, 64, 1), (2, 128, 3), (1, 256, 2)])
def test_w8a16_large_m_chunks_and_tiles(chunk_mb, bn, splits):
    """Small chunks (several dequantise + GEMM rounds over one scratch buffer, the last chunk ragged) and
    forced tile widths / split-K factors."""
    Kn = kernels()
    Kn.set_tuning("w8a16_chunk_mb", chunk_mb)
    Kn.set_tuning("umma_bn", bn)
    Kn.set_tuning("umma_splits", splits)
    m, k, n = 260, 1408, 1928
    c = O.make_case(77 + chunk_mb + bn, m, k, n)
    d = upload_case(c)
    name = Kn.variant_name(0, m, k, n)
    assert name.startswith("umma_w8a16_f16") and not name.endswith("_c1")
    y = run_linear("fp8_w8a16", d)
    assert_parity(y, oracle_linear("fp8_w8a16", c), f"w8a16 chunks {name}")
    y0 = run_linear("fp8_w8a16", d, bias=False)
    assert_parity(y0, oracle_linear("fp8_w8a16", c, bias=False), f"w8a16 chunks no bias {name}")


def test_tcgen05_matches_streaming_kernel():
    # the two W8A8 kernels quantise x identically, so they agree to accumulation order
    Kn = kernels()
    c = O.make_case(123, 64, 2048, 1024)
    d = upload_case(c)
    y_swap = run_linear("fp8_w8a8_static", d)
    Kn.set_tuning("swap_enable", 0)
    y_stream = run_linear("fp8_w8a8_static", d)
    assert_parity(y_swap, y_stream, "swap vs stream", ulps=1.0)
    Kn.set_tuning("stream_max_m", 0)
    y_umma = run_linear("fp8_w8a8_static", d)
    assert_parity(y_umma, y_stream, "umma vs stream", ulps=1.0)


def test_large_prefill_rows_sampled():
    # full-size 7B prefill shape (M=4096, qkv); the oracle checks 192 sampled rows
    m, k, n = 4096, 3584, 4608
    c = O.make_case(31337, m, k, n, calib_rows=512)
    d = upload_case(c)
    y = run_linear("fp8_w8a8_static", d)
    rows = np.random.default_rng(0).choice(m, 192, replace=False)
    rows.sort()
    assert_parity(y[rows], oracle_linear("fp8_w8a8_static", c, rows=rows), "prefill sample")
    # linearity in the bias: y(bias) - y(0) == bias within a bf16 ulp of y
    y0 = run_linear("fp8_w8a8_static", d, bias=False)
    np.testing.assert_allclose(y - y0, np.broadcast_to(c["bias"], y.shape), atol=2.0 ** -6 * np.abs(y).max())


@pytest.mark.parametrize("scheme", SCHEMES)
def test_layer_end_to_end(pkg, scheme):
    """Loader -> prepack -> apply through the layer classes, as a model would."""
    rng = np.random.default_rng(8)
    k, n_gate, n_up, m = 256, 192, 64, 9
    wg = (rng.standard_normal((n_gate, k)) * 0.02).astype(np.float32)
    wu = (rng.standard_normal((n_up, k)) * 0.02).astype(np.float32)
    qg, sg = O.quantize_weight_per_channel(wg)
    qu, su = O.quantize_weight_per_channel(wu)
    lay = pkg.MergedColumnParallelLinear(k, [n_gate, n_up], bias=True,
                                         quant_method=pkg.Fp8Config(scheme).get_quant_method(None, "gate_up"))
    lay.qweight.weight_loader(lay.qweight, torch.from_numpy(qg), 0)
    lay.qweight.weight_loader(lay.qweight, torch.from_numpy(qu), 1)
    lay.weight_scale.weight_loader(lay.weight_scale, torch.from_numpy(sg), 0)
    lay.weight_scale.weight_loader(lay.weight_scale, torch.from_numpy(su), 1)
    bias = O.bf16_round(rng.standard_normal(n_gate + n_up).astype(np.float32) * 0.01)
    in_scale = np.float32(0.0121)
    if scheme == "fp8_w8a8_static":
        lay.input_scale.weight_loader(lay.input_scale, torch.tensor(in_scale))
    lay.bias.data.copy_(torch.from_numpy(bias))
    lay = lay.cuda()
    lay.bias.data = lay.bias.data.to(torch.bfloat16)
    assert lay.qweight.dtype == torch.uint8 and lay.weight_scale.dtype == torch.float32
    pkg.process_weights_after_loading(lay)
    assert lay.qweight_packed.numel() == kernels().packed_bytes(k, n_gate + n_up)
    x = O.bf16_round(rng.standard_normal((3, m // 3, k), dtype=np.float32))
    y = from_bf16(lay(to_bf16_cuda(x)))
    assert y.shape == (3, 3, n_gate + n_up)
    wq = np.concatenate([qg, qu]); ws = np.concatenate([sg, su])
    x2 = x.reshape(-1, k)
    ref = (O.linear_w8a16(x2, wq, ws, bias) if scheme == "fp8_w8a16"
           else O.linear_w8a8(x2, wq, ws, in_scale, bias))
    assert_parity(y.reshape(-1, n_gate + n_up), ref, f"layer {scheme}")


CANARY_SHAPES = [
    # (scheme, M, K, N): one shape per kernel route, with ragged M and N where the route allows them
    ("fp8_w8a16", 3, 448, 576), ("fp8_w8a16", 40, 704, 72), ("fp8_w8a16", 150, 512, 264), ("fp8_w8a16", 300, 2368, 1000),
    ("fp8_w8a8_static", 1, 2048, 2048), ("fp8_w8a8_static", 7, 16, 24), ("fp8_w8a8_static", 12, 1408, 1000),
    ("fp8_w8a8_static", 33, 2368, 1000), ("fp8_w8a8_static", 64, 3584, 3584), ("fp8_w8a8_static", 130, 448, 576),
    ("fp8_w8a8_static", 300, 2368, 1000), ("fp8_w8a8_static", 1280, 256, 4000), ("fp8_w8a8_static", 2048, 8192, 2560),
    ("fp8_w8a8_static/pair", 300, 2368, 1000), ("fp8_w8a8_static/pair", 1025, 448, 520),
]


@pytest.mark.parametrize("scheme,m,k,n", CANARY_SHAPES)
def test_no_kernel_writes_outside_its_output_matrix(scheme, m, k, n):
    """The output is a window of a larger buffer filled with a sentinel: rows above and below it and the columns to
    its right (row pitch > N) must come back untouched, whatever tails the tiles have (TMA stores clip at the tensor
    map's extent, the other epilogues predicate).  Stands in for a memory checker on the store side."""
    Kn = kernels()
    if scheme.endswith("/pair"):
        Kn.set_tuning("umma_pair", 1)
        scheme = scheme.split("/")[0]
    c = O.make_case(777 + m + n, m, k, n, calib_rows=64)
    d = upload_case(c)
    pitch = (n + 8 + 7) // 8 * 8 + 8                       # a multiple of 8, at least 8 spare columns
    guard = 5
    sentinel = -24576.0                                    # exactly representable in bf16, far from any output
    buf = torch.full((m + 2 * guard, pitch), sentinel, dtype=torch.bfloat16, device="cuda")
    window = buf[guard:guard + m, :n]
    if scheme == "fp8_w8a16":
        Kn.launch_w8a16_gemm(d["x"], d["w_nk"], d["w_scale"], d["bias"], out=window)
    else:
        Kn.launch_w8a8_gemm(d["x"], d["w_nk"], d["input_scale"], d["w_scale"], d["bias"], out=window)
    torch.cuda.synchronize()
    got = buf.float().cpu().numpy()
    assert (got[:guard] == sentinel).all() and (got[guard + m:] == sentinel).all(), "rows outside the window were written"
    assert (got[guard:guard + m, n:] == sentinel).all(), "columns past N were written"
    assert_parity(got[guard:guard + m, :n], oracle_linear(scheme, c), f"windowed output {scheme} {m}x{k}x{n}")
