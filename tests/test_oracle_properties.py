"""Size-independent properties of the oracle's building blocks (CPU): codec round trips, monotone
quantisers, the packed layout as a bijection, linearity of the linears in the bias and in the row set."""
import numpy as np
from hypothesis import given, settings, strategies as st

from oracle import fp8_oracle as O


def test_codec_round_trip_over_all_codes():
    codes = np.arange(256, dtype=np.uint8)
    vals = O.e4m3_decode(codes)
    finite = np.isfinite(vals)
    assert finite.sum() == 254                                  # two NaN codes, no infinities
    back = O.e4m3_encode(vals[finite])
    # +0 and -0 keep their own codes; every other finite value is its own nearest code
    np.testing.assert_array_equal(back, codes[finite])
    assert np.abs(vals[finite]).max() == 448.0


@settings(max_examples=50, deadline=None)
@given(st.floats(min_value=1e-6, max_value=10.0, allow_nan=False), st.integers(0, 2**32 - 1))
def test_activation_quantiser_is_monotone_and_saturates(scale, seed):
    rng = np.random.default_rng(seed)
    x = np.sort(O.bf16_round((rng.standard_normal(512) * 50 * scale).astype(np.float32)))
    q = O.e4m3_decode(O.quantize_activation(x, np.float32(scale)))
    assert np.all(np.diff(q) >= 0)                              # order preserved
    assert np.abs(q).max() <= 448.0
    big = O.bf16_round(np.array([1e30, -1e30], np.float32))
    np.testing.assert_array_equal(O.e4m3_decode(O.quantize_activation(big, np.float32(scale))), [448.0, -448.0])


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 300), st.integers(1, 40), st.integers(0, 2**32 - 1))
def test_weight_quantiser_properties(n, k16, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, 16 * k16)) * rng.choice([1e-3, 0.02, 5.0])).astype(np.float32)
    q, s = O.quantize_weight_per_channel(w)
    assert q.dtype == np.uint8 and s.dtype == np.float32 and q.shape == w.shape and s.shape == (n,)
    deq = O.e4m3_decode(q) * s[:, None]
    amax = np.abs(w).max(axis=1)
    np.testing.assert_array_equal(np.abs(O.e4m3_decode(q)).max(axis=1)[amax > 1e-8], 448.0)      # the extreme maps to +-448
    # half a step of the top binade (and the fp32 roundings of w / scale and code * scale: a few ulps of slack)
    assert np.all(np.abs(deq - w) <= amax[:, None] / 448.0 * 16.0 * (1.0 + 1e-5) + 1e-12)
    # scaling a row by a power of two scales its scale and leaves the codes alone
    q2, s2 = O.quantize_weight_per_channel(w * 4.0)
    np.testing.assert_array_equal(q2, q)
    np.testing.assert_array_equal(s2, s * 4.0)


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 300), st.integers(1, 300), st.integers(0, 2**32 - 1))
def test_packed_layout_is_a_bijection_with_zero_padding(n, k, seed):
    rng = np.random.default_rng(seed)
    w = rng.integers(1, 256, size=(n, k), dtype=np.uint8)
    packed = O.pack_tiles(w)
    nt, kb = -(-n // 128), -(-k // 128)
    assert packed.size == nt * kb * 16384
    tiles = packed.reshape(nt, kb, 128, 128).transpose(0, 2, 1, 3).reshape(nt * 128, kb * 128)
    np.testing.assert_array_equal(tiles[:n, :k], w)
    assert tiles[n:].sum() == 0 and tiles[:, k:].sum() == 0


def test_linears_are_affine_in_the_bias_and_rowwise_independent():
    c = O.make_case(9, 24, 256, 80)
    for fn, extra in ((O.linear_w8a16, ()), (O.linear_w8a8, (c["input_scale"],))):
        y0 = fn(c["x"], c["wq"], c["w_scale"], *extra, None, round_out=False)
        yb = fn(c["x"], c["wq"], c["w_scale"], *extra, c["bias"], round_out=False)
        np.testing.assert_allclose(yb - y0, np.broadcast_to(c["bias"], y0.shape), rtol=0, atol=1e-5)
        rows = np.array([3, 17, 5])
        np.testing.assert_array_equal(fn(c["x"][rows], c["wq"], c["w_scale"], *extra, c["bias"]),
                                      fn(c["x"], c["wq"], c["w_scale"], *extra, c["bias"])[rows])


def test_mlp_restatement_composes_the_pinned_pieces():
    gu = O.make_case(4, 6, 128, 256)
    down = O.make_case(5, 6, 128, 64)
    y = O.mlp_w8a8(gu["x"], gu["wq"], gu["w_scale"], gu["input_scale"], gu["bias"],
                   down["wq"], down["w_scale"], down["input_scale"], down["bias"])
    h = O.silu_mul(O.linear_w8a8(gu["x"], gu["wq"], gu["w_scale"], gu["input_scale"], gu["bias"]))
    np.testing.assert_array_equal(y, O.linear_w8a8(h, down["wq"], down["w_scale"], down["input_scale"], down["bias"]))
    assert h.shape == (6, 128)
