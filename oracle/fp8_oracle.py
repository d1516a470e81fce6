"""CPU oracle for the FP8 quantized-linear path.  TEST INFRASTRUCTURE ONLY.

This module is a numpy restatement of the arithmetic of nano-vllm-moe's FP8
linear path.  It is the checker for the CUDA kernels: only the test-suite, the
smoke check and the bench's CPU-baseline leg may import it.  The product
package never does (the product fails loudly when its CUDA library is absent).

Parity status: PINNED.  Every function below is checked in
``tests/test_oracle_golden.py`` against fixtures under ``tests/golden/`` that
were produced by importing the reference's own Python code on CPU
(``tests/golden/make_golden.py`` is the generator).

Reference locations restated here (paths inside the reference project):

* e4m3 = ``torch.float8_e4m3fn`` (finite-only, max 448, one NaN code 0x7f/0xff).
* weight quantisation         scripts/quantization/quantize.py:52-56
* static input scale          scripts/quantization/quantize.py:200-203
* activation quantisation     nanovllm/quantization/kernels/fp8.py:250-252
* W8A16 epilogue algebra      nanovllm/quantization/kernels/fp8.py:57-76
* W8A8 epilogue algebra       nanovllm/quantization/kernels/fp8.py:281-338,
                              nanovllm/quantization/w8a8_jit.py:364-431
* dequant-then-matmul check   scripts/quantization/w8a16_linear_microbench.py:47-48,
                              scripts/quantization/fp8_linear_microbench.py:67,77,
                              scripts/debug/debug_ptx_mma.py:75-88
* row-parallel reduction      nanovllm/layers/linear.py:258-262
* SiluAndMul                  nanovllm/layers/activation.py:6-14
* RMSNorm                     nanovllm/layers/layernorm.py:17-41
* router                      nanovllm/executor/moe/router.py:24-34
* expert FFN                  nanovllm/executor/moe/experts/eager_experts.py:26-35
* top-k combine               nanovllm/executor/moe/prepare_finalize/no_ep.py:45
* EP dispatch/combine         nanovllm/executor/moe/prepare_finalize/torch_alltoall.py:19-93
"""
from __future__ import annotations

import numpy as np

FP8_MAX = 448.0

# --------------------------------------------------------------------------
# number formats
# --------------------------------------------------------------------------


def _build_e4m3_table() -> np.ndarray:
    """Value of each of the 256 e4m3fn codes (NaN for 0x7f and 0xff)."""
    tab = np.zeros(256, dtype=np.float32)
    for code in range(256):
        sign = -1.0 if code & 0x80 else 1.0
        exp = (code >> 3) & 0xF
        man = code & 0x7
        if exp == 0xF and man == 0x7:
            val = np.nan
        elif exp == 0:
            val = sign * man * 2.0 ** -9
        else:
            val = sign * (1.0 + man / 8.0) * 2.0 ** (exp - 7)
        tab[code] = val
    return tab


E4M3_TABLE = _build_e4m3_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    """uint8 e4m3fn codes -> float32 values (exact)."""
    return E4M3_TABLE[np.asarray(codes, dtype=np.uint8)]


def e4m3_encode(values: np.ndarray) -> np.ndarray:
    """float32 -> e4m3fn codes, round-to-nearest-even.

    Follows ``tensor.to(torch.float8_e4m3fn)``: magnitudes that round above
    448 (>= 464) and infinities become NaN (0x7f | sign); the callers clamp to
    +-448 first, exactly as the reference does, so that never happens on the
    hot path.  NaN stays NaN.
    """
    v = np.asarray(values, dtype=np.float32)
    out = np.zeros(v.shape, dtype=np.uint8)
    sign = (np.signbit(v)).astype(np.uint8) << 7
    a = np.abs(v).astype(np.float64)
    nan = np.isnan(v)
    # exponent of the e4m3 binade the value falls in (subnormals share 2^-6)
    with np.errstate(divide="ignore", invalid="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.clip(e, -6, 8)
    step = 2.0 ** (e - 3)  # spacing of e4m3 values in that binade
    q = a / step  # in units of the spacing
    r = np.rint(q)  # numpy rint is round-half-to-even
    mag = r * step
    # rebuild the code from the rounded magnitude
    with np.errstate(divide="ignore", invalid="ignore"):
        e2 = np.floor(np.log2(np.where(mag > 0, mag, 1.0)))
    e2 = np.clip(e2, -6, 8)
    man = np.rint(mag / 2.0 ** (e2 - 3)).astype(np.int64)  # 8..15 normal, 0..7 subnormal
    normal = man >= 8
    code = np.where(normal, ((e2 + 7).astype(np.int64) << 3) | (man - 8), man)
    code = np.where(mag > FP8_MAX, 0x7F, code)
    code = np.where(nan, 0x7F, code)
    out = (code.astype(np.uint8) & 0x7F) | sign
    return out.astype(np.uint8)


def bf16_round(values: np.ndarray) -> np.ndarray:
    """Round float32 to the nearest bfloat16 (ties to even), returned as float32."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    bits = v.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    rounded = ((bits + 0x7FFF + lsb) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(v), v, out).astype(np.float32)


def bf16_bits(values: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns (uint16) of float32 values after RNE rounding."""
    return (bf16_round(values).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------
# quantisers
# --------------------------------------------------------------------------


def quantize_weight_per_channel(weight_nk: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """[N,K] float weights -> (uint8 e4m3 codes [N,K], float32 scale [N]).

    scale = clamp(amax_row, 1e-8) / 448; q = e4m3(clamp(W / scale, +-448)).
    Reference: scripts/quantization/quantize.py:52-56.
    """
    w = np.asarray(weight_nk, dtype=np.float32)
    amax = np.maximum(np.abs(w).max(axis=1), np.float32(1e-8)).astype(np.float32)
    scale = (amax / np.float32(FP8_MAX)).astype(np.float32)
    q = np.clip((w / scale[:, None]).astype(np.float32), -FP8_MAX, FP8_MAX)
    return e4m3_encode(q), scale


def input_scale_from_amax(amax: float) -> np.float32:
    """Static activation scale = max(amax, 1e-8) / 448 (quantize.py:200-203)."""
    return np.float32(max(float(amax), 1e-8) / FP8_MAX)      # in double, rounded once, as the exporter does


def quantize_activation(x: np.ndarray, input_scale) -> np.ndarray:
    """bf16-valued float32 activations -> e4m3 codes with one static scale.

    q = e4m3(clamp(float(x) / max(scale, 1e-12), +-448)), true fp32 division.
    Reference: nanovllm/quantization/kernels/fp8.py:250-252.
    """
    s = np.maximum(np.float32(input_scale), np.float32(1e-12)).astype(np.float32)
    q = (np.asarray(x, dtype=np.float32) / s).astype(np.float32)
    return e4m3_encode(np.clip(q, -FP8_MAX, FP8_MAX))


# --------------------------------------------------------------------------
# the linear itself
# --------------------------------------------------------------------------


def _matmul_nt(a_mk: np.ndarray, b_nk: np.ndarray, exact: bool) -> np.ndarray:
    if exact:
        return (a_mk.astype(np.float64) @ b_nk.astype(np.float64).T).astype(np.float32)
    return a_mk.astype(np.float32) @ b_nk.astype(np.float32).T


def linear_w8a16(x, wq_nk, w_scale, bias=None, *, exact=True, round_out=True):
    """y = bf16((x . Wq^T) * w_scale[n] + bias[n]), single final rounding.

    x: [M,K] bf16-valued float32; wq_nk: [N,K] uint8 codes; w_scale: [N] f32;
    bias: [N] bf16-valued float32 or None.
    """
    acc = _matmul_nt(np.asarray(x, np.float32), e4m3_decode(wq_nk), exact)
    y = acc * np.asarray(w_scale, np.float32)[None, :]
    if bias is not None:
        y = y + np.asarray(bias, np.float32)[None, :]
    y = y.astype(np.float32)
    return bf16_round(y) if round_out else y


def linear_w8a8(x, wq_nk, w_scale, input_scale, bias=None, *, exact=True, round_out=True):
    """y = bf16((xq . Wq^T) * max(in_scale,1e-12) * w_scale[n] + bias[n]).

    Per-output-channel weight scales are kept (the reference's runtime folds
    them into one per-tensor scale at load, fp8.py:100-105; see
    ``requantize_per_tensor`` for that variant).
    """
    return linear_w8a8_preq(quantize_activation(x, input_scale), wq_nk, w_scale, input_scale, bias, exact=exact,
                            round_out=round_out)


def linear_w8a8_preq(xq_codes, wq_nk, w_scale, input_scale, bias=None, *, exact=True, round_out=True):
    """The W8A8 linear from activations that are already e4m3 codes (the same epilogue algebra)."""
    s = np.maximum(np.float32(input_scale), np.float32(1e-12)).astype(np.float32)
    xq = e4m3_decode(xq_codes)
    acc = _matmul_nt(xq, e4m3_decode(wq_nk), exact)
    y = (acc * s).astype(np.float32) * np.asarray(w_scale, np.float32)[None, :]
    if bias is not None:
        y = y + np.asarray(bias, np.float32)[None, :]
    y = y.astype(np.float32)
    return bf16_round(y) if round_out else y


def linear_dequant_matmul(x, wq_nk, w_scale):
    """The reference's check formula: ``mm(x_bf16, Wq.to(bf16) * scale.to(bf16))``.

    Scale and the dequantised weight are both rounded to bf16; the product is
    accumulated in fp32 and rounded to bf16 once (w8a16_linear_microbench.py:47-48).
    No bias, activations are NOT quantised.
    """
    w = bf16_round(e4m3_decode(wq_nk) * bf16_round(np.asarray(w_scale, np.float32))[:, None])
    return bf16_round(_matmul_nt(np.asarray(x, np.float32), w, exact=False))


def debug_reference_gemm(x, wq_nk, input_scale, weight_scale):
    """Quant-aware check of scripts/debug/debug_ptx_mma.py:75-88 (scalar scales)."""
    ws = bf16_round(np.float32(weight_scale))
    w = bf16_round(e4m3_decode(wq_nk) * ws)
    xq = e4m3_decode(e4m3_encode(np.clip((np.asarray(x, np.float32) / np.float32(input_scale)).astype(np.float32), -448, 448)))
    xd = bf16_round(xq * bf16_round(np.float32(input_scale)))
    return bf16_round(_matmul_nt(xd, w, exact=False))


def requantize_per_tensor(wq_nk, w_scale):
    """Reference runtime weight folding (nanovllm/quantization/fp8.py:100-105).

    Returns (codes [N,K], scalar scale).  Loses precision on low-amax channels;
    provided so tests can quantify the difference to per-channel scales.
    """
    ws = np.asarray(w_scale, np.float32)
    t = np.maximum(ws.max(), np.float32(1e-12)).astype(np.float32)
    scaled = (e4m3_decode(wq_nk) * (ws / t)[:, None]).astype(np.float32)
    return e4m3_encode(np.clip(scaled, -FP8_MAX, FP8_MAX)), t


# --------------------------------------------------------------------------
# tensor parallel
# --------------------------------------------------------------------------


def row_parallel(x, wq_nk, w_scale, input_scale, bias, tp, scheme):
    """Row-parallel linear: K split over ``tp`` ranks, bias on rank 0 only,
    each rank's output rounded to bf16, then summed (all-reduce) and rounded
    to bf16 (nanovllm/layers/linear.py:258-262).  The sum is taken in fp32 in
    rank order; NCCL's order may differ, callers allow ``tp`` bf16 ulps."""
    k = x.shape[1]
    assert k % tp == 0
    ks = k // tp
    total = None
    for r in range(tp):
        xs = x[:, r * ks:(r + 1) * ks]
        ws = wq_nk[:, r * ks:(r + 1) * ks]
        b = bias if r == 0 else None
        if scheme == "fp8_w8a16":
            part = linear_w8a16(xs, ws, w_scale, b)
        else:
            part = linear_w8a8(xs, ws, w_scale, input_scale, b)
        total = part if total is None else bf16_round(total + part)
    return total


def column_parallel(x, wq_nk, w_scale, input_scale, bias, tp, scheme):
    """Column-parallel linear: N split over ranks, outputs concatenated."""
    n = wq_nk.shape[0]
    assert n % tp == 0
    ns = n // tp
    outs = []
    for r in range(tp):
        sl = slice(r * ns, (r + 1) * ns)
        b = None if bias is None else bias[sl]
        if scheme == "fp8_w8a16":
            outs.append(linear_w8a16(x, wq_nk[sl], w_scale[sl], b))
        else:
            outs.append(linear_w8a8(x, wq_nk[sl], w_scale[sl], input_scale, b))
    return np.concatenate(outs, axis=1)


# --------------------------------------------------------------------------
# MoE expert FFN
# --------------------------------------------------------------------------


def softmax_topk(router_logits, top_k, renormalize=False):
    """fp32 softmax over experts, then top-k (router.py:30-34).

    Ties are broken towards the lower expert index (matches torch.topk on the
    seeded continuous inputs used in the tests, where ties do not occur)."""
    z = np.asarray(router_logits, np.float32)
    z = z - z.max(axis=-1, keepdims=True)
    e = np.exp(z).astype(np.float32)
    p = (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)
    ids = np.argsort(-p, axis=-1, kind="stable")[:, :top_k]
    w = np.take_along_axis(p, ids, axis=-1)
    if renormalize:
        w = w / w.sum(axis=-1, keepdims=True)
    return w.astype(np.float32), ids.astype(np.int64)


def silu_mul(gate_up: np.ndarray) -> np.ndarray:
    """bf16(silu(gate) * up) with gate/up the two halves of the last axis,
    evaluated in fp32 from bf16-valued inputs, ONE rounding: what the reference's
    ``SiluAndMul.forward`` computes as it is decorated (``@torch.compile`` fuses the two
    ops into one fp32 expression; nanovllm/layers/activation.py:11-14).  Pinned by
    ``activation.npz['compiled']``."""
    half = gate_up.shape[-1] // 2
    g = gate_up[..., :half].astype(np.float32)
    u = gate_up[..., half:].astype(np.float32)
    s = (g / (np.float32(1.0) + np.exp(-g).astype(np.float32))).astype(np.float32)
    return bf16_round((s * u).astype(np.float32))


def rmsnorm(x, weight, eps, residual=None, compiled=True):
    """RMSNorm.rms_forward / add_rms_forward (nanovllm/layers/layernorm.py:17-41) on bf16-valued
    float32 inputs, bf16 weight.  fp32: v = x [+ residual]; var = mean(v^2); n = v * rsqrt(var + eps).

    compiled=True (the form the reference runs: both methods are ``@torch.compile``d, and the
    compiler keeps the fused expression in fp32, dropping the intermediate ``.to(bf16)``):
    out = bf16(n * weight), one rounding.  compiled=False (the same Python run eagerly):
    out = bf16(bf16(n) * weight).  With a residual the second result is bf16(x + residual),
    the stream the next layer adds to; the normalisation uses the unrounded fp32 sum.
    Both forms are pinned by ``rmsnorm.npz``."""
    v = np.asarray(x, np.float32)
    new_res = None
    if residual is not None:
        v = (v + np.asarray(residual, np.float32)).astype(np.float32)
        new_res = bf16_round(v)
    var = (v.astype(np.float32) ** 2).mean(axis=-1, keepdims=True, dtype=np.float32)
    inv = (np.float32(1.0) / np.sqrt(var + np.float32(eps), dtype=np.float32)).astype(np.float32)
    normed = (v * inv).astype(np.float32)
    if not compiled:
        normed = bf16_round(normed)
    out = bf16_round((normed * np.asarray(weight, np.float32)[None, :]).astype(np.float32))
    return out if residual is None else (out, new_res)


def rmsnorm_quant(x, weight, eps, input_scale, residual=None):
    """RMSNorm feeding a W8A8-static linear: the norm's bf16 output quantised with the linear's static
    activation scale (layernorm.py:17-41 followed by kernels/fp8.py:250-252).  Returns (codes, new residual)."""
    r = rmsnorm(x, weight, eps, residual)
    out, new_res = (r, None) if residual is None else r
    return quantize_activation(out, input_scale), new_res


def mlp_w8a8(x, gu_q, gu_scale, gu_in_scale, gu_bias, down_q, down_scale, down_in_scale, down_bias):
    """Dense MLP block on W8A8-static linears; restates Qwen2MLP.forward
    (nanovllm/models/qwen2.py:110-114): gate_up_proj -> SiluAndMul
    (nanovllm/layers/activation.py:11-14, compiled: one rounding) -> down_proj.

    gu_q [2I,H] codes (gate rows then up rows), down_q [N,I] codes; scales per
    output channel, one activation scale per linear.  gate_up is rounded to
    bf16 (the tensor the reference materialises), h = bf16(silu(g) * u), and
    the down projection quantises h with its own static scale.
    """
    gu = linear_w8a8(x, gu_q, gu_scale, gu_in_scale, gu_bias)
    return linear_w8a8(silu_mul(gu), down_q, down_scale, down_in_scale, down_bias)


def moe_experts_w8a8(x, topk_ids, topk_weights, w13_q, w13_scale, w13_in_scale,
                     w2_q, w2_scale, w2_in_scale):
    """Routed expert FFN on FP8 operands; restates EagerExperts.apply
    (eager_experts.py:26-35) + NoEPPrepareFinalize.finalize (no_ep.py:45).

    x [T,H]; topk_ids/topk_weights [T,k]; w13_q [E,2I,H] codes, w13_scale [E,2I];
    w2_q [E,H,I] codes, w2_scale [E,H]; in-scales scalars (one per layer).
    Per routed row: gu = bf16(W8A8 linear); h = bf16(bf16(silu(g))*u) (eager, two roundings);
    o = (W8A8 linear)(h) * weight in fp32, rounded to bf16 once; the k routed
    rows of a token are then summed in fp32 in slot order and rounded to bf16.
    PARITY UNPINNED by the reference for the FP8 operands (its experts are
    bf16-only and discard the scales, eager_experts.py:25); the routing, FFN
    algebra and combine are pinned on bf16 inputs by the golden fixtures.
    """
    t, h = x.shape
    k = topk_ids.shape[1]
    n_exp = w13_q.shape[0]
    routed = np.zeros((t, k, w2_q.shape[1]), dtype=np.float32)
    for e in range(n_exp):
        tok, slot = np.nonzero(topk_ids == e)
        if tok.size == 0:
            continue
        gu = linear_w8a8(x[tok], w13_q[e], w13_scale[e], w13_in_scale)
        hmid = silu_mul_unfused(gu)
        o = linear_w8a8(hmid, w2_q[e], w2_scale[e], w2_in_scale, round_out=False)
        routed[tok, slot] = bf16_round(o * topk_weights[tok, slot][:, None].astype(np.float32))
    return bf16_round(routed.sum(axis=1, dtype=np.float32))


def moe_experts_dense(x, topk_ids, topk_weights, w13, w2):
    """Same FFN on bf16-valued dense weights (the reference's actual path),
    used to pin the routing/FFN/combine algebra against the golden fixture."""
    t = x.shape[0]
    k = topk_ids.shape[1]
    routed = np.zeros((t, k, w2.shape[1]), dtype=np.float32)
    for e in range(w13.shape[0]):
        tok, slot = np.nonzero(topk_ids == e)
        if tok.size == 0:
            continue
        gu = bf16_round(_matmul_nt(x[tok], w13[e], exact=False))
        hmid = silu_mul_unfused(gu)
        o = bf16_round(_matmul_nt(hmid, w2[e], exact=False))
        routed[tok, slot] = bf16_round(o * bf16_round(topk_weights[tok, slot])[:, None])
    return bf16_round(routed.sum(axis=1, dtype=np.float32))


def silu_mul_unfused(gate_up):
    """torch eager in bf16: bf16(silu(gate)) then bf16(. * up) -- the expert FFN's form
    (``F.silu(gate) * up`` outside any compiled region, experts/eager_experts.py:33).
    Pinned by ``activation.npz['eager']`` and through ``moe.npz['moe_out']``."""
    half = gate_up.shape[-1] // 2
    g = gate_up[..., :half].astype(np.float32)
    u = gate_up[..., half:].astype(np.float32)
    s = bf16_round((g / (np.float32(1.0) + np.exp(-g).astype(np.float32))).astype(np.float32))
    return bf16_round(s * u)


def ep_dispatch_plan(topk_ids, num_experts, ep_size):
    """Which routed row goes to which expert-parallel rank, and in what order.

    Restates torch_alltoall.py:26-36: target rank = id // (E/ep); rows are
    stably sorted by target rank; the local expert id is id % (E/ep).
    Returns (permute_indices, send_counts[ep], local_ids in permuted order).
    """
    local = num_experts // ep_size
    flat = np.asarray(topk_ids).reshape(-1)
    target = np.clip(flat // local, 0, ep_size - 1)
    perm = np.argsort(target, kind="stable")
    counts = np.bincount(target, minlength=ep_size)
    return perm, counts, (flat % local)[perm]


# --------------------------------------------------------------------------
# seeded synthetic inputs (the benchmark's stand-in for real checkpoints)
# --------------------------------------------------------------------------


def make_case(seed, m, k, n, *, with_bias=True, calib_rows=4096):
    """x ~ N(0,1) bf16; W ~ N(0,0.02) quantised per channel; bias ~ N(0,0.01)
    bf16; static input scale from a ``calib_rows`` x K N(0,1) bf16 draw."""
    rng = np.random.default_rng(seed)
    x = bf16_round(rng.standard_normal((m, k), dtype=np.float32))
    w = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    wq, ws = quantize_weight_per_channel(w)
    bias = bf16_round(rng.standard_normal(n, dtype=np.float32) * np.float32(0.01)) if with_bias else None
    calib = bf16_round(rng.standard_normal((calib_rows, k), dtype=np.float32))
    in_scale = input_scale_from_amax(np.abs(calib).max())
    return {"x": x, "wq": wq, "w_scale": ws, "bias": bias, "input_scale": in_scale}


def known_answer_case(pattern, m, n, k, seed=42):
    """The synthetic patterns of scripts/debug/debug_ptx_mma.py:33-65.

    Returns (x [M,K] bf16-valued, wq [N,K] codes, input_scale, weight_scale)."""
    if pattern == "ones":
        x = np.ones((m, k), np.float32); w = np.ones((n, k), np.float32); si, sw = 1.0, 1.0
    elif pattern == "identity":
        x = np.zeros((m, k), np.float32); w = np.zeros((n, k), np.float32)
        for i in range(min(m, k)):
            x[i, i] = 1.0
        for i in range(min(n, k)):
            w[i, i] = 1.0
        si, sw = 1.0, 1.0
    elif pattern == "xones_wramp":
        x = np.ones((m, k), np.float32)
        w = np.tile(np.arange(k, dtype=np.float32) / 16.0, (n, 1)); si, sw = 1.0, 16.0
    elif pattern == "xramp_wones":
        x = np.tile(np.arange(k, dtype=np.float32) / 16.0, (m, 1))
        w = np.ones((n, k), np.float32); si, sw = 16.0, 1.0
    elif pattern == "ramp":
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((m, k), dtype=np.float32)
        w = np.tile(np.arange(k, dtype=np.float32) / 16.0, (n, 1)); si, sw = 16.0, 16.0
    else:
        raise ValueError(f"unknown pattern: {pattern}")
    return bf16_round(x), e4m3_encode(w), np.float32(si), np.float32(sw)


def pack_tiles(wq_nk: np.ndarray) -> np.ndarray:
    """[N,K] codes -> the kernels' packed layout (this build's own format, no reference
    counterpart): 128 x 128-byte tiles, tile (n/128, k/128) at ((n/128)*KB + k/128)*16384,
    byte (n%128)*128 + k%128 inside it, zero padding."""
    n, k = wq_nk.shape
    nt, kb = -(-n // 128), -(-k // 128)
    pad = np.zeros((nt * 128, kb * 128), dtype=np.uint8)
    pad[:n, :k] = wq_nk
    return pad.reshape(nt, 128, kb, 128).transpose(0, 2, 1, 3).reshape(-1).copy()


# --------------------------------------------------------------------------
# tolerances shared by the tests
# --------------------------------------------------------------------------


def check_close(y, ref, ulps=1.0):
    """Tolerance for a bf16 result against the exact oracle:
    |y - ref| <= ulps * (2^-7 |ref| + 2^-7 rms(ref)); returns (ok, worst ratio)."""
    y = np.asarray(y, np.float32); ref = np.asarray(ref, np.float32)
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))) if ref.size else 0.0
    tol = ulps * (2.0 ** -7 * np.abs(ref) + 2.0 ** -7 * rms) + 1e-30
    ratio = np.abs(y - ref) / tol
    worst = float(ratio.max()) if ratio.size else 0.0
    return worst <= 1.0, worst


def cosine(a, b):
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    den = np.linalg.norm(a) * np.linalg.norm(b)
    return float(a @ b / den) if den > 0 else 1.0
