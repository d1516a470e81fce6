"""RMSNorm -> e4m3 fusion, the linears on pre-quantised activations, and a decode step replayed from a CUDA graph.

The reference's runner captures its decode step once per batch size and replays it
(nanovllm/engine/model_runner.py:488-541): static input/output buffers, no allocation, no host sync inside the
captured region.  The last test here holds this library to the same contract on the linear path of 28 decoder
layers (input norm -> qkv -> [attention stand-in] -> o_proj -> post-attention norm -> fused MLP).
"""
import importlib

import numpy as np
import pytest
import torch

from oracle import fp8_oracle as O
from helpers import assert_parity, from_bf16, kernels, to_bf16_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    torch.cuda.synchronize()
    assert kernels().read_status(torch.device("cuda", 0)) == 0


def _ulps(a, b):
    return np.abs(O.bf16_bits(a).astype(np.int64) - O.bf16_bits(b).astype(np.int64))


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_rmsnorm_matches_reference_fixture(golden, tag):
    """The kernel against what the reference's compiled RMSNorm produced (bf16 output, new residual)."""
    Kn = kernels()
    g = golden("rmsnorm")
    x, res, w, eps = g[f"{tag}_x"], g[f"{tag}_residual"], g[f"{tag}_weight"], float(g[f"{tag}_eps"])
    _, y = Kn.rmsnorm_quant(to_bf16_cuda(x), to_bf16_cuda(w), eps)
    r = to_bf16_cuda(res)
    _, y2 = Kn.rmsnorm_quant(to_bf16_cuda(x), to_bf16_cuda(w), eps, residual=r)
    for got, want in ((from_bf16(y), g[f"{tag}_compiled"]), (from_bf16(y2), g[f"{tag}_add_compiled"])):
        # the sum of squares is taken in another order than torch's: at most one bf16 ulp, rarely
        assert (O.bf16_bits(got) != O.bf16_bits(want)).mean() < 2e-3 and _ulps(got, want).max() <= 1
    np.testing.assert_array_equal(from_bf16(r), g[f"{tag}_add_residual_compiled"])


@pytest.mark.parametrize("m,h", [(1, 3584), (16, 3584), (64, 2048), (300, 8192), (5, 264), (2048, 3584)])
def test_rmsnorm_quant_codes_match_oracle(m, h):
    Kn = kernels()
    rng = np.random.default_rng(m + h)
    x = O.bf16_round(rng.standard_normal((m, h), dtype=np.float32) * 3.0)
    res = O.bf16_round(rng.standard_normal((m, h), dtype=np.float32))
    w = O.bf16_round(1.0 + 0.2 * rng.standard_normal(h).astype(np.float32))
    scale = np.float32(6.0 / 448.0)
    want_codes, want_res = O.rmsnorm_quant(x, w, 1e-6, scale, res)
    want_y, _ = O.rmsnorm(x, w, 1e-6, res)
    r = to_bf16_cuda(res)
    xq, y = Kn.rmsnorm_quant(to_bf16_cuda(x), to_bf16_cuda(w), 1e-6, input_scale=torch.tensor(float(scale), device="cuda"),
                             residual=r, want_bf16=True)
    np.testing.assert_array_equal(from_bf16(r), want_res)
    got_y = from_bf16(y)
    assert (O.bf16_bits(got_y) != O.bf16_bits(want_y)).mean() < 2e-3 and _ulps(got_y, want_y).max() <= 1
    # the codes are exactly the quantiser's codes of the kernel's own bf16 output ...
    np.testing.assert_array_equal(xq.cpu().numpy(), O.quantize_activation(got_y, scale))
    # ... and differ from the oracle's only where that output differs by its one ulp
    assert (xq.cpu().numpy() != want_codes).mean() < 2e-3
    # without a residual, and codes only
    xq2, y2 = Kn.rmsnorm_quant(to_bf16_cuda(x), to_bf16_cuda(w), 1e-6, input_scale=torch.tensor(float(scale), device="cuda"))
    assert y2 is None
    assert (xq2.cpu().numpy() != O.rmsnorm_quant(x, w, 1e-6, scale)[0]).mean() < 2e-3


def test_rmsnorm_argument_checks(pkg):
    lib, L = pkg._lib.load(), pkg._lib
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device="cuda")
    w = torch.ones(64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((4, 64), dtype=torch.uint8, device="cuda")
    sc = torch.ones((), dtype=torch.float32, device="cuda")
    call = lambda h, xq, y, scale, ld=64: lib.fp8lin_rmsnorm_quant(x.data_ptr(), ld, None, 0, w.data_ptr(), 1e-6, scale, xq, y, 64, 4, h, None)
    assert call(64, None, None, sc.data_ptr()) == L.ERR_NULL            # nothing to write
    assert call(64, out.data_ptr(), None, None) == L.ERR_NULL           # codes without a scale
    assert call(60, out.data_ptr(), None, sc.data_ptr()) == L.ERR_SHAPE
    assert call(8200, out.data_ptr(), None, sc.data_ptr()) == L.ERR_SHAPE
    assert call(64, out.data_ptr(), None, sc.data_ptr(), ld=60) == L.ERR_SHAPE
    assert lib.fp8lin_rmsnorm_quant(x.data_ptr(), 64, None, 0, w.data_ptr(), 1e-6, sc.data_ptr(), out.data_ptr(), None, 0, 0, 64, None) == L.OK


@pytest.mark.parametrize("m,k,n", [(1, 3584, 4608), (7, 448, 576), (16, 2048, 11008), (64, 18944, 3584), (130, 448, 576),
                                   (1024, 2048, 11008), (4096, 3584, 4608)])
def test_linear_on_prequantised_activations(m, k, n):
    """fp8lin_w8a8_preq on the quantiser's codes gives what fp8lin_w8a8 gives on the bf16 activations
    (to the accumulation order: the route may differ), and matches the oracle."""
    Kn = kernels()
    c = O.make_case(10 + m + n, m, k, n, calib_rows=256)
    from helpers import oracle_linear, upload_case
    d = upload_case(c)
    xq = Kn.quantize_activation(d["x"], d["input_scale"])
    np.testing.assert_array_equal(xq.cpu().numpy(), O.quantize_activation(c["x"], c["input_scale"]))
    y = from_bf16(Kn.launch_w8a8_preq(xq, d["w_nk"], d["input_scale"], d["w_scale"], d["bias"]))
    rows = np.arange(m) if m <= 256 else np.random.default_rng(0).choice(m, 64, replace=False)
    ref = oracle_linear("fp8_w8a8_static", c, rows=rows)
    assert_parity(y[rows], ref, f"preq {m}x{k}x{n}")
    y_full = from_bf16(Kn.launch_w8a8_gemm(d["x"], d["w_nk"], d["input_scale"], d["w_scale"], d["bias"]))
    assert_parity(y, y_full, "preq vs quantise-inside", ulps=1.0)


def test_layer_api_with_quantised_activation(pkg):
    """RMSNorm.forward_quant -> ColumnParallelLinear / FusedFp8MLP, against RMSNorm.forward -> the same layers."""
    Kn = kernels()
    rng = np.random.default_rng(4)
    m, h, inter = 9, 512, 640
    norm = pkg.RMSNorm(h, 1e-6).cuda()
    norm.weight.data = to_bf16_cuda(1.0 + 0.1 * rng.standard_normal(h).astype(np.float32))
    cfg = pkg.Fp8Config("fp8_w8a8_static")

    def make(cls, k, n, **kw):
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        q, s = O.quantize_weight_per_channel(w)
        lay = cls(k, n, quant_method=cfg.get_quant_method(None, "t"), **kw) if cls is not pkg.MergedColumnParallelLinear else \
            cls(k, [n // 2, n // 2], quant_method=cfg.get_quant_method(None, "t"))
        if cls is pkg.MergedColumnParallelLinear:
            for i in (0, 1):
                lay.qweight.weight_loader(lay.qweight, torch.from_numpy(q[i * n // 2:(i + 1) * n // 2]), i)
                lay.weight_scale.weight_loader(lay.weight_scale, torch.from_numpy(s[i * n // 2:(i + 1) * n // 2]), i)
        else:
            lay.qweight.weight_loader(lay.qweight, torch.from_numpy(q))
            lay.weight_scale.weight_loader(lay.weight_scale, torch.from_numpy(s))
        lay.input_scale.weight_loader(lay.input_scale, torch.tensor(5.0 / 448.0))
        lay = lay.cuda()
        pkg.process_weights_after_loading(lay)
        return lay
    qkv = make(pkg.ColumnParallelLinear, h, 768)
    gate_up = make(pkg.MergedColumnParallelLinear, h, 2 * inter)
    down = make(pkg.RowParallelLinear, inter, h)
    mlp = pkg.FusedFp8MLP(gate_up, down)
    x = to_bf16_cuda(rng.standard_normal((m, h), dtype=np.float32))
    res = to_bf16_cuda(rng.standard_normal((m, h), dtype=np.float32))
    y_plain, res_plain = norm(x, res)
    qa, res_q = norm.forward_quant(x, qkv.input_scale, res.clone())
    assert torch.equal(res_q, res_plain) and qa.codes.dtype == torch.uint8
    assert torch.equal(qa.codes, Kn.quantize_activation(y_plain, qkv.input_scale))
    assert_parity(from_bf16(qkv(qa)), from_bf16(qkv(y_plain)), "qkv from codes", ulps=1.0)
    assert_parity(from_bf16(mlp(qa)), from_bf16(mlp(y_plain)), "mlp from codes", ulps=1.0)
    other = pkg.QuantizedActivation(qa.codes, torch.tensor(0.5, device="cuda"))
    with pytest.raises(ValueError, match="scale"):
        qkv(other)


def _decode_weights(layers, h, inter, qkv_n, seed):
    exp = importlib.import_module("nano-vllm-moe_b200.quantization.export")
    Kn = kernels()
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = []
    for _ in range(layers):
        L = {}
        for name, (k, n) in {"qkv": (h, qkv_n), "o": (h, h), "gate_up": (h, 2 * inter), "down": (inter, h)}.items():
            q, s = exp.quantize_weight(torch.randn((n, k), generator=g, device="cuda") * (0.04 if name in ("o", "down") else 0.02))
            L[name] = (Kn.pack_weight_nk(q), s)
            L[name + "_codes"] = q
        L["gate_up_il"] = Kn.interleave_gate_up(L["gate_up"][0], L["gate_up"][1], None, inter)[:2]
        L["norm1"] = (1.0 + 0.1 * torch.randn(h, generator=g, device="cuda")).to(torch.bfloat16)
        L["norm2"] = (1.0 + 0.1 * torch.randn(h, generator=g, device="cuda")).to(torch.bfloat16)
        out.append(L)
    return out


class _DecodeStep:
    """The linear path of a stack of decoder layers on static buffers (nothing is allocated in `run`)."""

    def __init__(self, weights, m, h, inter, qkv_n):
        dev = "cuda"
        self.w, self.m, self.h = weights, m, h
        f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=dev)
        self.s_qkv, self.s_o, self.s_gu, self.s_down = f32(6.0 / 448), f32(3.0 / 448), f32(6.0 / 448), f32(2.0 / 448)
        self.hidden = torch.zeros((m, h), dtype=torch.bfloat16, device=dev)        # static input
        self.work = torch.zeros((m, h), dtype=torch.bfloat16, device=dev)
        self.residual = torch.zeros((m, h), dtype=torch.bfloat16, device=dev)
        self.xq = torch.zeros((m, h), dtype=torch.uint8, device=dev)
        self.qkv = torch.zeros((m, qkv_n), dtype=torch.bfloat16, device=dev)
        self.attn = torch.zeros((m, h), dtype=torch.bfloat16, device=dev)
        self.out = torch.zeros((m, h), dtype=torch.bfloat16, device=dev)           # static output
        Kn = kernels()
        Kn.reserve_workspace(torch.device(dev, 0), max(
            Kn.workspace_bytes(1, m, h, qkv_n), Kn.workspace_bytes(1, m, h, h),
            int(importlib.import_module("nano-vllm-moe_b200")._lib.load().fp8lin_mlp_workspace_bytes(m, h, inter, h))))

    def run(self):
        Kn = kernels()
        self.work.copy_(self.hidden)
        self.residual.zero_()
        for L in self.w:
            Kn.rmsnorm_quant(self.work, L["norm1"], 1e-6, input_scale=self.s_qkv, residual=self.residual, xq_out=self.xq)
            Kn.launch_w8a8_preq(self.xq, L["qkv"][0], self.s_qkv, L["qkv"][1], None, out=self.qkv)
            # attention itself is outside this library: its stand-in passes the first H columns on
            Kn.launch_w8a8_gemm(self.qkv[:, :self.h], L["o"][0], self.s_o, L["o"][1], None, out=self.attn)
            Kn.rmsnorm_quant(self.attn, L["norm2"], 1e-6, input_scale=self.s_gu, residual=self.residual, xq_out=self.xq)
            Kn.launch_mlp_w8a8(self.xq, L["gate_up_il"][0], L["gate_up_il"][1], self.s_gu, None, L["down"][0], L["down"][1],
                               self.s_down, None, out=self.work)
        self.out.copy_(self.work)


def test_decode_step_two_layers_against_the_oracle():
    m, h, inter, qkv_n = 5, 256, 384, 384
    w = _decode_weights(2, h, inter, qkv_n, 3)
    step = _DecodeStep(w, m, h, inter, qkv_n)
    x = O.bf16_round(np.random.default_rng(8).standard_normal((m, h), dtype=np.float32))
    step.hidden.copy_(to_bf16_cuda(x))
    step.run()
    work, res = x, np.zeros_like(x)
    f = lambda t: np.float32(t.item())
    for L in w:
        codes, res = O.rmsnorm_quant(work, from_bf16(L["norm1"]), 1e-6, f(step.s_qkv), res)
        qkv = O.linear_w8a8_preq(codes, L["qkv_codes"].cpu().numpy(), L["qkv"][1].cpu().numpy(), f(step.s_qkv))
        attn = O.linear_w8a8(qkv[:, :h], L["o_codes"].cpu().numpy(), L["o"][1].cpu().numpy(), f(step.s_o))
        codes, res = O.rmsnorm_quant(attn, from_bf16(L["norm2"]), 1e-6, f(step.s_gu), res)
        gu = O.linear_w8a8_preq(codes, L["gate_up_codes"].cpu().numpy(), L["gate_up"][1].cpu().numpy(), f(step.s_gu))
        work = O.linear_w8a8(O.silu_mul(gu), L["down_codes"].cpu().numpy(), L["down"][1].cpu().numpy(), f(step.s_down))
    # ten roundings in a row (two norms, four linears, the activation per layer): a loose elementwise bound, a tight cosine
    assert_parity(from_bf16(step.out), work, "two decoder layers", ulps=8.0, min_cos=0.9995)
    assert_parity(from_bf16(step.residual), res, "residual stream", ulps=8.0, min_cos=0.9995)


@pytest.mark.parametrize("m", [1, 16])
def test_decode_step_of_28_layers_replays_from_a_cuda_graph(m):
    h, inter, qkv_n, layers = 1024, 2816, 1536, 28
    w = _decode_weights(layers, h, inter, qkv_n, 11)
    step = _DecodeStep(w, m, h, inter, qkv_n)
    g0 = torch.Generator(device="cuda").manual_seed(1)
    inputs = [torch.randn((m, h), generator=g0, device="cuda").to(torch.bfloat16) for _ in range(3)]
    side = torch.cuda.Stream()
    Kn = kernels()
    with torch.cuda.stream(side):
        Kn.reserve_workspace(torch.device("cuda", 0), 64 << 20)          # the capture stream's own scratch
        eager = []
        for x in inputs:
            step.hidden.copy_(x)
            step.run()
            eager.append(step.out.clone())
        torch.cuda.synchronize()
        launches0 = Kn.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            before = torch.cuda.memory_stats()["allocation.all.allocated"]      # (starting a capture allocates its RNG state)
            step.run()
            allocated = torch.cuda.memory_stats()["allocation.all.allocated"] - before
        # nothing was allocated while the step was captured, and one kernel-launch sequence per layer was recorded
        assert allocated == 0
        per_step = Kn.launch_count() - launches0
        assert layers * 5 <= per_step <= layers * 9
        for x, want in zip(inputs, eager):
            step.hidden.copy_(x)
            step.out.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(step.out, want)               # bit for bit the eager sequence
    assert torch.isfinite(eager[0].float()).all() and eager[0].float().abs().max() > 0
    assert not torch.equal(eager[0], eager[1])
