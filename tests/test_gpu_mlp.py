"""GPU parity of the fused MLP call (gate_up -> silu * up -> quantise -> down, both linears W8A8-static)
against the oracle's restatement of the reference's MLP block, and against the same three steps run
separately through the C ABI.  Tolerance: three roundings on the way (gate_up to bf16, h to bf16, h to
e4m3), so 3 x T1 and cosine >= 0.9999, as for the expert FFN."""
import importlib

import numpy as np
import pytest
import torch

from oracle import fp8_oracle as O
from helpers import assert_parity, from_bf16, kernels, to_bf16_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean_status():
    Kn = kernels()
    yield
    Kn.set_tuning("umma_pair", -1)
    torch.cuda.synchronize()
    assert Kn.read_status(torch.device("cuda", 0)) == 0


def make_mlp_case(seed, m, h, inter, n):
    """Two seeded linears chained: the down projection's activation scale is calibrated on the
    intermediate tensor the oracle computes."""
    gu = O.make_case(seed, m, h, 2 * inter)
    g = O.linear_w8a8(gu["x"], gu["wq"], gu["w_scale"], gu["input_scale"], gu["bias"])
    hmid = O.silu_mul(g)
    rng = np.random.default_rng(seed + 1)
    w = (rng.standard_normal((n, inter)) * 0.02).astype(np.float32)
    wq, ws = O.quantize_weight_per_channel(O.bf16_round(w))
    down = {"wq": wq, "w_scale": ws, "bias": O.bf16_round((rng.standard_normal(n) * 0.01).astype(np.float32)),
            "input_scale": O.input_scale_from_amax(float(np.abs(hmid).max()) if hmid.size else 1.0)}
    return gu, down


def upload_mlp(gu, down, inter):
    Kn = kernels()
    dev = "cuda"
    w_gu = Kn.pack_weight_nk(torch.from_numpy(gu["wq"]).to(dev))
    s_gu = torch.from_numpy(gu["w_scale"]).to(dev)
    b_gu = to_bf16_cuda(gu["bias"])
    w_il, s_il, b_il = Kn.interleave_gate_up(w_gu, s_gu, b_gu, inter)
    d = {
        "x": to_bf16_cuda(gu["x"]), "w_gu": w_gu, "s_gu": s_gu, "b_gu": b_gu, "w_il": w_il, "s_il": s_il, "b_il": b_il,
        "in_gu": torch.tensor(float(gu["input_scale"]), dtype=torch.float32, device=dev),
        "w_d": Kn.pack_weight_nk(torch.from_numpy(down["wq"]).to(dev)), "s_d": torch.from_numpy(down["w_scale"]).to(dev),
        "b_d": to_bf16_cuda(down["bias"]), "in_d": torch.tensor(float(down["input_scale"]), dtype=torch.float32, device=dev),
    }
    return d


def run_fused(d, bias=True):
    Kn = kernels()
    return from_bf16(Kn.launch_mlp_w8a8(d["x"], d["w_il"], d["s_il"], d["in_gu"], d["b_il"] if bias else None,
                                        d["w_d"], d["s_d"], d["in_d"], d["b_d"] if bias else None))


def run_three_steps(d):
    Kn = kernels()
    gu = Kn.launch_w8a8_gemm(d["x"], d["w_gu"], d["in_gu"], d["s_gu"], d["b_gu"]).float()
    g, u = gu.chunk(2, -1)
    h = (g / (1.0 + torch.exp(-g)) * u).to(torch.bfloat16)
    return from_bf16(Kn.launch_w8a8_gemm(h, d["w_d"], d["in_d"], d["s_d"], d["b_d"]))


MLP_SHAPES = [(1, 512, 384, 512), (16, 448, 256, 264), (64, 512, 384, 512), (65, 512, 384, 512), (130, 448, 256, 264),
              (300, 1024, 1408, 1000), (1024, 2048, 1408, 2048)]


@pytest.mark.parametrize("m,h,inter,n", MLP_SHAPES)
def test_fused_mlp_parity(m, h, inter, n):
    gu, down = make_mlp_case(7100 + m + h + inter, m, h, inter, n)
    d = upload_mlp(gu, down, inter)
    y = run_fused(d)
    ref = O.mlp_w8a8(gu["x"], gu["wq"], gu["w_scale"], gu["input_scale"], gu["bias"],
                     down["wq"], down["w_scale"], down["input_scale"], down["bias"])
    assert_parity(y, ref, f"fused mlp {m}x{h}x{inter}x{n}", ulps=3.0, min_cos=0.9999)
    np.testing.assert_array_equal(y, run_fused(d))
    assert_parity(y, run_three_steps(d), "fused vs three separate steps", ulps=3.0, min_cos=0.9999)


def test_fused_mlp_without_bias_and_large_rows():
    m, h, inter, n = 2048, 3584, 2560, 3584            # 7B hidden size, a slice of the intermediate size
    gu, down = make_mlp_case(99, m, h, inter, n)
    d = upload_mlp(gu, down, inter)
    y = run_fused(d, bias=False)
    rows = np.sort(np.random.default_rng(1).choice(m, 96, replace=False))
    ref = O.mlp_w8a8(gu["x"][rows], gu["wq"], gu["w_scale"], gu["input_scale"], None,
                     down["wq"], down["w_scale"], down["input_scale"], None)
    assert_parity(y[rows], ref, "fused mlp, sampled rows", ulps=3.0, min_cos=0.9999)


def test_fused_mlp_rejects_bad_arguments():
    Kn = kernels()
    gu, down = make_mlp_case(5, 8, 256, 128, 256)
    d = upload_mlp(gu, down, 128)
    with pytest.raises(ValueError):
        Kn.interleave_gate_up(d["w_gu"], d["s_gu"], d["b_gu"], 96)          # not a multiple of 128
    with pytest.raises(ValueError):
        Kn.launch_mlp_w8a8(d["x"], d["w_il"], d["s_il"], d["in_gu"], d["b_il"], d["w_gu"], d["s_d"], d["in_d"], d["b_d"])


def test_fused_mlp_layer_matches_separate_layers():
    pkg = importlib.import_module("nano-vllm-moe_b200")
    m, h, inter = 200, 512, 384
    gu, down = make_mlp_case(31, m, h, inter, h)
    cfg = pkg.Fp8Config("fp8_w8a8_static")
    gate_up = pkg.MergedColumnParallelLinear(h, [inter, inter], bias=True, quant_method=cfg.get_quant_method(None, "mlp.gate_up_proj"))
    down_l = pkg.RowParallelLinear(inter, h, bias=True, quant_method=cfg.get_quant_method(None, "mlp.down_proj"))
    for shard in (0, 1):
        rows = slice(shard * inter, (shard + 1) * inter)
        gate_up.qweight.weight_loader(gate_up.qweight, torch.from_numpy(gu["wq"][rows]), shard)
        gate_up.weight_scale.weight_loader(gate_up.weight_scale, torch.from_numpy(gu["w_scale"][rows]), shard)
    gate_up.input_scale.weight_loader(gate_up.input_scale, torch.tensor(np.float32(gu["input_scale"])))
    gate_up.bias.data.copy_(torch.from_numpy(gu["bias"]))
    down_l.qweight.weight_loader(down_l.qweight, torch.from_numpy(down["wq"]))
    down_l.weight_scale.weight_loader(down_l.weight_scale, torch.from_numpy(down["w_scale"]))
    down_l.input_scale.weight_loader(down_l.input_scale, torch.tensor(np.float32(down["input_scale"])))
    down_l.bias.data.copy_(torch.from_numpy(down["bias"]))
    layers = []
    for lay in (gate_up, down_l):
        lay = lay.cuda()
        lay.bias.data = lay.bias.data.to(torch.bfloat16)
        pkg.process_weights_after_loading(lay)
        layers.append(lay)
    gate_up, down_l = layers
    mlp = pkg.FusedFp8MLP(gate_up, down_l)
    x = to_bf16_cuda(gu["x"])
    y = from_bf16(mlp(x))
    g = gate_up(x).float()
    a, b = g.chunk(2, -1)
    sep = from_bf16(down_l((a / (1.0 + torch.exp(-a)) * b).to(torch.bfloat16)))
    ref = O.mlp_w8a8(gu["x"], gu["wq"], gu["w_scale"], gu["input_scale"], gu["bias"],
                     down["wq"], down["w_scale"], down["input_scale"], down["bias"])
    assert_parity(y, ref, "fused mlp layer", ulps=3.0, min_cos=0.9999)
    assert_parity(y, sep, "fused mlp layer vs separate layers", ulps=3.0, min_cos=0.9999)


@pytest.mark.parametrize("m,h,inter,n", [(1, 512, 384, 512), (5, 448, 256, 264), (16, 512, 1408, 520), (3, 3584, 18944, 3584)])
def test_fused_mlp_from_codes_on_decode_rows(m, h, inter, n):
    """Up to 16 pre-quantised rows, with and without the opt-in form in which CTA pairs of the decode kernel take (gate,
    up) tile pairs and write e4m3 h themselves: same bits as the default (a separate silu-multiply-quantise pass), and
    parity with the oracle."""
    Kn = kernels()
    gu, down = make_mlp_case(8200 + m + h + inter, m, h, inter, n)
    d = upload_mlp(gu, down, inter)
    codes = Kn.quantize_activation(d["x"], d["in_gu"])
    args = (codes, d["w_il"], d["s_il"], d["in_gu"], d["b_il"], d["w_d"], d["s_d"], d["in_d"], d["b_d"])
    y = Kn.launch_mlp_w8a8(*args)
    Kn.set_tuning("mlp_decode_fused", 1)
    try:
        y_one = Kn.launch_mlp_w8a8(*args)
    finally:
        Kn.set_tuning("mlp_decode_fused", -1)
    assert torch.equal(y, y_one)
    assert torch.equal(y, Kn.launch_mlp_w8a8(*args))
    ref = O.mlp_w8a8(gu["x"], gu["wq"], gu["w_scale"], gu["input_scale"], gu["bias"],
                     down["wq"], down["w_scale"], down["input_scale"], down["bias"])
    assert_parity(from_bf16(y), ref, f"decode mlp from codes {m}x{h}x{inter}x{n}", ulps=3.0, min_cos=0.9999)
