"""GPU tests of the checkpoint exporter's kernels: byte-exact against the oracle's restatement and
against what the reference's exporter itself wrote (fixtures ``weight_quant.npz``, ``checkpoint.npz``),
then a round trip: export -> safetensors -> load_model -> prepack -> forward."""
import importlib
import json

import numpy as np
import pytest
import torch
from torch import nn

from oracle import fp8_oracle as O
from helpers import assert_parity, from_bf16, to_bf16_cuda

pytestmark = pytest.mark.gpu


def export_mod():
    return importlib.import_module("nano-vllm-moe_b200.quantization.export")


def test_weight_quantiser_reproduces_the_reference_exporter(golden):
    g = golden("weight_quant")
    q, s = export_mod().quantize_weight(torch.from_numpy(g["w"]).cuda())
    np.testing.assert_array_equal(q.cpu().numpy(), g["codes"])
    np.testing.assert_array_equal(s.cpu().numpy(), g["scale"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,k", [(80, 64), (257, 1000), (4, 18944), (1, 2)])
def test_weight_quantiser_matches_oracle(n, k, dtype):
    rng = np.random.default_rng(n * 31 + k)
    w = (rng.standard_normal((n, k)) * rng.choice([1e-4, 0.02, 3.0, 500.0], size=(n, 1))).astype(np.float32)
    if n > 3:
        w[1] = 0.0                                   # all-zero channel: scale 1e-8 / 448, codes 0
        w[2, ::3] = -np.abs(w[2]).max()              # the extreme is negative and repeated
        w[3] *= 1e-12                                # below the 1e-8 floor of the maximum
    if dtype == torch.bfloat16:
        w = O.bf16_round(w)
    t = torch.from_numpy(w).to(dtype).cuda()
    q, s = export_mod().quantize_weight(t)
    want_q, want_s = O.quantize_weight_per_channel(w)
    np.testing.assert_array_equal(s.cpu().numpy(), want_s)
    np.testing.assert_array_equal(q.cpu().numpy(), want_q)
    # strided rows (a slice of a wider matrix)
    wide = torch.zeros((n, k + 6), dtype=dtype, device="cuda")
    wide[:, :k] = t
    q2, s2 = export_mod().quantize_weight(wide[:, :k])
    assert torch.equal(q2, q) and torch.equal(s2, s)


def test_abs_max_observer():
    ex = export_mod()
    obs = ex.AmaxObserver()
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn((37, 512), generator=g, device="cuda").to(torch.bfloat16)
    b = (torch.randn((3, 5, 512), generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    c = (torch.randn((9, 100), generator=g, device="cuda") * 7).to(torch.bfloat16)      # 100 columns: padded path
    obs.update("x", a)
    assert obs.amax("x") == float(a.float().abs().max())
    obs.update("x", b)                                                                   # smaller batch: maximum stays
    assert obs.amax("x") == float(a.float().abs().max())
    obs.update("y", c)
    obs.update("y", torch.zeros((0, 100), dtype=torch.bfloat16, device="cuda"))
    assert obs.amax("y") == float(c.float().abs().max())
    # fp32 / fp16 activations keep their own precision (a bf16 cast could round the maximum down)
    f = torch.tensor([[1.00390625, -0.5], [0.25, 1.0]], device="cuda")          # 1 + 2^-8: not a bf16 value
    obs.update("z", f)
    assert obs.amax("z") == 1.00390625
    obs.update("z", f.half() * 0.5)
    assert obs.amax("z") == 1.00390625
    obs.update("z", torch.zeros((0, 2), device="cuda"))
    scales = obs.input_scales()
    assert scales["x"].dtype == torch.float32 and scales["x"].shape == ()
    np.testing.assert_array_equal(scales["x"].numpy(), O.input_scale_from_amax(obs.amax("x")))


def test_export_state_dict_equals_the_reference_exporter(golden):
    g = golden("checkpoint")
    ex = export_mod()
    # rebuild the plain state dict the fixture was exported from: dequantising is not exact, so take the
    # tensors the exporter left alone as they are and re-derive the quantised ones from the generator's seed
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
    plain = _tiny_state_dict()
    tensors = {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in plain.items()}
    in_scales = {}
    for i, (name, t) in enumerate(tensors.items()):
        if ex.should_quantize(name, t):
            in_scales[name[: -len(".weight")]] = torch.tensor(0.01 + 0.001 * i, dtype=torch.float32)
    out, manifest = ex.export_state_dict(tensors, "fp8_w8a8_static", in_scales)
    want = {k[len("ckpt/"):]: g[k] for k in g.files if k.startswith("ckpt/")}
    assert set(out) == set(want)
    for name, t in out.items():
        got = t.float().numpy() if t.dtype in (torch.bfloat16, torch.float32) else t.numpy()
        np.testing.assert_array_equal(got, want[name], err_msg=name)
    assert manifest["quantized_tensors"] == 8 and manifest["scale_tensors"] == ["weight_scale", "input_scale"]


def _tiny_state_dict():
    """Same seeded plain checkpoint as tests/golden/make_golden.py::tiny_state_dict."""
    rng = np.random.default_rng(11)
    hidden, inter = 64, 96
    w = lambda n, k: O.bf16_round((rng.standard_normal((n, k)) * 0.05).astype(np.float32))          # noqa: E731
    pre = "model.layers.0."
    return {
        pre + "self_attn.q_proj.weight": w(64, hidden), pre + "self_attn.k_proj.weight": w(32, hidden),
        pre + "self_attn.v_proj.weight": w(32, hidden), pre + "self_attn.o_proj.weight": w(hidden, 64),
        pre + "self_attn.q_proj.bias": w(1, 64)[0], pre + "self_attn.k_proj.bias": w(1, 32)[0],
        pre + "self_attn.v_proj.bias": w(1, 32)[0],
        pre + "mlp.gate_proj.weight": w(inter, hidden), pre + "mlp.up_proj.weight": w(inter, hidden),
        pre + "mlp.down_proj.weight": w(hidden, inter),
        pre + "input_layernorm.weight": w(1, hidden)[0], "model.norm.weight": w(1, hidden)[0],
        "model.embed_tokens.weight": w(40, hidden), "lm_head.weight": w(40, hidden),
        "model.layers.0.unknown_extra.weight": w(4, 4),
    }


def test_export_load_forward_round_trip(pkg, tmp_path):
    """Plain safetensors checkpoint -> export_checkpoint -> load_model into this package's layers ->
    process_weights_after_loading -> the gate_up layer's output equals the oracle's W8A8 linear on the
    exported codes."""
    from safetensors.torch import save_file
    ex = export_mod()
    loader = importlib.import_module("nano-vllm-moe_b200.utils.loader")
    plain = _tiny_state_dict()
    src, dst = tmp_path / "src", tmp_path / "dst"
    src.mkdir()
    save_file({k: torch.from_numpy(v).to(torch.bfloat16) for k, v in plain.items()}, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"hidden_size": 64}))
    obs = ex.AmaxObserver()
    x = to_bf16_cuda(O.bf16_round(np.random.default_rng(2).standard_normal((24, 64)).astype(np.float32)))
    for base in ("model.layers.0.mlp.gate_proj", "model.layers.0.mlp.up_proj"):
        obs.update(base, x)
    manifest = ex.export_checkpoint(str(src), str(dst), "fp8_w8a8_static", obs.input_scales())
    cfg = json.loads((dst / "config.json").read_text())
    assert cfg["quantization_type"] == "fp8_w8a8_static" and cfg["hidden_size"] == 64
    assert (dst / "quantization_manifest.json").exists() and manifest["quantized_tensors"] == 8

    qcfg = pkg.Fp8Config("fp8_w8a8_static")

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_up_proj = pkg.MergedColumnParallelLinear(64, [96, 96], quant_method=qcfg.get_quant_method(self, "mlp.gate_up_proj"))
            self.down_proj = pkg.RowParallelLinear(96, 64, quant_method=qcfg.get_quant_method(self, "mlp.down_proj"))

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = Mlp()

    class Inner(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Layer()])

    class Model(nn.Module):
        packed_modules_mapping = {"gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}

        def __init__(self):
            super().__init__()
            self.model = Inner()

    model = Model()
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        loader.load_model(model, str(dst))
    model = model.cuda()
    pkg.process_weights_after_loading(model)
    y = from_bf16(model.model.layers[0].mlp.gate_up_proj(x))
    wq = np.concatenate([O.quantize_weight_per_channel(plain["model.layers.0.mlp.gate_proj.weight"])[0],
                         O.quantize_weight_per_channel(plain["model.layers.0.mlp.up_proj.weight"])[0]])
    ws = np.concatenate([O.quantize_weight_per_channel(plain["model.layers.0.mlp.gate_proj.weight"])[1],
                         O.quantize_weight_per_channel(plain["model.layers.0.mlp.up_proj.weight"])[1]])
    in_scale = O.input_scale_from_amax(float(x.float().abs().max()))
    assert_parity(y, O.linear_w8a8(from_bf16(x), wq, ws, in_scale, None), "round trip gate_up")
