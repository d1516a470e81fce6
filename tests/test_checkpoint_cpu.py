"""Checkpoint format on the CPU: the loader's name routing against the reference's own loader
(fixture ``checkpoint.npz``: the reference exporter's tensors loaded by the reference's ``load_model``
into a block of its own layer classes at tp=1 and tp=2), and the exporter's host logic (names,
skip rules, config block).  The quantisation kernels themselves are GPU tests."""
import importlib
import warnings

import numpy as np
import pytest
import torch
import torch.distributed as dist
from torch import nn

from oracle import fp8_oracle as O


class FakeTP:
    def __init__(self, size, rank):
        self.size, self.rank = size, rank

    def __enter__(self):
        self.saved = (dist.is_initialized, dist.get_world_size, dist.get_rank)
        dist.is_initialized = lambda: True
        dist.get_world_size = lambda group=None: self.size
        dist.get_rank = lambda group=None: self.rank

    def __exit__(self, *exc):
        dist.is_initialized, dist.get_world_size, dist.get_rank = self.saved


def tiny_block(pkg):
    """The block the fixture was made with, built from this package's layer classes."""
    cfg = pkg.Fp8Config("fp8_w8a8_static")
    hidden, heads, kv_heads, head_dim, inter = 64, 4, 2, 16, 96

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv_proj = pkg.QKVParallelLinear(hidden, head_dim, heads, kv_heads, bias=True,
                                                  quant_method=cfg.get_quant_method(self, "self_attn.qkv_proj"))
            self.o_proj = pkg.RowParallelLinear(heads * head_dim, hidden, quant_method=cfg.get_quant_method(self, "self_attn.o_proj"))

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_up_proj = pkg.MergedColumnParallelLinear(hidden, [inter, inter],
                                                               quant_method=cfg.get_quant_method(self, "mlp.gate_up_proj"))
            self.down_proj = pkg.RowParallelLinear(inter, hidden, quant_method=cfg.get_quant_method(self, "mlp.down_proj"))

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn, self.mlp = Attn(), Mlp()
            self.input_layernorm = nn.LayerNorm(hidden)

    class Inner(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Layer()])
            self.norm = nn.LayerNorm(hidden)

    class Model(nn.Module):
        packed_modules_mapping = {"q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"),
                                  "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}

        def __init__(self):
            super().__init__()
            self.model = Inner()

    return Model()


def write_checkpoint(g, folder):
    from safetensors.torch import save_file
    tensors = {}
    for key in g.files:
        if key.startswith("ckpt/"):
            tensors[key[len("ckpt/"):]] = torch.from_numpy(np.array(g[key]))
    save_file(tensors, str(folder / "model.safetensors"))
    return tensors


@pytest.mark.parametrize("tp,rank", [(1, 0), (2, 0), (2, 1)])
def test_load_model_fills_the_block_like_the_reference_loader(pkg, golden, tmp_path, tp, rank):
    g = golden("checkpoint")
    write_checkpoint(g, tmp_path)
    loader = importlib.import_module("nano-vllm-moe_b200.utils.loader")
    with FakeTP(tp, rank):
        model = tiny_block(pkg)
        with warnings.catch_warnings(record=True) as caught:
            warnings.simplefilter("always")
            unmatched = loader.load_model(model, str(tmp_path))
    named = dict(model.named_parameters())
    named.update(dict(model.named_buffers()))
    tag = f"tp{tp}_r{rank}/"
    loaded = {"qweight", "weight_scale", "input_scale"}
    checked = 0
    for key in g.files:
        if not key.startswith(tag) or key.endswith("__warned__"):
            continue
        name = key[len(tag):]
        if name.rsplit(".", 1)[-1] not in loaded and "norm.weight" not in name and not name.endswith("qkv_proj.bias"):
            continue                                   # never loaded: initial values (LayerNorm bias)
        np.testing.assert_array_equal(named[name].detach().float().numpy() if named[name].dtype != torch.uint8
                                      else named[name].numpy(), g[key], err_msg=name)
        checked += 1
    assert checked >= 15
    # the same names are left over, reported in one warning of the same wording
    want = str(g[tag + "__warned__"][0])
    assert sorted(unmatched) == sorted(want.split(": ", 1)[1].split(", "))
    assert len(caught) == 1 and str(caught[0].message).startswith(f"{len(unmatched)} unmatched checkpoint keys while loading")


def test_route_checkpoint_name():
    loader = importlib.import_module("nano-vllm-moe_b200.utils.loader")
    m = {"q_proj": ("qkv_proj", "q"), "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1)}
    r = loader.route_checkpoint_name
    assert r("model.layers.7.self_attn.q_proj.qweight", m) == ("model.layers.7.self_attn.qkv_proj.qweight", ("q",))
    assert r("model.layers.7.mlp.up_proj.input_scale", m) == ("model.layers.7.mlp.gate_up_proj.input_scale", (1,))
    assert r("model.layers.7.self_attn.o_proj.weight_scale", m) == ("model.layers.7.self_attn.o_proj.weight_scale", ())
    assert r("model.layers.7.self_attn.q_proj.bias", m) == ("model.layers.7.self_attn.qkv_proj.bias", ("q",))
    assert r("model.norm.weight", m) == ("model.norm.weight", ())
    stacked = lambda layer: layer == 2                                                    # noqa: E731
    assert r("model.layers.2.mlp.experts.5.gate_proj.weight", m, stacked) == ("model.layers.2.mlp.w13_stacked", (5, 0))
    assert r("model.layers.2.mlp.experts.5.up_proj.qweight", m, stacked) == ("model.layers.2.mlp.w13_stacked", (5, 1))
    assert r("model.layers.2.mlp.experts.9.down_proj.weight", m, stacked) == ("model.layers.2.mlp.w2_stacked", (9,))
    # a block without stacked expert tensors falls through to the packed-module rule
    want = ("model.layers.3.mlp.experts.5.gate_up_proj.weight", (0,))
    assert r("model.layers.3.mlp.experts.5.gate_proj.weight", m, stacked) == want


def test_exporter_host_logic(golden):
    ex = importlib.import_module("nano-vllm-moe_b200.quantization.export")
    w2 = torch.zeros(4, 8)
    assert ex.should_quantize("model.layers.0.mlp.down_proj.weight", w2)
    assert not ex.should_quantize("model.embed_tokens.weight", w2)
    assert not ex.should_quantize("lm_head.weight", w2)
    assert not ex.should_quantize("model.norm.weight", torch.zeros(8))
    assert not ex.should_quantize("model.layers.0.self_attn.q_proj.bias", torch.zeros(8))
    cfg = ex.quantization_config("fp8_w8a8_static")
    assert cfg["format"] == "fp8_w8a8_static" and cfg["weight_dtype"] == "float8_e4m3fn"
    assert cfg["weight_scale"] == "per_output_channel" and cfg["activation_scale"] == "static_per_linear"
    assert ex.quantization_config("fp8_w8a16")["activation_dtype"] == "bfloat16"
    with pytest.raises(ValueError):
        ex.export_state_dict({}, "int4")
    with pytest.raises(ValueError, match="GPU"):
        ex.quantize_weight(torch.zeros(4, 8))              # no CPU fallback
    # the fixture's tensor set has exactly the names the exporter contract gives
    g = golden("checkpoint")
    names = {k[len("ckpt/"):] for k in g.files if k.startswith("ckpt/")}
    assert "model.layers.0.mlp.gate_proj.qweight" in names and "model.layers.0.mlp.gate_proj.weight" not in names
    assert "model.embed_tokens.weight" in names and "model.embed_tokens.qweight" not in names
    # and its codes are what the oracle's restatement of the exporter gives for the dequantised weight
    q = g["ckpt/model.layers.0.mlp.down_proj.qweight"]; s = g["ckpt/model.layers.0.mlp.down_proj.weight_scale"]
    assert q.dtype == np.uint8 and s.dtype == np.float32 and q.shape == (64, 96) and s.shape == (64,)
    assert np.abs(O.e4m3_decode(q)).max() == 448.0          # every channel's largest element maps to +-448
