"""Host-side logic that needs no GPU: buffer/loader parity with the reference
(golden fixtures), the C-ABI surface, and argument validation."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent


class FakeTP:
    """Pretend to be rank ``rank`` of ``size`` without a process group (the
    layers only query world size and rank)."""

    def __init__(self, size, rank):
        self.size, self.rank = size, rank

    def __enter__(self):
        self.saved = (dist.is_initialized, dist.get_world_size, dist.get_rank)
        dist.is_initialized = lambda: True
        dist.get_world_size = lambda group=None: self.size
        dist.get_rank = lambda group=None: self.rank

    def __exit__(self, *exc):
        dist.is_initialized, dist.get_world_size, dist.get_rank = self.saved


def _build_layers(pkg, g, tp, rank):
    T = lambda a: torch.from_numpy(np.array(a))
    with FakeTP(tp, rank):
        cfg = pkg.Fp8Config("fp8_w8a8_static")
        col = pkg.ColumnParallelLinear(64, 80, bias=True, quant_method=cfg.get_quant_method(None, "col"))
        col.qweight.weight_loader(col.qweight, T(g["ckpt_col_q"]))
        col.weight_scale.weight_loader(col.weight_scale, T(g["ckpt_col_s"]))
        col.input_scale.weight_loader(col.input_scale, T(g["ckpt_in_s"]))
        mrg = pkg.MergedColumnParallelLinear(64, [96, 32], quant_method=cfg.get_quant_method(None, "gate_up"))
        for sid, nm in ((0, "gate"), (1, "up")):
            mrg.qweight.weight_loader(mrg.qweight, T(g[f"ckpt_{nm}_q"]), sid)
            mrg.weight_scale.weight_loader(mrg.weight_scale, T(g[f"ckpt_{nm}_s"]), sid)
        mrg.input_scale.weight_loader(mrg.input_scale, T(g["ckpt_in_s"]))
        qkv = pkg.QKVParallelLinear(64, 16, 4, 2, bias=True, quant_method=cfg.get_quant_method(None, "qkv"))
        for sid in ("q", "k", "v"):
            qkv.qweight.weight_loader(qkv.qweight, T(g[f"ckpt_{sid}_q"]), sid)
            qkv.weight_scale.weight_loader(qkv.weight_scale, T(g[f"ckpt_{sid}_s"]), sid)
        qkv.input_scale.weight_loader(qkv.input_scale, T(g["ckpt_in_s"]))
        row = pkg.RowParallelLinear(128, 48, bias=True, quant_method=cfg.get_quant_method(None, "down"))
        row.qweight.weight_loader(row.qweight, T(g["ckpt_row_q"]))
        row.weight_scale.weight_loader(row.weight_scale, T(g["ckpt_row_s"]))
        row.input_scale.weight_loader(row.input_scale, T(g["ckpt_in_s"]))
        col2 = pkg.ColumnParallelLinear(64, 80, quant_method=pkg.Fp8Config("fp8_w8a16").get_quant_method(None, "c2"))
        col2.weight_scale.weight_loader(col2.weight_scale, torch.tensor([0.25]))
    return {"col": col, "mrg": mrg, "qkv": qkv, "row": row, "col2": col2}


@pytest.mark.parametrize("tp,rank", [(1, 0), (2, 0), (2, 1)])
def test_loaders_fill_buffers_like_the_reference(pkg, golden, tp, rank):
    g = golden("loaders")
    layers = _build_layers(pkg, g, tp, rank)
    for nm in ("col", "mrg", "qkv", "row"):
        tag = f"tp{tp}_r{rank}_{nm}"
        lay = layers[nm]
        assert lay.qweight.dtype == torch.uint8 and lay.weight_scale.dtype == torch.float32
        np.testing.assert_array_equal(lay.qweight.numpy(), g[tag + "_qweight"])
        np.testing.assert_array_equal(lay.weight_scale.numpy(), g[tag + "_weight_scale"])
        np.testing.assert_array_equal(lay.input_scale.numpy(), g[tag + "_input_scale"])
    # scalar weight scale: the reference fills element 0 only (the rest of its buffer is
    # uninitialised memory); this build broadcasts the value to every channel
    assert layers["col2"].weight_scale.numpy()[0] == g[f"tp{tp}_r{rank}_col2_weight_scale"][0]
    np.testing.assert_array_equal(layers["col2"].weight_scale.numpy(), np.full(80 // tp, 0.25, np.float32))
    assert hasattr(layers["col2"], "input_scale") == bool(g[f"tp{tp}_r{rank}_has_input_scale_w8a16"])


def test_layer_attributes_match_reference_contract(pkg):
    with FakeTP(2, 1):
        qkv = pkg.QKVParallelLinear(64, 16, 4, 2, quant_method=pkg.Fp8Config().get_quant_method(None))
    assert (qkv.tp_dim, qkv.tp_size, qkv.tp_rank) == (0, 2, 1)
    assert (qkv.num_heads, qkv.num_kv_heads) == (2, 1)
    assert qkv.get_quant_output_offset_size("k") == (32, 16)
    with pytest.raises(AssertionError):
        with FakeTP(8, 0):
            pkg.QKVParallelLinear(3584, 128, 28, 4)          # 28 heads do not divide by 8
    with FakeTP(4, 3):
        row = pkg.RowParallelLinear(128, 48, quant_method=pkg.Fp8Config().get_quant_method(None))
    assert row.tp_dim == 1 and row.input_size_per_partition == 32 and row.qweight.shape == (32, 48)


def test_config_registry(pkg):
    class HF:
        quantization_type = "fp8_w8a8_static"
    cfg = pkg.get_quant_config(HF())
    assert isinstance(cfg, pkg.Fp8Config) and cfg.get_name() == "fp8"
    assert pkg.get_quant_config(object()) is None
    with pytest.raises(ValueError):
        pkg.Fp8Config("int4")
    assert isinstance(cfg.get_quant_method(None, "x"), pkg.QuantizeMethodBase)


def test_apply_raises_on_cpu_like_the_reference(pkg):
    for scheme, text in (("fp8_w8a8_static", "FP8 W8A8 static requires CUDA"), ("fp8_w8a16", "requires CUDA")):
        lay = pkg.ColumnParallelLinear(32, 16, quant_method=pkg.Fp8Config(scheme).get_quant_method(None))
        pkg.process_weights_after_loading(lay)            # no-op on CPU, as in the reference
        with pytest.raises(RuntimeError, match=text):
            lay(torch.zeros(2, 32, dtype=torch.bfloat16))


def test_unquantized_layers_still_work(pkg):
    lay = pkg.ColumnParallelLinear(8, 4, bias=True)
    lay.weight.weight_loader(lay.weight, torch.eye(4, 8))
    lay.bias.weight_loader(lay.bias, torch.ones(4))
    y = lay(torch.ones(2, 8))
    np.testing.assert_allclose(y.detach().numpy(), np.full((2, 4), 2.0))


# ---- the C ABI ----------------------------------------------------------------

def _declared_symbols():
    text = (ROOT / "include" / "fp8lin.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fp8lin_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg._lib.load()
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fp8lin.h but not exported"
        assert n in pkg._lib.SIGNATURES, f"{n} has no ctypes prototype"
    assert lib.fp8lin_version() == 1


def test_argument_validation_without_a_gpu(pkg):
    lib = pkg._lib.load()
    L = pkg._lib
    buf = ctypes.create_string_buffer(4096)
    p = (ctypes.addressof(buf) + 255) & ~255
    # K not a multiple of 16
    rc = lib.fp8lin_w8a8(p, 40, p, p, p, None, p, 64, 1, 40, 64, None, 0, None)
    assert rc == L.ERR_SHAPE and "multiple of 16" in L.last_error()
    rc = lib.fp8lin_w8a16(None, 64, p, p, None, p, 64, 1, 64, 64, None, 0, None)
    assert rc == L.ERR_NULL
    rc = lib.fp8lin_w8a16(p + 2, 64, p, p, None, p, 64, 1, 64, 64, None, 0, None)
    assert rc == L.ERR_ALIGN
    rc = lib.fp8lin_w8a16(p, 32, p, p, None, p, 64, 1, 64, 64, None, 0, None)
    assert rc == L.ERR_SHAPE                                  # ldx < K
    assert lib.fp8lin_w8a16(p, 64, p, p, None, p, 64, 0, 64, 64, None, 0, None) == L.OK   # M == 0: nothing to do
    assert lib.fp8lin_set_tuning(b"no_such_knob", 1) == L.ERR_ARG
    assert lib.fp8lin_prepack_weight(None, p, 64, 64, None) == L.ERR_NULL
    with pytest.raises(ValueError):
        L.raise_for(L.ERR_SHAPE, "x")
    with pytest.raises(RuntimeError):
        L.raise_for(L.ERR_LAUNCH, "x")


def test_workspace_and_variant_queries(pkg):
    lib = pkg._lib.load()
    L = pkg._lib
    assert lib.fp8lin_packed_bytes(2048, 11008) == 2048 * 11008
    assert lib.fp8lin_packed_bytes(448, 576) == 4 * 5 * 16384      # K and N padded to 128
    for scheme in (L.W8A16, L.W8A8_STATIC):
        for m, k, n in [(1, 2048, 2048), (16, 2048, 11008), (256, 11008, 2048), (1024, 2048, 11008), (64, 18944, 3584)]:
            need = lib.fp8lin_workspace_bytes(scheme, m, k, n)
            assert need >= L.WS_HEADER_BYTES and need % 256 == 0
            assert need < (1 << 31)
    assert lib.fp8lin_variant_name(L.W8A8_STATIC, 1024, 2048, 11008).decode().startswith("umma_w8a8_128x")
    assert lib.fp8lin_variant_name(L.W8A8_STATIC, 16, 2048, 11008).decode().startswith("umma_swap_w8a8_m16")
    assert lib.fp8lin_variant_name(L.W8A16, 1, 2048, 2048).decode().startswith("stream_mma_w8a16_m8")


def test_routing_of_large_shapes(pkg):
    """Which kernel family a shape goes to is a pure host function: check the rules that need no device."""
    lib = pkg._lib.load()
    L = pkg._lib
    name = lambda s, m, k, n: lib.fp8lin_variant_name(s, m, k, n).decode()          # noqa: E731
    assert name(L.W8A8_STATIC, 4096, 3584, 37888) == "umma_pair_w8a8_256x256"         # 16 x 148 pair tiles: 32 full rounds
    assert name(L.W8A8_STATIC, 4096, 18944, 3584).startswith("umma_w8a8_128x256_s1+tail")   # 224 pair tiles = 3.03 rounds
    assert name(L.W8A8_STATIC, 1024, 2048, 11008) == "umma_w8a8_128x256_s1+half48"    # 344 tiles: last 48 as halves
    assert name(L.W8A16, 255, 3584, 4608).startswith("stream_mma_w8a16")
    assert name(L.W8A16, 256, 3584, 4608).startswith("umma_w8a16_f16")
    assert name(L.W8A16, 4096, 3584, 37888).endswith("_c5")                            # five chunks of <= 64 MB of f16
    assert name(L.W8A16, 40, 3584, 4608).startswith("umma_swap_w8a16_m64")
    # a 4 MB layer at one row: eight cluster slices of the swapped tcgen05 kernel, all resident at once
    # up to 8 rows on layers of a few MB with a short K: the streaming kernel (cluster hand-over of its split-K sums)
    assert name(L.W8A8_STATIC, 1, 2048, 2048).startswith("stream_mma_w8a8_m8")
    assert name(L.W8A8_STATIC, 8, 3584, 3584).startswith("stream_mma_w8a8_m8")
    assert name(L.W8A8_STATIC, 9, 3584, 3584).startswith("umma_swap_w8a8_m16_s")
    assert name(L.W8A8_STATIC, 1, 2048, 11008).startswith("umma_swap_w8a8_m16_s")    # tcgen05 from the first row elsewhere
    assert name(L.W8A8_STATIC, 1, 18944, 3584) == "umma_swap_w8a8_m16_s8"
    assert name(L.W8A8_STATIC, 1, 3584, 37888) == "umma_swap_w8a8_m16_s1"          # a channel tile for every SM: no split-K
    # W8A16 from 256 rows needs the f16 scratch: activations + one chunk
    need = lib.fp8lin_workspace_bytes(L.W8A16, 4096, 3584, 37888)
    assert need >= L.WS_HEADER_BYTES + 4096 * 3584 * 2 and need <= L.WS_HEADER_BYTES + 4096 * 3584 * 2 + (65 << 20)
    # fused MLP scratch: quantised x and h for large M, plus the bf16 gate_up tensor for decode sizes
    big = lib.fp8lin_mlp_workspace_bytes(4096, 3584, 18944, 3584)
    assert big >= L.WS_HEADER_BYTES + 4096 * (3584 + 18944)
    small = lib.fp8lin_mlp_workspace_bytes(16, 3584, 18944, 3584)
    assert small >= L.WS_HEADER_BYTES + 16 * 18944 * 5


def test_gate_up_interleave_is_a_tile_row_permutation():
    """interleave_gate_up(pack(W)) == pack(W with its 128-row blocks alternating gate / up)."""
    from importlib import import_module
    from oracle import fp8_oracle as O
    K = import_module("nano-vllm-moe_b200.quantization.kernels")
    rng = np.random.default_rng(3)
    inter, k = 384, 200
    wq = rng.integers(0, 255, size=(2 * inter, k), dtype=np.uint8)
    scale = rng.random(2 * inter).astype(np.float32)
    bias = torch.from_numpy(rng.random(2 * inter).astype(np.float32)).to(torch.bfloat16)
    order = np.concatenate([np.r_[g * 128:(g + 1) * 128, inter + g * 128:inter + (g + 1) * 128] for g in range(inter // 128)])
    w_il, s_il, b_il = K.interleave_gate_up(torch.from_numpy(O.pack_tiles(wq)), torch.from_numpy(scale), bias, inter)
    np.testing.assert_array_equal(w_il.numpy(), O.pack_tiles(wq[order]))
    np.testing.assert_array_equal(s_il.numpy(), scale[order])
    assert torch.equal(b_il, bias[torch.from_numpy(order)])
    with pytest.raises(ValueError):
        K.interleave_gate_up(torch.from_numpy(O.pack_tiles(wq)), torch.from_numpy(scale), None, 200)


def test_fused_mlp_wrapper_checks_its_layers(pkg):
    cfg = pkg.Fp8Config("fp8_w8a8_static")
    gate_up = pkg.MergedColumnParallelLinear(64, [128, 128], quant_method=cfg.get_quant_method(None, "mlp.gate_up_proj"))
    down = pkg.RowParallelLinear(128, 64, quant_method=cfg.get_quant_method(None, "mlp.down_proj"))
    with pytest.raises(ValueError, match="process_weights_after_loading"):
        pkg.FusedFp8MLP(gate_up, down)                     # not prepacked (CPU-resident layers never are)
    plain = pkg.RowParallelLinear(128, 64)
    with pytest.raises(ValueError):
        pkg.FusedFp8MLP(gate_up, plain)                    # unquantised projection


def test_kernels_refuse_cpu_tensors(pkg):
    from importlib import import_module
    K = import_module("nano-vllm-moe_b200.quantization.kernels")
    x = torch.zeros(2, 32, dtype=torch.bfloat16)
    w = torch.zeros(16384, dtype=torch.uint8)
    s = torch.ones(16)
    with pytest.raises(ValueError, match="CUDA"):
        K.launch_w8a16_gemm(x, w, s)
    with pytest.raises(ValueError, match="CUDA"):
        K.launch_w8a8_gemm(x, w, torch.ones(()), s)


def test_decode_planners_give_well_formed_plans(pkg):
    """The slice planners of the decode kernels are pure host functions: over a grid of shapes every plan names a
    kernel, its split factor is 1..8 (cluster size) and never larger than the number of 128-element K blocks, and the
    workspace it asks for is bounded by the header plus one quantised copy of the activations."""
    import re
    lib = pkg._lib.load()
    L = pkg._lib
    rng = np.random.default_rng(11)
    shapes = [(m, k, n) for m in (1, 3, 8, 9, 16, 17, 32, 33, 64)
              for k, n in ((16, 8), (448, 576), (1408, 2048), (2048, 2048), (2048, 11008), (3584, 4608), (3584, 37888), (18944, 3584))]
    shapes += [(int(rng.integers(1, 65)), 16 * int(rng.integers(1, 1200)), int(rng.integers(1, 40000))) for _ in range(200)]
    for scheme in (L.W8A16, L.W8A8_STATIC):
        for m, k, n in shapes:
            name = lib.fp8lin_variant_name(scheme, m, k, n).decode()
            assert name.startswith(("stream_mma_", "umma_swap_")), (scheme, m, k, n, name)
            s = int(re.search(r"_s(\d+)", name).group(1))
            kblocks = -(-k // 128)
            if name.startswith("umma_swap_"):
                assert 1 <= s <= 8 and s <= kblocks, (m, k, n, name)
                assert f"_m{16 if m <= 16 else 32 if m <= 32 else 64}_" in name, (m, k, n, name)
            else:
                assert 1 <= s <= max(1, -(-k // 256)), (m, k, n, name)
                if m <= 16:
                    assert s <= 8, (m, k, n, name)          # up to 16 rows the slices form a cluster
            need = lib.fp8lin_workspace_bytes(scheme, m, k, n)
            assert L.WS_HEADER_BYTES <= need <= L.WS_HEADER_BYTES + max(m * k + 256, 8 * m * n * 4 * 8 + 4096), (m, k, n, need)
