"""Generate the golden fixtures under tests/golden/ from the reference itself.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/nano-vllm-moe

It imports the reference's own Python modules on CPU and records what they
produce on small seeded inputs.  The ``.npz`` files it writes are committed;
the tests only read those files, never the reference checkout.

What is recorded, and which reference code produced it:
  e4m3_codec.npz    torch.float8_e4m3fn casts (the number format itself)
  act_quant.npz     nanovllm/quantization/kernels/fp8.py  quantize_activation_torch
  weight_quant.npz  scripts/quantization/quantize.py      quantize_fp8_per_output_channel
  loaders.npz       nanovllm/quantization/fp8.py Fp8LinearMethod.create_weights + loaders,
                    driven through nanovllm/layers/linear.py layer classes at tp=1 and tp=2
  linear.npz        scripts/debug/debug_ptx_mma.py reference_gemm on the five
                    known-answer patterns; the dequant-then-matmul formula of
                    scripts/quantization/w8a16_linear_microbench.py:47-48; and the
                    epilogue algebra of kernels/fp8.py:331-338 evaluated with torch
  checkpoint.npz    scripts/quantization/quantize.py should_quantize + quantize_fp8_per_output_channel over a
                    tiny state dict, written as safetensors and loaded by nanovllm/utils/loader.py
                    load_model into a block built from the reference's own layer classes (tp=1 and tp=2)
  moe.npz           executor/moe/router.py SoftmaxTopKRouter, experts/eager_experts.py
                    EagerExperts, prepare_finalize/no_ep.py NoEPPrepareFinalize,
                    utils/moe.py moe_align_block_size
  activation.npz    nanovllm/layers/activation.py SiluAndMul.forward, run twice: as plain eager torch
                    (two bf16 roundings: silu, then the product) and through torch.compile as the
                    reference decorates it (one fused fp32 expression, one rounding)
  rmsnorm.npz       nanovllm/layers/layernorm.py RMSNorm.rms_forward / add_rms_forward with bf16
                    weights (the reference builds its models under a bf16 default dtype), eager
                    and compiled

Optional further arguments name the generators to run (codec act_quant weight_quant loaders
linear moe checkpoint activation rmsnorm); without them all run.  The two compiled fixtures need
a host C++ compiler that inductor can use with OpenMP (``CXX=/usr/bin/g++`` in the build
container, whose default g++ wrapper lacks libgomp.spec).
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("NANOVLLM_REFERENCE", ""))
ONLY = set(sys.argv[2:])
if not (REF / "nanovllm").is_dir():
    raise SystemExit("usage: make_golden.py <reference checkout>")
sys.path.insert(0, str(REF))
sys.path.insert(0, str(REF / "scripts" / "quantization"))
sys.path.insert(0, str(REF / "scripts" / "debug"))
sys.path.insert(0, str(REPO))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from oracle import fp8_oracle as O  # noqa: E402  (input generators only)


def bf16_t(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16)


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().to(torch.float32).cpu().numpy()


def codes_t(codes: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(codes, dtype=np.uint8)).view(torch.float8_e4m3fn)


def gen_codec():
    all_codes = np.arange(256, dtype=np.uint8)
    decoded = f32(codes_t(all_codes))
    rng = np.random.default_rng(1)
    vals = np.concatenate([
        rng.standard_normal(4096).astype(np.float32) * 100,
        rng.standard_normal(4096).astype(np.float32),
        rng.standard_normal(4096).astype(np.float32) * 0.01,
        # exact ties between neighbouring codes, both signs
        np.array([(O.E4M3_TABLE[c] + O.E4M3_TABLE[c + 1]) / 2 for c in range(0, 0x7E)], np.float32),
        -np.array([(O.E4M3_TABLE[c] + O.E4M3_TABLE[c + 1]) / 2 for c in range(0, 0x7E)], np.float32),
        np.array([0.0, -0.0, 448.0, -448.0, 463.9, 464.0, 2.0 ** -10, 2.0 ** -9, 3 * 2.0 ** -10, 1e-8], np.float32),
    ])
    enc = torch.from_numpy(vals).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    np.savez_compressed(HERE / "e4m3_codec.npz", decoded=decoded, values=vals, encoded=enc)


def gen_act_quant():
    from nanovllm.quantization.kernels.fp8 import quantize_activation_torch
    rng = np.random.default_rng(2)
    x = np.concatenate([
        rng.standard_normal(8192).astype(np.float32),
        rng.standard_normal(2048).astype(np.float32) * 30,
        np.array([0.0, -0.0, 1.0, -1.0, 5.5, 6.0, 1000.0, -1000.0, 1e-6, 65504.0], np.float32),
    ])
    x = O.bf16_round(x)
    scales = np.array([0.0123, 0.0118, 1.0, 16.0, 1e-13, 0.5, 0.003173828125], np.float32)
    outs = []
    for s in scales:
        q = quantize_activation_torch(bf16_t(x), torch.tensor(s, dtype=torch.float32))
        outs.append(q.view(torch.uint8).numpy())
    np.savez_compressed(HERE / "act_quant.npz", x=x, scales=scales, codes=np.stack(outs))


def gen_weight_quant():
    import quantize as ref_quantize
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((40, 96)) * 0.02).astype(np.float32)
    w[5] = 0.0                      # all-zero channel exercises the 1e-8 clamp
    w[6] *= 1e-6
    w[7, 3] = 3.0
    q, s = ref_quantize.quantize_fp8_per_output_channel(torch.from_numpy(w))
    np.savez_compressed(HERE / "weight_quant.npz", w=w, codes=q.numpy(), scale=s.numpy())


class _FakeDist:
    """Make the reference layers believe they run at a given (tp_size, tp_rank)
    without a process group: they only query world size and rank."""

    def __init__(self, size, rank):
        self.size, self.rank = size, rank

    def __enter__(self):
        self.saved = (dist.is_initialized, dist.get_world_size, dist.get_rank)
        dist.is_initialized = lambda: True
        dist.get_world_size = lambda group=None: self.size
        dist.get_rank = lambda group=None: self.rank
        return self

    def __exit__(self, *exc):
        dist.is_initialized, dist.get_world_size, dist.get_rank = self.saved


def gen_loaders():
    from nanovllm.layers.linear import (ColumnParallelLinear, MergedColumnParallelLinear,
                                        QKVParallelLinear, RowParallelLinear)
    from nanovllm.quantization.fp8 import Fp8Config
    rng = np.random.default_rng(4)
    out = {}
    ckpt = {
        "col_q": rng.integers(0, 256, (80, 64), dtype=np.uint8), "col_s": rng.random(80, dtype=np.float32),
        "gate_q": rng.integers(0, 256, (96, 64), dtype=np.uint8), "gate_s": rng.random(96, dtype=np.float32),
        "up_q": rng.integers(0, 256, (32, 64), dtype=np.uint8), "up_s": rng.random(32, dtype=np.float32),
        "q_q": rng.integers(0, 256, (64, 64), dtype=np.uint8), "q_s": rng.random(64, dtype=np.float32),
        "k_q": rng.integers(0, 256, (32, 64), dtype=np.uint8), "k_s": rng.random(32, dtype=np.float32),
        "v_q": rng.integers(0, 256, (32, 64), dtype=np.uint8), "v_s": rng.random(32, dtype=np.float32),
        "row_q": rng.integers(0, 256, (48, 128), dtype=np.uint8), "row_s": rng.random(48, dtype=np.float32),
        "in_s": np.array(0.0117, np.float32),
    }
    for k, v in ckpt.items():
        out["ckpt_" + k] = v
    T = torch.from_numpy
    for tp in (1, 2):
        for rank in range(tp):
            with _FakeDist(tp, rank):
                cfg = Fp8Config("fp8_w8a8_static")
                col = ColumnParallelLinear(64, 80, bias=True, quant_method=cfg.get_quant_method(None, "col"))
                col.qweight.weight_loader(col.qweight, T(ckpt["col_q"]))
                col.weight_scale.weight_loader(col.weight_scale, T(ckpt["col_s"]))
                col.input_scale.weight_loader(col.input_scale, T(ckpt["in_s"]))
                mrg = MergedColumnParallelLinear(64, [96, 32], quant_method=cfg.get_quant_method(None, "gate_up"))
                for sid, nm in ((0, "gate"), (1, "up")):
                    mrg.qweight.weight_loader(mrg.qweight, T(ckpt[nm + "_q"]), sid)
                    mrg.weight_scale.weight_loader(mrg.weight_scale, T(ckpt[nm + "_s"]), sid)
                mrg.input_scale.weight_loader(mrg.input_scale, T(ckpt["in_s"]))
                qkv = QKVParallelLinear(64, 16, 4, 2, bias=True, quant_method=cfg.get_quant_method(None, "qkv"))
                for sid in ("q", "k", "v"):
                    qkv.qweight.weight_loader(qkv.qweight, T(ckpt[sid + "_q"]), sid)
                    qkv.weight_scale.weight_loader(qkv.weight_scale, T(ckpt[sid + "_s"]), sid)
                qkv.input_scale.weight_loader(qkv.input_scale, T(ckpt["in_s"]))
                row = RowParallelLinear(128, 48, bias=True, quant_method=cfg.get_quant_method(None, "down"))
                row.qweight.weight_loader(row.qweight, T(ckpt["row_q"]))
                row.weight_scale.weight_loader(row.weight_scale, T(ckpt["row_s"]))
                row.input_scale.weight_loader(row.input_scale, T(ckpt["in_s"]))
                # scalar weight scale broadcast (loader fill_ branch)
                col2 = ColumnParallelLinear(64, 80, quant_method=Fp8Config("fp8_w8a16").get_quant_method(None, "c2"))
                col2.weight_scale.weight_loader(col2.weight_scale, torch.tensor([0.25]))
                for nm, layer in (("col", col), ("mrg", mrg), ("qkv", qkv), ("row", row)):
                    tag = f"tp{tp}_r{rank}_{nm}"
                    out[tag + "_qweight"] = layer.qweight.numpy().copy()
                    out[tag + "_weight_scale"] = layer.weight_scale.numpy().copy()
                    out[tag + "_input_scale"] = layer.input_scale.numpy().copy()
                out[f"tp{tp}_r{rank}_col2_weight_scale"] = col2.weight_scale.numpy().copy()
                out[f"tp{tp}_r{rank}_has_input_scale_w8a16"] = np.array(hasattr(col2, "input_scale"))
    np.savez_compressed(HERE / "loaders.npz", **out)


def gen_linear():
    import debug_ptx_mma as ref_debug
    from nanovllm.quantization.kernels.fp8 import quantize_activation_torch
    out = {}
    shapes = [(16, 8, 32), (1, 256, 256), (16, 256, 512), (3, 40, 96)]
    pats = ["ones", "identity", "xones_wramp", "xramp_wones", "ramp"]
    out["kat_shapes"] = np.array(shapes)
    for si, (m, n, k) in enumerate(shapes):
        for p in pats:
            x, wq, s_in, s_w = O.known_answer_case(p, m, n, k)
            ref = ref_debug.reference_gemm(bf16_t(x), codes_t(wq),
                                           torch.tensor([s_in]), torch.tensor([s_w]))
            out[f"kat_{si}_{p}"] = f32(ref)
    # seeded random cases: the dequant-then-matmul formula and the fused-kernel
    # epilogue algebra, both evaluated with torch on CPU
    cases = [(1, 256, 128), (5, 192, 72), (16, 512, 320), (33, 128, 96)]
    out["rand_shapes"] = np.array(cases)
    for ci, (m, k, n) in enumerate(cases):
        c = O.make_case(1000 + ci, m, k, n, calib_rows=64)
        x_t = bf16_t(c["x"]); w_t = codes_t(c["wq"]); ws = torch.from_numpy(c["w_scale"])
        b_t = bf16_t(c["bias"]); s_in = torch.tensor(float(c["input_scale"]), dtype=torch.float32)
        w_kn = w_t.t()
        # w8a16_linear_microbench.py:47-48
        w_bf16 = w_kn.to(torch.bfloat16) * ws.to(torch.bfloat16).unsqueeze(0)
        out[f"rand_{ci}_oref"] = f32(torch.mm(x_t, w_bf16))
        # kernels/fp8.py:57-76 (W8A16): fp32 accumulate, acc*scale + bias, one rounding
        acc = x_t.float() @ w_kn.float()
        out[f"rand_{ci}_w8a16"] = f32((acc * ws[None, :] + b_t.float()[None, :]).to(torch.bfloat16))
        out[f"rand_{ci}_w8a16_nobias"] = f32((acc * ws[None, :]).to(torch.bfloat16))
        # kernels/fp8.py:331-338 (W8A8): acc * in_scale * w_scale + bias
        xq = quantize_activation_torch(x_t, s_in)
        acc8 = xq.float() @ w_kn.float()
        xs = s_in.clamp(min=1e-12)
        out[f"rand_{ci}_w8a8"] = f32((acc8 * xs * ws[None, :] + b_t.float()[None, :]).to(torch.bfloat16))
        out[f"rand_{ci}_xq"] = xq.view(torch.uint8).numpy()
    np.savez_compressed(HERE / "linear.npz", **out)


def gen_moe():
    from types import SimpleNamespace
    from nanovllm.executor.moe.experts.eager_experts import EagerExperts
    from nanovllm.executor.moe.prepare_finalize.no_ep import NoEPPrepareFinalize
    from nanovllm.executor.moe.router import SoftmaxTopKRouter
    from nanovllm.utils.moe import moe_align_block_size
    rng = np.random.default_rng(5)
    T, H, I, E, K = 24, 32, 16, 12, 4
    logits = rng.standard_normal((T, E)).astype(np.float32)
    out = {"logits": logits}
    for ren in (False, True):
        w, ids = SoftmaxTopKRouter(K, ren).select_experts(None, torch.from_numpy(logits))
        out[f"topk_w_ren{int(ren)}"] = w.numpy(); out[f"topk_ids_ren{int(ren)}"] = ids.numpy()
    x = O.bf16_round(rng.standard_normal((T, H)).astype(np.float32))
    w13 = O.bf16_round((rng.standard_normal((E, 2 * I, H)) * 0.2).astype(np.float32))
    w2 = O.bf16_round((rng.standard_normal((E, H, I)) * 0.2).astype(np.float32))
    out.update(x=x, w13=w13, w2=w2)
    w, ids = SoftmaxTopKRouter(K, False).select_experts(None, torch.from_numpy(logits))
    pf = NoEPPrepareFinalize(SimpleNamespace(ep_size=1, tp_size=1, tp_group=None))
    prep = pf.prepare(bf16_t(x), w, ids)
    eo = EagerExperts().apply(prep.hidden_states, prep.topk_ids, prep.topk_weights, bf16_t(w13), bf16_t(w2),
                              local_num_experts=E, local_inter_size=I, hidden_size=H, model_dtype=torch.bfloat16)
    y = pf.finalize(eo, prep, output_shape=(T, H), model_dtype=torch.bfloat16, reduce_tp=False)
    out["moe_out"] = f32(y)
    st, sw, eids, nb = moe_align_block_size(ids, E, 8)
    out.update(align_sorted_token_ids=st.numpy(), align_sorted_weight_idx=sw.numpy(),
               align_expert_ids=eids.numpy(), align_total_blocks=np.array(nb))
    np.savez_compressed(HERE / "moe.npz", **out)


def _eager_and_compiled(fn):
    """Run ``fn`` (a call into a torch.compile-decorated reference method) without and with compilation."""
    import torch._inductor.config as inductor_config
    cxx = os.environ.get("CXX")
    if cxx:
        inductor_config.cpp.cxx = (cxx,)
    with torch.compiler.set_stance("force_eager"):
        eager = fn()
    return eager, fn()


def gen_activation():
    from nanovllm.layers.activation import SiluAndMul
    rng = np.random.default_rng(21)
    parts = [rng.standard_normal((96, 512)).astype(np.float32) * s for s in (0.1, 1.0, 4.0)]
    edge = np.zeros((8, 512), np.float32)
    edge[:, :256] = np.linspace(-30.0, 30.0, 8 * 256, dtype=np.float32).reshape(8, 256)     # gate sweep
    edge[:, 256:] = rng.standard_normal((8, 256)).astype(np.float32) * 3.0
    x = O.bf16_round(np.concatenate(parts + [edge]))
    act = SiluAndMul()
    eager, compiled = _eager_and_compiled(lambda: act(bf16_t(x)))
    np.savez_compressed(HERE / "activation.npz", x=x, eager=f32(eager), compiled=f32(compiled))


def gen_rmsnorm():
    from nanovllm.layers.layernorm import RMSNorm
    rng = np.random.default_rng(22)
    out = {}
    for tag, (rows, hidden, eps) in {"a": (24, 256, 1e-6), "b": (7, 3584, 1e-6), "c": (5, 64, 1e-5)}.items():
        x = O.bf16_round(rng.standard_normal((rows, hidden)).astype(np.float32) * 2.0)
        res = O.bf16_round(rng.standard_normal((rows, hidden)).astype(np.float32))
        w = O.bf16_round(1.0 + 0.25 * rng.standard_normal(hidden).astype(np.float32))
        prev = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)        # as the reference's model runner does before it builds the model
        try:
            norm = RMSNorm(hidden, eps)
        finally:
            torch.set_default_dtype(prev)
        assert norm.weight.dtype == torch.bfloat16
        norm.weight.data.copy_(bf16_t(w))
        e1, c1 = _eager_and_compiled(lambda: norm(bf16_t(x)))
        e2, c2 = _eager_and_compiled(lambda: norm(bf16_t(x), bf16_t(res)))
        out.update({f"{tag}_x": x, f"{tag}_residual": res, f"{tag}_weight": w, f"{tag}_eps": np.float32(eps),
                    f"{tag}_eager": f32(e1), f"{tag}_compiled": f32(c1),
                    f"{tag}_add_eager": f32(e2[0]), f"{tag}_add_compiled": f32(c2[0]),
                    f"{tag}_add_residual_eager": f32(e2[1]), f"{tag}_add_residual_compiled": f32(c2[1])})
    np.savez_compressed(HERE / "rmsnorm.npz", **out)


def _tiny_block(layers_mod, cfg, nn):
    """model.layers.0.{self_attn.{qkv_proj,o_proj}, mlp.{gate_up_proj,down_proj}} + model.norm, the
    fused-module naming of the reference's Qwen2 (models/qwen2.py:193-199)."""
    hidden, heads, kv_heads, head_dim, inter = 64, 4, 2, 16, 96

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv_proj = layers_mod.QKVParallelLinear(hidden, head_dim, heads, kv_heads, bias=True,
                                                         quant_method=cfg.get_quant_method(self, "self_attn.qkv_proj"))
            self.o_proj = layers_mod.RowParallelLinear(heads * head_dim, hidden,
                                                       quant_method=cfg.get_quant_method(self, "self_attn.o_proj"))

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_up_proj = layers_mod.MergedColumnParallelLinear(hidden, [inter, inter],
                                                                      quant_method=cfg.get_quant_method(self, "mlp.gate_up_proj"))
            self.down_proj = layers_mod.RowParallelLinear(inter, hidden, quant_method=cfg.get_quant_method(self, "mlp.down_proj"))

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


def tiny_state_dict():
    """Seeded plain checkpoint of the tiny block (HF naming: separate q/k/v and gate/up)."""
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


def gen_checkpoint():
    import tempfile
    import warnings

    import quantize as ref_export
    from nanovllm.layers import linear as ref_layers
    from nanovllm.quantization.fp8 import Fp8Config
    from nanovllm.utils.loader import load_model
    from safetensors.torch import save_file
    from torch import nn

    state = tiny_state_dict()
    out = {}
    tensors = {}
    in_scales = {}
    for i, (name, arr) in enumerate(state.items()):
        t = torch.from_numpy(arr).to(torch.bfloat16)
        if ref_export.should_quantize(name, t):
            base = name[: -len(".weight")]
            q, s = ref_export.quantize_fp8_per_output_channel(t)
            tensors[base + ".qweight"], tensors[base + ".weight_scale"] = q, s
            in_scales[base] = torch.tensor(0.01 + 0.001 * i, dtype=torch.float32)
            tensors[base + ".input_scale"] = in_scales[base]
        else:
            tensors[name] = t
    for name, t in tensors.items():
        out["ckpt/" + name] = f32(t) if t.dtype == torch.bfloat16 else t.numpy()
    with tempfile.TemporaryDirectory() as tmp:
        save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(tmp, "model.safetensors"))
        for tp in (1, 2):
            for rank in range(tp):
                with _FakeDist(tp, rank):
                    model = _tiny_block(ref_layers, Fp8Config("fp8_w8a8_static"), nn)
                    with warnings.catch_warnings(record=True) as caught:
                        warnings.simplefilter("always")
                        load_model(model, tmp)
                    named = dict(model.named_parameters())
                    named.update(dict(model.named_buffers()))
                    for name, t in named.items():
                        out[f"tp{tp}_r{rank}/" + name] = f32(t) if t.dtype in (torch.bfloat16, torch.float32) else t.numpy()
                    out[f"tp{tp}_r{rank}/__warned__"] = np.array([str(w.message) for w in caught])
    np.savez_compressed(HERE / "checkpoint.npz", **out)


if __name__ == "__main__":
    torch.manual_seed(0)
    torch.set_num_threads(1)
    for name, gen in (("codec", gen_codec), ("act_quant", gen_act_quant), ("weight_quant", gen_weight_quant),
                      ("loaders", gen_loaders), ("linear", gen_linear), ("moe", gen_moe), ("checkpoint", gen_checkpoint),
                      ("activation", gen_activation), ("rmsnorm", gen_rmsnorm)):
        if not ONLY or name in ONLY:
            gen()
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size)
