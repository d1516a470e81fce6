"""Checkpoint side of the FP8 schemes: what the reference's offline exporter writes
(``scripts/quantization/quantize.py``) produced with this build's CUDA kernels.

The exporter's arithmetic is two reductions and a cast:

* per linear weight ``[N, K]``: ``weight_scale[n] = max(amax_k |w|, 1e-8) / 448`` and
  ``qweight = e4m3(clamp(w / weight_scale, +-448))`` stored as raw bytes
  (``quantize_fp8_per_output_channel``, quantize.py:51-55) -> ``fp8lin_quantize_weight``;
* per linear input (W8A8-static): the maximum ``|x|`` seen during calibration, then
  ``input_scale = max(amax, 1e-8) / 448`` (quantize.py:154-164, :200-203) -> ``fp8lin_abs_max``.

Tensor names, skip rules and the ``config.json`` keys follow the exporter (quantize.py:47-48,
:78-97, :226-246), so a checkpoint written here loads through the reference's loader and through
``nano-vllm-moe_b200.utils.loader`` alike.  Running a model over calibration text is the caller's
business (it needs the model zoo and a dataset): hook ``AmaxObserver.update`` in front of every
linear and pass ``observer.input_scales()`` to ``export_state_dict``.
"""
from __future__ import annotations

import json
import os
import shutil
from pathlib import Path

import torch

from .. import _lib
from . import kernels

FP8_MAX = 448.0
SKIP_KEYS = ("embed_tokens", "lm_head")                 # quantize.py:21
SCHEMES = ("fp8_w8a16", "fp8_w8a8_static")


def should_quantize(name: str, tensor: torch.Tensor) -> bool:
    """2-D ``*.weight`` tensors except the embedding and the LM head (quantize.py:47-48)."""
    return tensor.dim() == 2 and name.endswith(".weight") and not any(k in name for k in SKIP_KEYS)


def quantize_weight(weight: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``weight`` [N, K] bf16 or fp32 on a CUDA device -> (uint8 e4m3 codes [N, K], float32 scale [N])."""
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D [N, K]")
    if not weight.is_cuda:
        raise ValueError("quantize_weight runs on the GPU: move the weight to a CUDA device (no CPU fallback)")
    if weight.dtype not in (torch.bfloat16, torch.float32):
        weight = weight.float()                          # the exporter upcasts too (quantize.py:52)
    if weight.stride(1) != 1:
        weight = weight.contiguous()
    n, k = weight.shape
    if k % 2:
        raise ValueError("K must be even")
    q = torch.empty((n, k), dtype=torch.uint8, device=weight.device)
    scale = torch.empty((n,), dtype=torch.float32, device=weight.device)
    with torch.cuda.device(weight.device):
        rc = _lib.load().fp8lin_quantize_weight(weight.data_ptr(), int(weight.dtype == torch.float32), weight.stride(0),
                                                q.data_ptr(), scale.data_ptr(), n, k, kernels._stream_ptr(weight.device))
    _lib.raise_for(rc, "fp8lin_quantize_weight")
    return q, scale


class AmaxObserver:
    """Running ``max |x|`` per linear, kept on the device (no host sync per batch)."""

    def __init__(self) -> None:
        self._amax: dict[str, torch.Tensor] = {}

    def update(self, name: str, x: torch.Tensor) -> None:
        if not x.is_cuda:
            raise ValueError("AmaxObserver.update needs a CUDA tensor")
        x2 = x.detach().reshape(-1, x.shape[-1])
        if x2.dtype != torch.bfloat16:
            # The reference's hook takes abs().float().max() of the activation in its own dtype (quantize.py make_hook).
            # Rounding an fp32 / fp16 activation to bf16 first could round the maximum DOWN and shrink the scale, so
            # other dtypes are folded in at full precision on the device (calibration only: not a hot path).
            slot = self._amax.get(name)
            if slot is None:
                slot = self._amax[name] = torch.zeros((), dtype=torch.float32, device=x.device)
            if x2.numel():
                torch.maximum(slot, x2.abs().amax().to(torch.float32), out=slot)
            return
        if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.shape[1] % 8:
            x2 = torch.nn.functional.pad(x2, (0, (-x2.shape[1]) % 8)).contiguous()
        slot = self._amax.get(name)
        if slot is None:
            slot = self._amax[name] = torch.zeros((), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            rc = _lib.load().fp8lin_abs_max(x2.data_ptr(), x2.stride(0), x2.shape[0], x2.shape[1], slot.data_ptr(),
                                            kernels._stream_ptr(x.device))
        _lib.raise_for(rc, "fp8lin_abs_max")

    def amax(self, name: str) -> float:
        return float(self._amax[name].item())

    def input_scales(self) -> dict[str, torch.Tensor]:
        """``max(amax, 1e-8) / 448`` per observed linear (quantize.py:200-203), as CPU float32 scalars."""
        # in double on the host and rounded once to float32, exactly as the exporter computes it
        return {name: torch.tensor(max(float(t.item()), 1e-8) / FP8_MAX, dtype=torch.float32) for name, t in self._amax.items()}


def export_state_dict(tensors: dict[str, torch.Tensor], scheme: str, input_scales: dict[str, torch.Tensor] | None = None,
                      device: torch.device | str = "cuda") -> tuple[dict[str, torch.Tensor], dict]:
    """Turn a plain state dict into the exporter's tensor set.

    ``<base>.weight`` of every quantised linear becomes ``<base>.qweight`` (uint8 [N, K]) and
    ``<base>.weight_scale`` (float32 [N]); with ``fp8_w8a8_static`` also ``<base>.input_scale``
    (float32 scalar; 1.0 where calibration supplied none, as ``default_input_scale``).  Other tensors
    pass through.  Returns the tensors (on the CPU) and the manifest the exporter writes beside them.
    """
    if scheme not in SCHEMES:
        raise ValueError(f"Unsupported scheme={scheme!r}")
    out: dict[str, torch.Tensor] = {}
    quantized, skipped, bases = [], [], []
    for name, tensor in tensors.items():
        if should_quantize(name, tensor):
            base = name[: -len(".weight")]
            q, s = quantize_weight(tensor.to(device))
            out[f"{base}.qweight"] = q.cpu()
            out[f"{base}.weight_scale"] = s.cpu()
            bases.append(base)
            quantized.append(name)
        else:
            out[name] = tensor
            skipped.append(name)
    if scheme == "fp8_w8a8_static":
        given = input_scales or {}
        for base in bases:
            scale = given.get(base)
            out[f"{base}.input_scale"] = (scale.to(torch.float32).reshape(()).cpu() if scale is not None
                                          else torch.tensor(1.0, dtype=torch.float32))
    manifest = {
        "scheme": scheme,
        "total_tensors": len(tensors),
        "quantized_tensors": len(quantized),
        "skipped_tensors": len(skipped),
        "quantized_examples": quantized[:20],
        "skipped_examples": skipped[:20],
        "scale_tensors": ["weight_scale"] if scheme == "fp8_w8a16" else ["weight_scale", "input_scale"],
    }
    return out, manifest


def quantization_config(scheme: str) -> dict:
    """The ``quantization_config`` block of ``config.json`` (quantize.py:83-91).  One value differs on
    purpose: the exporter marks ``fp8_w8a8_static`` as ``"export_contract_only"`` because the reference had
    no runtime for it when the exporter was written; here both schemes run, so both say ``"implemented"``."""
    w8a16 = scheme == "fp8_w8a16"
    return {
        "format": scheme,
        "weight_dtype": "float8_e4m3fn",
        "weight_scale": "per_output_channel",
        "activation_dtype": "bfloat16" if w8a16 else "float8_e4m3fn",
        "activation_scale": None if w8a16 else "static_per_linear",
        "runtime_status": "implemented",
        "manifest_file": "quantization_manifest.json",
    }


def export_checkpoint(model_path: str, output_path: str, scheme: str,
                      input_scales: dict[str, torch.Tensor] | None = None, device: torch.device | str = "cuda") -> dict:
    """Directory in, directory out: every ``*.safetensors`` shard of ``model_path`` is read, quantised and
    written as ``output_path/model.safetensors``; the other files are copied and ``config.json`` gains
    ``quantization_type`` / ``quantization_config`` (quantize.py:211-246, :59-97)."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    src, dst = Path(model_path), Path(output_path)
    dst.mkdir(parents=True, exist_ok=True)
    for item in sorted(os.listdir(src)):
        if item.endswith(".safetensors") or item == "model.safetensors.index.json":
            continue
        a, b = src / item, dst / item
        if a.is_dir():
            shutil.copytree(a, b, dirs_exist_ok=True)
        else:
            shutil.copy2(a, b)
    tensors: dict[str, torch.Tensor] = {}
    for shard in sorted(src.glob("*.safetensors")):
        with safe_open(str(shard), "pt", "cpu") as f:
            for key in f.keys():
                tensors[key] = f.get_tensor(key)
    out, manifest = export_state_dict(tensors, scheme, input_scales, device)
    save_file({k: v.contiguous() for k, v in out.items()}, str(dst / "model.safetensors"))
    manifest.update({"source_model_path": str(model_path), "output_path": str(output_path)})
    cfg_path = dst / "config.json"
    config = json.loads(cfg_path.read_text(encoding="utf-8")) if cfg_path.exists() else {}
    config["quantization_type"] = scheme
    config["quantization_config"] = quantization_config(scheme)
    cfg_path.write_text(json.dumps(config, indent=2, ensure_ascii=False) + "\n", encoding="utf-8")
    (dst / "quantization_manifest.json").write_text(json.dumps(manifest, indent=2, ensure_ascii=False) + "\n", encoding="utf-8")
    return manifest
