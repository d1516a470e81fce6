"""Which checkpoint tensor reaches which weight loader: the name routing of the reference's
``nanovllm/utils/loader.py:40-133`` for the FP8 checkpoint format.

A checkpoint name is ``<module path>.<suffix>`` with suffix ``weight`` | ``qweight`` |
``weight_scale`` | ``input_scale`` (also ``qzeros`` | ``scales``).  If the module path contains a key
of the model's ``packed_modules_mapping`` (``q_proj -> (qkv_proj, "q")``, ``gate_proj ->
(gate_up_proj, 0)`` ...) the tensor goes to the fused module's parameter or buffer of the same
suffix with that shard id; otherwise to the tensor of the same name.  Expert weights
``model.layers.L.mlp.experts.E.{gate,up,down}_proj.<suffix>`` go to the stacked expert tensors of
layer L when the block has them.  Targets may be parameters or buffers (the quantised tensors are
buffers); a target without a ``weight_loader`` is copied into.  Names with no target are
collected and reported in one warning.
"""
from __future__ import annotations

import re
import warnings
from pathlib import Path

import torch
from torch import nn

SUFFIXES = ("qweight", "qzeros", "scales", "weight", "weight_scale", "input_scale")
_EXPERT = re.compile(r"^model\.layers\.(\d+)\.mlp\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.(" + "|".join(SUFFIXES) + r")$")


def _lookup(model: nn.Module, name: str):
    for getter in (model.get_parameter, model.get_buffer):
        try:
            return getter(name)
        except AttributeError:
            continue
    return None


def route_checkpoint_name(name: str, packed_modules_mapping: dict, has_stacked_experts=lambda layer: False):
    """-> (target tensor name, loader arguments after (param, tensor)).

    Pure function of the name: ``("…qkv_proj.qweight", ("q",))``, ``("…o_proj.qweight", ())``,
    ``("model.layers.3.mlp.w13_stacked", (expert, 0))`` ...
    """
    m = _EXPERT.match(name)
    if m is not None and has_stacked_experts(int(m.group(1))):
        prefix = f"model.layers.{m.group(1)}.mlp."
        expert, proj = int(m.group(2)), m.group(3)
        if proj == "down_proj":
            return prefix + "w2_stacked", (expert,)
        return prefix + "w13_stacked", (expert, 0 if proj == "gate_proj" else 1)
    base, dot, last = name.rpartition(".")
    suffix = ""
    if dot and last in SUFFIXES:
        suffix = "." + last
    else:
        base = name
    for key, (fused, shard_id) in packed_modules_mapping.items():
        if key in base:
            return base.replace(key, fused) + suffix, (shard_id,)
    return name, ()


def load_tensor(model: nn.Module, name: str, tensor: torch.Tensor) -> bool:
    """Route one checkpoint tensor into ``model``; False when nothing takes it."""
    mapping = getattr(model, "packed_modules_mapping", {})

    def stacked(layer: int) -> bool:
        try:
            return hasattr(model.get_submodule(f"model.layers.{layer}.mlp"), "w13_stacked")
        except AttributeError:
            return False

    target, args = route_checkpoint_name(name, mapping, stacked)
    param = _lookup(model, target)
    if param is None:
        return False
    loader = getattr(param, "weight_loader", None)
    if loader is None:
        if args:
            raise AttributeError(f"{target} takes shard arguments {args} but has no weight_loader")
        param.data.copy_(tensor)
    else:
        loader(param, tensor, *args)
    return True


def load_model(model: nn.Module, path: str) -> list[str]:
    """Load every ``*.safetensors`` file under ``path``; returns (and warns about) the names nothing took."""
    from safetensors import safe_open

    unmatched: list[str] = []
    for file in sorted(Path(path).glob("*.safetensors")):
        with safe_open(str(file), "pt", "cpu") as f:
            for name in f.keys():
                if not load_tensor(model, name, f.get_tensor(name)):
                    unmatched.append(name)
    if unmatched:
        more = " ..." if len(unmatched) > 8 else ""
        warnings.warn(f"{len(unmatched)} unmatched checkpoint keys while loading {path}: {', '.join(unmatched[:8])}{more}",
                      stacklevel=2)
    return unmatched
