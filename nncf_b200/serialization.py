"""Carrying a compressed model across processes, and turning it back into a plain one.

The counterpart of the reference's ``nncf.torch.get_config`` / ``nncf.torch.load_from_config``
(src/nncf/torch/function_hook/serialization.py:49-207: the compressed state is the model's ``state_dict``, the
structure needed to rebuild the decompressors travels as a small JSON-able config) and of
``nncf.strip(model, strip_format=StripFormat.IN_PLACE)`` for compressed weights
(src/nncf/torch/function_hook/strip.py:41-203: decompressors are folded away, the model holds ordinary dense
weights again).  Only shapes, modes and dtypes are handled here; the arithmetic stays in the decompressors."""

from __future__ import annotations

from types import SimpleNamespace
from typing import Any, Optional

import torch
from torch import nn
from torch.nn.utils import parametrize

from .config import WeightCompressionConfig
from .decompressors import BaseWeightsDecompressor
from .parameters import CompressWeightsMode

_ATTR = "_nncf_b200_compression"


def _compressed_modules(model: nn.Module):
    for name, mod in model.named_modules():
        if parametrize.is_parametrized(mod, "weight") and isinstance(mod.parametrizations.weight[0], BaseWeightsDecompressor):
            yield name, mod


def record(module: nn.Module, config: WeightCompressionConfig, weight_shape: tuple, dtype: torch.dtype) -> None:
    """Called when a decompressor is installed: remembers what is needed to rebuild it."""
    setattr(module, _ATTR, {"mode": config.mode.value, "group_size": int(config.group_size),
                            "weight_shape": [int(d) for d in weight_shape], "dtype": str(dtype).replace("torch.", "")})


def get_config(model: nn.Module) -> dict:
    """JSON-able description of every compressed weight: module name -> mode, group size, dense shape, dtype.
    Together with ``model.state_dict()`` it restores the compressed model in another process."""
    return {"format": "nncf_b200/1",
            "weights": {name: dict(getattr(mod, _ATTR)) for name, mod in _compressed_modules(model)}}


def load_from_config(model: nn.Module, config: dict, state_dict: Optional[dict] = None) -> nn.Module:
    """Install (empty) decompressors on a freshly built, uncompressed ``model`` as ``config`` describes, so that the
    compressed ``state_dict`` fits; loads it when given.  Mirrors nncf.torch.load_from_config."""
    from .compress_api import _make_decompressor  # shapes of the buffers live next to the code that fills them

    if config.get("format") != "nncf_b200/1":
        msg = f"unknown compression config format {config.get('format')!r}"
        raise ValueError(msg)
    modules = dict(model.named_modules())
    for name, entry in config["weights"].items():
        if name not in modules:
            msg = f"the model has no module named {name!r}"
            raise KeyError(msg)
        mod = modules[name]
        shape = tuple(entry["weight_shape"])
        if tuple(mod.weight.shape) != shape:
            msg = f"{name}: weight shape {tuple(mod.weight.shape)} does not match the recorded {shape}"
            raise ValueError(msg)
        cfg = WeightCompressionConfig(CompressWeightsMode(entry["mode"]), entry["group_size"])
        dtype = getattr(torch, entry["dtype"])
        dev = mod.weight.device
        out_ch, in_ch = shape
        groups = out_ch * (in_ch // cfg.group_size if cfg.group_size != -1 else 1)
        item = SimpleNamespace(scale=torch.zeros(groups, dtype=torch.float32, device=dev),
                               zero_point=torch.zeros(groups, dtype=torch.int32, device=dev),
                               scale_e8m0=torch.zeros(groups, dtype=torch.uint8, device=dev))
        p = SimpleNamespace(compression_config=cfg, weight=torch.empty(shape, dtype=dtype, device="meta"))
        dec = _make_decompressor(p, item).to(dev)
        numel = out_ch * in_ch
        if cfg.num_bits == 4:
            packed = torch.zeros((numel // 2, 1), dtype=torch.uint8, device=dev)
        else:
            signed = cfg.mode == CompressWeightsMode.INT8_SYM
            packed = torch.zeros(shape, dtype=torch.int8 if signed else torch.uint8, device=dev)
        mod.weight.requires_grad_(False)
        mod.weight.data = packed
        parametrize.register_parametrization(mod, "weight", dec, unsafe=True)
        record(mod, cfg, shape, dtype)
    if state_dict is not None:
        model.load_state_dict(state_dict)
    return model


def strip(model: nn.Module) -> nn.Module:
    """Fold every decompressor away: each compressed weight becomes an ordinary dense parameter holding the
    decompressed values (what the compressed model computes with), and the model no longer depends on this
    package.  In place; returns the model."""
    for _, mod in list(_compressed_modules(model)):
        with torch.no_grad():
            dense = mod.weight.detach().clone()  # evaluates the decompressor
        # torch cannot leave a float value in place of the packed uint8 original itself: drop the
        # parametrization with the original restored, then swap the parameter
        parametrize.remove_parametrizations(mod, "weight", leave_parametrized=False)
        mod.weight = nn.Parameter(dense, requires_grad=False)
        if hasattr(mod, _ATTR):
            delattr(mod, _ATTR)
    return model


def compressed_nbytes(model: nn.Module) -> dict[str, Any]:
    """Bytes held by compressed weights (codes + parameters) against their dense size."""
    packed = dense = 0
    for _, mod in _compressed_modules(model):
        entry = getattr(mod, _ATTR)
        packed += mod.parametrizations.weight.original.numel() * mod.parametrizations.weight.original.element_size()
        packed += sum(b.numel() * b.element_size() for b in mod.parametrizations.weight[0].buffers())
        n = 1
        for d in entry["weight_shape"]:
            n *= d
        dense += n * torch.empty(0, dtype=getattr(torch, entry["dtype"])).element_size()
    return {"compressed_bytes": packed, "dense_bytes": dense}
