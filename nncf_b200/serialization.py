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


def record_adapters(module: nn.Module, adapters) -> None:
    """Called when LoRA-correction adapters are attached to a compressed module."""
    getattr(module, _ATTR)["lora_correction"] = {"rank": int(adapters.rank), "int8": bool(adapters.int8)}


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
        if "lora_correction" in entry:
            from .lora_correction import attach_adapters, empty_adapters

            lc = entry["lora_correction"]
            adapters = empty_adapters(out_ch, in_ch, int(lc["rank"]), dtype, bool(lc["int8"]), dev)
            attach_adapters(mod, adapters)
            record_adapters(mod, adapters)
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
        if hasattr(mod, "lora_correction"):
            # y = x W^T + (x A^T) B^T = x (W + B A)^T: the adapters fold into the dense weight
            from .lora_correction import detach_adapters

            with torch.no_grad():
                lc = mod.lora_correction
                dense = (dense.float() + lc.b().float() @ lc.a().float()).to(dense.dtype)
            detach_adapters(mod)
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


# --------------------------------------------------------------------------------------------------
# interchange: reference-compatible state dict, safetensors file, GPTQ-style layout
# --------------------------------------------------------------------------------------------------
_REF_HOOK = "__nncf_hooks.post_hooks.{path}:weight__0.0.{buffer}"


def reference_state_dict(model: nn.Module) -> dict:
    """The model's state dict under the key names the reference gives a compressed torch model
    (src/nncf/torch/function_hook/serialization.py:49-207, hook_storage.py): the packed weight stays at
    ``<module>.weight`` and the decompressor's buffers live at
    ``__nncf_hooks.post_hooks.<module path with ':' for '.'>:weight__0.0._scale`` / ``._zero_point``.
    Tensor contents and shapes are identical in both namings; only the keys differ."""
    out = {}
    compressed = dict(_compressed_modules(model))
    for key, value in model.state_dict().items():
        mod_name, _, rest = key.partition(".parametrizations.weight.")
        if rest and mod_name in compressed:
            if rest == "original":
                out[f"{mod_name}.weight"] = value
            else:  # "0.<buffer>"
                out[_REF_HOOK.format(path=mod_name.replace(".", ":"), buffer=rest.split(".", 1)[1])] = value
        else:
            out[key] = value
    return out


def from_reference_state_dict(model: nn.Module, state: dict) -> dict:
    """Inverse of ``reference_state_dict`` for a model that already carries its decompressors
    (``load_from_config``): keys renamed to this package's parametrization names."""
    out = {}
    compressed = dict(_compressed_modules(model))
    for key, value in state.items():
        if key.startswith("__nncf_hooks.post_hooks."):
            path, _, buffer = key[len("__nncf_hooks.post_hooks."):].partition(":weight__0.0.")
            out[f"{path.replace(':', '.')}.parametrizations.weight.0.{buffer}"] = value
        elif key.endswith(".weight") and key[: -len(".weight")] in compressed:
            out[f"{key[: -len('.weight')]}.parametrizations.weight.original"] = value
        else:
            out[key] = value
    return out


def save_safetensors(model: nn.Module, path: str, reference_keys: bool = True) -> None:
    """One ``.safetensors`` file holding every tensor of the compressed model (reference-compatible key names by
    default) with the manifest needed to rebuild the decompressors (``get_config``) as JSON in the file's
    metadata.  Tensors that share storage (tied weights) are written once each under their own key."""
    import json

    from safetensors.torch import save_file

    state = reference_state_dict(model) if reference_keys else model.state_dict()
    tensors = {k: v.detach().contiguous().cpu().clone() for k, v in state.items()}
    meta = {"nncf_b200_config": json.dumps(get_config(model)), "key_names": "reference" if reference_keys else "nncf_b200"}
    save_file(tensors, path, metadata=meta)


def load_safetensors(model: nn.Module, path: str) -> nn.Module:
    """Rebuilds the compressed model from a freshly constructed dense ``model`` and a file written by
    ``save_safetensors``."""
    import json

    from safetensors import safe_open

    with safe_open(path, framework="pt", device="cpu") as f:
        meta = f.metadata() or {}
        state = {k: f.get_tensor(k) for k in f.keys()}
    if "nncf_b200_config" not in meta:
        msg = f"{path} carries no compression manifest"
        raise ValueError(msg)
    load_from_config(model, json.loads(meta["nncf_b200_config"]))
    if meta.get("key_names") == "reference":
        state = from_reference_state_dict(model, state)
    model.load_state_dict(state)
    return model


def gptq_layout(module: nn.Module) -> dict:
    """The compressed weight of one Linear in the layout GPTQ-style kernels read (the target of the reference's
    converter, src/nncf/experimental/torch/gptqmodel/convertor.py:35-132, which handles INT8 only; here INT4 and
    INT8, symmetric and asymmetric): with ``pack = 32 // bits`` codes per int32, lowest bits first,

        qweight  int32 [in / pack, out]   unsigned codes, packed along the input dimension
        qzeros   int32 [groups, out / pack]  unsigned zero points, packed along the output dimension
        scales   fp16  [groups, out]
        g_idx    int32 [in]               group of every input channel

    so that  W[o, i] = scales[g_idx[i], o] * (code[i, o] - zero[g_idx[i], o]).  Symmetric modes store their
    signed codes with an offset of 2^(bits-1) and that offset as the zero point.  ``out`` must be a multiple of
    ``pack``."""
    if not (parametrize.is_parametrized(module, "weight") and isinstance(module.parametrizations.weight[0],
                                                                        BaseWeightsDecompressor)):
        msg = "the module carries no compressed weight"
        raise ValueError(msg)
    entry = getattr(module, _ATTR)
    cfg = WeightCompressionConfig(CompressWeightsMode(entry["mode"]), entry["group_size"])
    if not cfg.is_integer:
        msg = f"{cfg.mode.value} has no GPTQ-style layout"
        raise ValueError(msg)
    out_ch, in_ch = entry["weight_shape"]
    bits = cfg.num_bits
    pack = 32 // bits
    if out_ch % pack or in_ch % pack:
        msg = f"a [{out_ch}, {in_ch}] weight does not fill whole int32 words of {pack} codes"
        raise ValueError(msg)
    dec = module.parametrizations.weight[0]
    stored = module.parametrizations.weight.original
    gs = cfg.group_size if cfg.group_size != -1 else in_ch
    groups = in_ch // gs
    if bits == 4:
        flat = stored.reshape(-1)
        codes = torch.stack((flat & 15, flat >> 4), dim=-1).reshape(out_ch, in_ch).to(torch.int32)   # unsigned, +8 for sym
    elif cfg.is_asym_mode:
        codes = stored.reshape(out_ch, in_ch).to(torch.int32)
    else:
        codes = stored.reshape(out_ch, in_ch).to(torch.int32) + 128
    if cfg.is_asym_mode:
        zp = dec._zero_point
        if bits == 4:
            zf = zp.reshape(-1)
            zeros = torch.stack((zf & 15, zf >> 4), dim=-1).reshape(-1)[: out_ch * groups].reshape(out_ch, groups).to(torch.int32)
        else:
            zeros = zp.reshape(out_ch, groups).to(torch.int32)
    else:
        zeros = torch.full((out_ch, groups), 1 << (bits - 1), dtype=torch.int32, device=stored.device)
    shifts = (torch.arange(pack, device=stored.device, dtype=torch.int64) * bits)

    def pack_rows(t: torch.Tensor) -> torch.Tensor:
        """[n, m] unsigned values -> int32 [n / pack, m], `pack` consecutive rows per word, lowest bits first."""
        n, m = t.shape
        words = (t.to(torch.int64).reshape(n // pack, pack, m) << shifts.view(1, pack, 1)).sum(dim=1)
        return torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)

    return {"qweight": pack_rows(codes.t().contiguous()),
            "qzeros": pack_rows(zeros.contiguous()).t().contiguous(),
            "scales": dec._scale.reshape(out_ch, groups).t().contiguous().to(torch.float16),
            "g_idx": (torch.arange(in_ch, device=stored.device, dtype=torch.int32) // gs).to(torch.int32),
            "bits": bits, "group_size": cfg.group_size, "sym": not cfg.is_asym_mode}
