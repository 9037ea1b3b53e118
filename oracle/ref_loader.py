"""Import of the unmodified reference package from ``oracle/_ref`` (TEST / BENCH INFRASTRUCTURE ONLY).

``oracle/_ref`` is made by ``oracle/make_ref.py`` (a byte-for-byte copy of the reference's ``src/nncf``).
``load()`` puts it on ``sys.path`` and imports it; ``compress_and_pack`` is the reference's own per-weight
step of ``PTWeightCompressionAlgoBackend.transform_model``
(src/nncf/quantization/algorithms/weight_compression/torch_backend.py:463-468 ``compress_weight`` followed by
``decompressor.pack_weight``, :381-404) called on one weight, with nothing of this repository on the path.
Only tests, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` may use this module.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"

_state: dict = {}


def available() -> bool:
    return (REF_DIR / "nncf" / "__init__.py").exists()


def load():
    """Returns the imported reference package, or raises ImportError with the reason."""
    if "nncf" in _state:
        return _state["nncf"]
    if not available():
        msg = "oracle/_ref/nncf is absent: run `python oracle/make_ref.py --reference <checkout>` first"
        raise ImportError(msg)
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    sys.dont_write_bytecode = True
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import logging

    import nncf  # noqa: PLC0415

    logging.getLogger("nncf").setLevel(logging.ERROR)
    if Path(nncf.__file__).resolve().parent != (REF_DIR / "nncf").resolve():
        msg = f"`import nncf` resolved to {nncf.__file__}, not to oracle/_ref"
        raise ImportError(msg)
    _state["nncf"] = nncf
    return nncf


def _api():
    if "api" not in _state:
        load()
        from nncf.parameters import CompressWeightsMode
        from nncf.quantization.algorithms.weight_compression import weight_lowering
        from nncf.quantization.algorithms.weight_compression.config import WeightCompressionConfig
        from nncf.tensor import Tensor
        from nncf.torch.quantization import layers

        _state["api"] = (CompressWeightsMode, WeightCompressionConfig, weight_lowering, Tensor, layers)
    return _state["api"]


def compress_weight(weight, mode: str, group_size: int, reduction_axes=1):
    """The reference's ``compress_weight`` on a torch tensor; returns its ``CompressedWeight``."""
    Mode, Config, wl, Tensor, _ = _api()
    return wl.compress_weight(Tensor(weight), reduction_axes, Config(Mode(mode), group_size))


def compress_and_pack(weight, mode: str, group_size: int):
    """One weight through the reference's compress + pack steps (integer modes, as its torch backend
    supports).  Returns (packed tensor, scale, zero point or None) as torch tensors."""
    Mode, Config, wl, Tensor, layers = _api()
    cfg = Config(Mode(mode), group_size)
    cw = wl.compress_weight(Tensor(weight), 1, cfg)
    if cfg.mode == Mode.INT8_SYM:
        dec = layers.INT8SymmetricWeightsDecompressor(cw.scale.data, result_dtype=weight.dtype)
    elif cfg.mode == Mode.INT8_ASYM:
        dec = layers.INT8AsymmetricWeightsDecompressor(cw.scale.data, cw.zero_point.data, result_dtype=weight.dtype)
    elif cfg.mode == Mode.INT4_SYM:
        dec = layers.INT4SymmetricWeightsDecompressor(
            scale=cw.scale.data, compressed_weight_shape=cw.tensor.shape, result_shape=weight.shape,
            result_dtype=weight.dtype)
    elif cfg.mode == Mode.INT4_ASYM:
        dec = layers.INT4AsymmetricWeightsDecompressor(
            scale=cw.scale.data, zero_point=cw.zero_point.data, compressed_weight_shape=cw.tensor.shape,
            result_shape=weight.shape, result_dtype=weight.dtype)
    else:
        msg = f"the reference's torch backend has no storage format for {mode}"
        raise ValueError(msg)
    packed = dec.pack_weight(cw.tensor.data)
    return packed, cw.scale.data, (cw.zero_point.data if cw.zero_point is not None else None)
