"""Binding of libnncf_b200 into an installed reference (``nncf``) at its own implementation seam.

The reference routes five functions of
src/nncf/quantization/algorithms/weight_compression/weight_lowering.py to an alternative implementation
when ``_can_run_optimized(tensor, mode)`` says so (:687-702; call sites :220-223, :271-282, :353-358,
:485-488, :533-545): it then imports the function of the same name from
``nncf.openvino.optimized_functions`` and calls it with ``nncf.tensor.Tensor`` arguments.  ``install()``
uses exactly that seam: it answers True for CUDA torch tensors in the modes the library has and provides a
module under that name whose five functions unwrap the tensors, call the host mirror of this package
(one fused kernel launch each through the C ABI) and wrap the results in the reference's own
``CompressedWeight``.  Everything else of the reference - graph tracing, algorithm orchestration, the
decompressor modules, ``pack_weight`` - runs unchanged, so ``nncf.compress_weights(model_on_cuda, ...)``
becomes the drop-in.  ``uninstall()`` restores the reference.

The reference itself must be importable as ``nncf`` (this package does not ship it).
"""

from __future__ import annotations

import sys
import types
from typing import Optional

import torch

from . import weight_lowering as wl
from .config import WeightCompressionConfig
from .parameters import CompressWeightsMode

_SEAM = "nncf.openvino.optimized_functions"
_INT_MODES = ("int8_sym", "int8_asym", "int4_sym", "int4_asym")
_FLOAT_MODES = ("nf4", "mxfp4", "fp4", "fp8_e4m3", "mxfp8_e4m3")
_installed: dict = {}


def _cfg(config, group_size: Optional[int] = None) -> WeightCompressionConfig:
    return WeightCompressionConfig(CompressWeightsMode(config.mode.value),
                                   config.group_size if group_size is None else group_size)


def _data(t):
    return None if t is None else t.data


def install() -> None:
    """Route the reference's weight lowering of CUDA torch tensors to this library (idempotent)."""
    if _installed:
        return
    from nncf.quantization.algorithms.weight_compression import weight_lowering as ref_wl
    from nncf.quantization.algorithms.weight_compression.parameters import CompressedWeight as RefCompressedWeight
    from nncf.tensor import Tensor
    from nncf.tensor.definitions import TensorBackend

    def on_b200(inp, mode) -> bool:
        return (inp.backend == TensorBackend.torch and isinstance(inp.data, torch.Tensor) and inp.data.is_cuda
                and mode.value in _INT_MODES + _FLOAT_MODES)

    original_can_run = ref_wl._can_run_optimized

    def _can_run_optimized(inp, mode) -> bool:
        return on_b200(inp, mode) or original_can_run(inp, mode)

    def _wrap(cw) -> "RefCompressedWeight":
        return RefCompressedWeight(Tensor(cw.tensor), Tensor(cw.scale),
                                   Tensor(cw.zero_point) if cw.zero_point is not None else None)

    # The reference reshapes a weight into groups before the seam (:482, :217), so the quantisation functions
    # receive [a1, G, gs, a2] with the axis of `gs` as the reduction axis: per-"row" along that axis here.
    def do_integer_quantization(weight, config, reduction_axes=None, precomputed_scale=None,
                                precomputed_zero_point=None):
        cw = wl.do_integer_quantization(weight.data, _cfg(config, -1), reduction_axes, _data(precomputed_scale),
                                        _data(precomputed_zero_point))
        return _wrap(cw)

    def do_float_quantization(weight, config, reduction_axes=None, precomputed_scale=None):
        cw = wl.do_float_quantization(weight.data, _cfg(config, -1), reduction_axes, _data(precomputed_scale))
        return RefCompressedWeight(Tensor(cw.tensor), Tensor(cw.scale))

    # These three are reached before any reshape (:271, :353, :533): the weight is whole and the config's
    # group size applies.
    def integer_quantize_dequantize_weight(weight, config, reduction_axes=None, precomputed_scale=None,
                                           precomputed_zero_point=None, return_compressed_weight=False):
        dq, cw = wl.integer_quantize_dequantize_weight(weight.data, _cfg(config), reduction_axes, _data(precomputed_scale),
                                                       _data(precomputed_zero_point), True)
        return (Tensor(dq), _wrap(cw)) if return_compressed_weight else Tensor(dq)

    def float_quantize_dequantize_weight(weight, config, reduction_axes=None, precomputed_scale=None,
                                         return_compressed_weight=False):
        dq, cw = wl.float_quantize_dequantize_weight(weight.data, _cfg(config), reduction_axes, _data(precomputed_scale),
                                                     True)
        if return_compressed_weight:
            return Tensor(dq), RefCompressedWeight(Tensor(cw.tensor), Tensor(cw.scale))
        return Tensor(dq)

    def get_integer_quantization_error(weight, reduction_axes, config, reduction="max_mean") -> float:
        return wl.get_integer_quantization_error(weight.data, reduction_axes, _cfg(config), reduction)

    seam = types.ModuleType(_SEAM)
    seam.__doc__ = "libnncf_b200 implementations bound at the reference's optimized-function seam"
    for fn in (do_integer_quantization, do_float_quantization, integer_quantize_dequantize_weight,
               float_quantize_dequantize_weight, get_integer_quantization_error):
        setattr(seam, fn.__name__, fn)
    _installed.update(ref_wl=ref_wl, can_run=original_can_run, previous=sys.modules.get(_SEAM))
    sys.modules[_SEAM] = seam
    ref_wl._can_run_optimized = _can_run_optimized


def uninstall() -> None:
    if not _installed:
        return
    _installed["ref_wl"]._can_run_optimized = _installed["can_run"]
    if _installed["previous"] is not None:
        sys.modules[_SEAM] = _installed["previous"]
    else:
        sys.modules.pop(_SEAM, None)
    _installed.clear()
