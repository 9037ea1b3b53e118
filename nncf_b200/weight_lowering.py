"""Host-side mirror of the reference's weight-lowering interface
(src/nncf/quantization/algorithms/weight_compression/weight_lowering.py, "WC/weight_lowering.py"
below): same function names, argument meaning, result shapes and error behaviour, with the
arithmetic done by one fused CUDA kernel launch per call (``nncfb_quantize``) instead of a chain
of tensor operations.  Inputs are CUDA tensors (fp32 / fp16 / bf16); there is no CPU path.
"""

from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

from . import _lib
from .config import CompressedWeight, WeightCompressionConfig
from .errors import InternalError, InvalidGroupSizeError, UnsupportedModelError
from .parameters import CompressWeightsMode

ReductionAxes = Union[int, Sequence[int]]

_SUPPORTED_FLOAT = (CompressWeightsMode.NF4, CompressWeightsMode.MXFP4, CompressWeightsMode.FP4,
                    CompressWeightsMode.FP8_E4M3, CompressWeightsMode.MXFP8_E4M3)


def get_reduction_channel_size(weight_shape: Sequence[int], reduction_axes: ReductionAxes) -> tuple[int, int]:
    """WC/weight_lowering.py:40-54."""
    if isinstance(reduction_axes, (tuple, list)) and len(reduction_axes) == 1:
        reduction_axes = reduction_axes[0]
    if not isinstance(reduction_axes, int):
        msg = f"Group-wise quantization expects a single reduction axis, but given: {reduction_axes}."
        raise UnsupportedModelError(msg)
    return weight_shape[reduction_axes], reduction_axes


def reshape_weight_for_grouped_quantization(weight: torch.Tensor, reduction_axes: ReductionAxes,
                                            group_size: int) -> tuple[torch.Tensor, int]:
    """[a1, r, a2] -> [a1, r // gs, gs, a2] (a view) and the new reduction axis.  WC/weight_lowering.py:57-81."""
    assert group_size != -1
    channel_size, axis = get_reduction_channel_size(tuple(weight.shape), reduction_axes)
    if channel_size % group_size != 0:
        msg = f"Channel size {channel_size} should be divisible by size of group {group_size}."
        raise InvalidGroupSizeError(msg)
    axis = axis % weight.ndim
    shape = list(weight.shape)
    shape[axis:axis + 1] = (channel_size // group_size, group_size)
    return weight.reshape(shape), axis + 1


def ungroup_weights(weights: torch.Tensor, reduction_axis: int) -> torch.Tensor:
    """WC/weight_lowering.py:410-425."""
    shape = list(weights.shape)
    shape[reduction_axis] = shape[reduction_axis] * shape[reduction_axis + 1]
    shape[reduction_axis + 1] = 1
    return weights.reshape(shape).squeeze()


# ------------------------------------------------------------------------------------------------
# the single gateway to the kernel
# ------------------------------------------------------------------------------------------------
def _check_weight(weight: torch.Tensor) -> torch.Tensor:
    if not isinstance(weight, torch.Tensor):
        msg = f"expected a torch.Tensor, got {type(weight)}"
        raise TypeError(msg)
    if not weight.is_cuda:
        msg = "nncf_b200 compresses CUDA tensors only: there is no CPU fallback"
        raise ValueError(msg)
    if weight.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        weight = weight.float()
    return weight.contiguous()


def _axis_split(shape: Sequence[int], axis: int) -> tuple[int, int, int]:
    outer = 1
    for d in shape[:axis]:
        outer *= d
    inner = 1
    for d in shape[axis + 1:]:
        inner *= d
    return outer, shape[axis], inner


def _infer_axis_from_params(weight_shape: Sequence[int], param_shape: Sequence[int]) -> int:
    """Reduction axis of an already grouped weight, deduced from the broadcast shape of the
    precomputed scale: the one axis where the scale has extent 1 and the weight does not."""
    if len(param_shape) != len(weight_shape):
        msg = f"precomputed scale of shape {tuple(param_shape)} does not broadcast over weight {tuple(weight_shape)}"
        raise ValueError(msg)
    axes = [i for i, (w, p) in enumerate(zip(weight_shape, param_shape)) if p == 1 and w != 1]
    for i, (w, p) in enumerate(zip(weight_shape, param_shape)):
        if p not in (1, w):
            msg = f"precomputed scale of shape {tuple(param_shape)} does not broadcast over weight {tuple(weight_shape)}"
            raise ValueError(msg)
    if len(axes) > 1:
        msg = "precomputed parameters must share one reduction axis"
        raise UnsupportedModelError(msg)
    if axes:
        return axes[0]
    # every element has its own parameters (e.g. a single column): any unit axis works
    ones = [i for i, w in enumerate(weight_shape) if w == 1]
    return ones[-1] if ones else len(weight_shape) - 1


def quantize_launch(
    weight: torch.Tensor,
    config: WeightCompressionConfig,
    reduction_axis: int,
    group_size: int,
    precomputed_scale: Optional[torch.Tensor] = None,
    precomputed_zero_point: Optional[torch.Tensor] = None,
    *,
    want_codes: str = "byte",
    want_values: bool = False,
    want_dq: bool = False,
    want_sqerr: bool = False,
    want_scale_f16: bool = False,
    want_params: bool = True,
    want_zp_packed: bool = False,
) -> dict:
    """One ``nncfb_quantize`` launch on ``weight`` viewed as [outer, reduce, inner] around
    ``reduction_axis`` with groups of ``group_size`` (must divide the axis).

    Returns a dict of flat/unshaped outputs: codes, scale, zp, values, dq, sqerr, scale_f16,
    scale_e8m0 plus 'param_shape' (keepdims-style shape of per-group tensors for an
    ungrouped weight: the reduction axis replaced by the number of groups)."""
    weight = _check_weight(weight)
    mode_id = _lib.MODE_IDS.get(config.mode.value)
    if mode_id is None:
        msg = f"{config.mode.value} is not supported."
        raise InternalError(msg)
    axis = reduction_axis % weight.ndim
    outer, reduce, inner = _axis_split(tuple(weight.shape), axis)
    if reduce % group_size != 0:
        msg = f"Channel size {reduce} should be divisible by size of group {group_size}."
        raise InvalidGroupSizeError(msg)
    n_groups = outer * (reduce // group_size) * inner
    dev = weight.device
    n = weight.numel()
    args = _lib.QuantizeArgs()
    args.weight = _lib.ptr(weight)
    args.weight_dtype = _lib.DTYPE_IDS[weight.dtype]
    args.mode = mode_id
    args.outer, args.reduce, args.inner, args.group_size = outer, reduce, inner, group_size
    keep = [weight]
    out: dict = {}
    if precomputed_scale is not None:
        ps = precomputed_scale.to(device=dev, dtype=torch.float32).contiguous()
        if ps.numel() != n_groups:
            msg = f"precomputed scale has {ps.numel()} elements, expected {n_groups}"
            raise ValueError(msg)
        keep.append(ps)
        args.pre_scale = _lib.ptr(ps)
    if precomputed_zero_point is not None and config.is_asym_mode:
        pz = precomputed_zero_point.to(device=dev)
        if pz.dtype == torch.float32:
            args.pre_zp_dtype = _lib.F32
        else:
            pz = pz.to(torch.int32)
            args.pre_zp_dtype = _lib.I32
        pz = pz.contiguous()
        if pz.numel() != n_groups:
            msg = f"precomputed zero point has {pz.numel()} elements, expected {n_groups}"
            raise ValueError(msg)
        keep.append(pz)
        args.pre_zp = _lib.ptr(pz)
    four_bit = config.num_bits == 4
    if want_codes == "nibble":
        nibble_ok = four_bit and n % 2 == 0 and ((inner > 1 and inner % 2 == 0) or (inner == 1 and group_size % 2 == 0))
        if not nibble_ok:
            want_codes = "byte+pack"
    if want_codes in ("byte", "byte+pack"):
        signed = config.is_integer and not config.is_asym_mode
        out["codes"] = torch.empty(n, dtype=torch.int8 if signed else torch.uint8, device=dev)
        args.codes_format = _lib.CODES_BYTE
        args.codes_out = _lib.ptr(out["codes"])
    elif want_codes == "nibble":
        out["packed"] = torch.empty(n // 2, dtype=torch.uint8, device=dev)
        args.codes_format = _lib.CODES_NIBBLE
        args.codes_out = _lib.ptr(out["packed"])
    else:
        args.codes_format = _lib.CODES_NONE
    if want_params:
        out["scale"] = torch.empty(n_groups, dtype=torch.float32, device=dev)
        args.scale_out = _lib.ptr(out["scale"])
        if config.is_asym_mode:
            out["zp"] = torch.empty(n_groups, dtype=torch.int32, device=dev)
            args.zp_out = _lib.ptr(out["zp"])
        if config.mode in (CompressWeightsMode.MXFP4, CompressWeightsMode.MXFP8_E4M3):
            out["scale_e8m0"] = torch.empty(n_groups, dtype=torch.uint8, device=dev)
            args.scale_e8m0_out = _lib.ptr(out["scale_e8m0"])
    if want_scale_f16:
        out["scale_f16"] = torch.empty(n_groups, dtype=torch.float16, device=dev)
        args.scale_f16_out = _lib.ptr(out["scale_f16"])
    if want_zp_packed and config.is_integer and config.is_asym_mode:
        # the decompressor's `_zero_point` buffer: uint8 per group, or two 4-bit groups per byte
        nbytes = (n_groups + 7) // 8 * 4 if four_bit else n_groups
        out["zp_packed"] = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        args.zp_packed_out = _lib.ptr(out["zp_packed"])
    if want_values:
        out["values"] = torch.empty(n, dtype=torch.float32, device=dev)
        args.values_out = _lib.ptr(out["values"])
    if want_dq:
        out["dq"] = torch.empty(n, dtype=torch.float32, device=dev)
        args.dq_out = _lib.ptr(out["dq"])
    if want_sqerr:
        out["sqerr"] = torch.empty(n_groups, dtype=torch.float32, device=dev)
        args.sqerr_out = _lib.ptr(out["sqerr"])
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.nncfb_quantize(args, _lib.stream_handle(dev)))
        if want_codes == "byte+pack" and four_bit and n % 2 == 0:
            out["packed"] = torch.empty(n // 2, dtype=torch.uint8, device=dev)
            add = 8 if config.mode == CompressWeightsMode.INT4_SYM else 0
            _lib.check(_lib.lib.nncfb_pack_nibbles(_lib.ptr(out["codes"]), n, add, _lib.ptr(out["packed"]),
                                                   _lib.stream_handle(dev)))
    del keep
    shape = list(weight.shape)
    shape[axis] = reduce // group_size
    out["param_shape"] = tuple(shape)
    return out


class _MultiAxis:
    """Several reduction axes at once (convolutions: every axis but the output channel,
    src/nncf/torch/model_graph_manager.py:374-380; always per channel, never grouped).  The weight is viewed as
    [kept, reduced]: kept axes first, reduced axes flattened behind them.  For the usual layout (reduced axes
    trailing) that is a free reshape; otherwise (transposed convolutions keep axis 1) one permuted copy.  The
    kernel then sees an ordinary per-row problem and the results are shaped back."""

    def __init__(self, weight: torch.Tensor, axes: Sequence[int]):
        nd = weight.ndim
        self.reduced = sorted({a % nd for a in axes})
        self.kept = [i for i in range(nd) if i not in self.reduced]
        self.perm = self.kept + self.reduced
        self.shape = tuple(weight.shape)
        kept_n = 1
        for i in self.kept:
            kept_n *= self.shape[i]
        self.flat = weight.permute(self.perm).contiguous().reshape(kept_n, -1)
        self.param_shape = tuple(1 if i in self.reduced else d for i, d in enumerate(self.shape))

    def restore(self, t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """[kept, reduced]-shaped result -> the weight's own layout."""
        if t is None:
            return None
        inv = [0] * len(self.perm)
        for pos, ax in enumerate(self.perm):
            inv[ax] = pos
        return t.reshape([self.shape[i] for i in self.perm]).permute(inv).contiguous()

    def params(self, t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        return None if t is None else t.reshape(self.param_shape)

    def flat_params(self, t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        return None if t is None else t.reshape(-1, 1)


def _multi_axis(weight: torch.Tensor, config: WeightCompressionConfig, reduction_axes) -> Optional[_MultiAxis]:
    if not isinstance(reduction_axes, (tuple, list)) or len(reduction_axes) <= 1:
        return None
    if config.group_size != -1:
        msg = f"Group-wise quantization expects a single reduction axis, but given: {reduction_axes}."
        raise UnsupportedModelError(msg)
    return _MultiAxis(weight, reduction_axes)


def _grouped(weight: torch.Tensor, config: WeightCompressionConfig, reduction_axes, scale):
    """Resolves (weight as the caller will see it, axis into it, group size along that axis)."""
    if config.group_size != -1 and reduction_axes is not None:
        grouped, axis = reshape_weight_for_grouped_quantization(weight, reduction_axes, config.group_size)
        return grouped, axis, config.group_size
    if reduction_axes is not None:
        if isinstance(reduction_axes, (tuple, list)):
            if len(reduction_axes) != 1:
                msg = f"a single reduction axis is supported, got {reduction_axes}"
                raise UnsupportedModelError(msg)
            reduction_axes = reduction_axes[0]
        axis = reduction_axes % weight.ndim
        return weight, axis, weight.shape[axis]
    if scale is None:
        msg = "Reduction axes are required for computing the scale and (zero point) vectors."
        raise ValueError(msg)
    axis = _infer_axis_from_params(tuple(weight.shape), tuple(scale.shape))
    return weight, axis, weight.shape[axis]


def _keepdims_shape(weight_shape: Sequence[int], axis: int) -> tuple:
    s = list(weight_shape)
    s[axis] = 1
    return tuple(s)


# ------------------------------------------------------------------------------------------------
# integer modes
# ------------------------------------------------------------------------------------------------
def calculate_integer_quantization_params(weight: torch.Tensor, reduction_axes: ReductionAxes,
                                          config: WeightCompressionConfig):
    """Scale (fp32, keepdims) and zero point (int32 or None).  WC/weight_lowering.py:292-326."""
    if not config.is_integer:
        msg = "The function supports integer quantization only"
        raise InternalError(msg)
    ma = _multi_axis(weight, WeightCompressionConfig(config.mode, -1), reduction_axes)
    if ma is not None:
        scale, zp = calculate_integer_quantization_params(ma.flat, 1, config)
        return ma.params(scale), ma.params(zp)
    w, axis, gs = _grouped(weight, WeightCompressionConfig(config.mode, -1), reduction_axes, None)
    o = quantize_launch(w, config, axis, gs, want_codes="none")
    shape = _keepdims_shape(w.shape, axis)
    zp = o["zp"].reshape(shape) if config.is_asym_mode else None
    return o["scale"].reshape(shape), zp


def do_integer_quantization(weight: torch.Tensor, config: WeightCompressionConfig,
                            reduction_axes: Optional[ReductionAxes] = None,
                            precomputed_scale: Optional[torch.Tensor] = None,
                            precomputed_zero_point: Optional[torch.Tensor] = None) -> CompressedWeight:
    """WC/weight_lowering.py:451-508: codes int8 (symmetric) / uint8 (asymmetric) in the grouped
    shape, fp32 scale and int32 zero point with keepdims shapes."""
    cw, _ = _integer(weight, config, reduction_axes, precomputed_scale, precomputed_zero_point, dq=False)
    return cw


def _integer(weight, config, reduction_axes, precomputed_scale, precomputed_zero_point, dq: bool, sqerr: bool = False):
    if not config.is_integer:
        msg = "The function supports integer quantization only"
        raise InternalError(msg)
    if config.is_asym_mode and (precomputed_scale is None) != (precomputed_zero_point is None):
        msg = ("If precomputed quantization parameters are provided, both scale and zero point are required "
               "for asymmetric quantization.")
        raise ValueError(msg)
    ma = _multi_axis(weight, config, reduction_axes)
    if ma is not None:
        cw, extra = _integer(ma.flat, config, 1, ma.flat_params(precomputed_scale), ma.flat_params(precomputed_zero_point),
                             dq, sqerr)
        cw = CompressedWeight(ma.restore(cw.tensor), ma.params(cw.scale), ma.params(cw.zero_point))
        extra = {"dq": ma.restore(extra["dq"]), "sqerr": extra["sqerr"], "shape": ma.shape, "axis": None}
        return cw, extra
    w, axis, gs = _grouped(weight, config, reduction_axes, precomputed_scale)
    o = quantize_launch(w, config, axis, gs, precomputed_scale, precomputed_zero_point, want_codes="byte",
                        want_dq=dq, want_sqerr=sqerr)
    pshape = _keepdims_shape(w.shape, axis)
    scale = precomputed_scale if precomputed_scale is not None else o["scale"].reshape(pshape)
    zp = None
    if config.is_asym_mode:
        zp = precomputed_zero_point if precomputed_zero_point is not None else o["zp"].reshape(pshape)
    cw = CompressedWeight(o["codes"].reshape(w.shape), scale, zp)
    extra = {"dq": o["dq"].reshape(w.shape) if dq else None, "sqerr": o.get("sqerr"), "shape": w.shape, "axis": axis}
    return cw, extra


def do_integer_dequantization(compressed_weights: CompressedWeight, reduction_axis: int = -1) -> torch.Tensor:
    """(int32(q) - zp) as the scale's dtype, times scale.  WC/weight_lowering.py:428-448.
    Elementwise torch expression: it is not on the compression hot path (the run-time twin is
    the decompression kernel)."""
    t, zp, s = compressed_weights.tensor, compressed_weights.zero_point, compressed_weights.scale
    d = t.to(torch.int32) - zp if zp is not None else t
    d = d.to(s.dtype) * s
    if reduction_axis > -1:
        d = ungroup_weights(d, reduction_axis)
    return d


def integer_quantize_dequantize_weight(weight: torch.Tensor, config: WeightCompressionConfig,
                                       reduction_axes: Optional[ReductionAxes] = None,
                                       precomputed_scale: Optional[torch.Tensor] = None,
                                       precomputed_zero_point: Optional[torch.Tensor] = None,
                                       return_compressed_weight: Optional[bool] = False):
    """Quantise then dequantise to fp32 in the same kernel launch.  WC/weight_lowering.py:511-554."""
    cw, extra = _integer(weight, config, reduction_axes, precomputed_scale, precomputed_zero_point, dq=True)
    if return_compressed_weight:
        return extra["dq"], cw
    return extra["dq"]


def get_integer_quantization_error(weight: torch.Tensor, reduction_axes: ReductionAxes,
                                   config: WeightCompressionConfig, reduction: str = "max_mean") -> float:
    """max over channels of mean((dq - w)^2) or the Frobenius norm of dq - w.
    WC/weight_lowering.py:329-374.  The kernel emits per-group sums of squared error while it
    quantises; only those few values are reduced here."""
    if reduction not in ("max_mean", "frobenius"):
        msg = f"Unsupported aggregation mode: {reduction}."
        raise InternalError(msg)
    if not config.is_integer:
        msg = "The function supports integer quantization only"
        raise InternalError(msg)
    ma = _multi_axis(weight, config, reduction_axes)
    if ma is not None:
        return get_integer_quantization_error(ma.flat, 1, config, reduction)
    w, axis, gs = _grouped(weight, config, reduction_axes, None)
    o = quantize_launch(w, config, axis, gs, want_codes="none", want_sqerr=True, want_params=False)
    sq = o["sqerr"].reshape(_keepdims_shape(w.shape, axis))
    if reduction == "frobenius":
        return float(sq.double().sum().sqrt().item())
    # mean over the *original* reduction axis: sum the groups of each channel
    channel_size, orig_axis = get_reduction_channel_size(tuple(weight.shape), reduction_axes)
    if config.group_size != -1:
        sq = sq.sum(dim=axis - 1, keepdim=True)
    return float((sq / channel_size).max().item())


# ------------------------------------------------------------------------------------------------
# float (code-book) modes
# ------------------------------------------------------------------------------------------------
def calculate_float_quantization_params(weight: torch.Tensor, reduction_axes: ReductionAxes,
                                        config: WeightCompressionConfig, signed: bool = False) -> torch.Tensor:
    """Scale for NF4 / FP4 / MXFP4 / FP8 / MXFP8.  WC/weight_lowering.py:84-128."""
    assert not config.is_integer
    if signed:
        msg = "signed scales are used by code-book modes only, which are not supported"
        raise InternalError(msg)
    ma = _multi_axis(weight, WeightCompressionConfig(config.mode, -1), reduction_axes)
    if ma is not None:
        return ma.params(calculate_float_quantization_params(ma.flat, 1, config))
    w, axis, gs = _grouped(weight, WeightCompressionConfig(config.mode, -1), reduction_axes, None)
    o = quantize_launch(w, config, axis, gs, want_codes="none")
    return o["scale"].reshape(_keepdims_shape(w.shape, axis))


def _float(weight, config, reduction_axes, precomputed_scale, dq: bool):
    assert not config.is_integer
    if config.mode not in _SUPPORTED_FLOAT:
        msg = f"{config.mode.value} is not supported."
        raise InternalError(msg)
    ma = _multi_axis(weight, config, reduction_axes)
    if ma is not None:
        cw, dqv = _float(ma.flat, config, 1, ma.flat_params(precomputed_scale), dq)
        out = CompressedWeight(ma.restore(cw.tensor), ma.params(cw.scale))
        out.packed = ma.restore(cw.packed)
        if getattr(cw, "scale_e8m0", None) is not None:
            out.scale_e8m0 = ma.params(cw.scale_e8m0)
        return out, ma.restore(dqv)
    w, axis, gs = _grouped(weight, config, reduction_axes, precomputed_scale)
    o = quantize_launch(w, config, axis, gs, precomputed_scale, None, want_codes="byte", want_values=True, want_dq=dq)
    pshape = _keepdims_shape(w.shape, axis)
    scale = precomputed_scale if precomputed_scale is not None else o["scale"].reshape(pshape)
    cw = CompressedWeight(o["values"].reshape(w.shape), scale)
    cw.packed = o["codes"].reshape(w.shape)  # one format byte per element
    if "scale_e8m0" in o:
        cw.scale_e8m0 = o["scale_e8m0"].reshape(pshape)
    return cw, (o["dq"].reshape(w.shape) if dq else None)


def do_float_quantization(weight: torch.Tensor, config: WeightCompressionConfig,
                          reduction_axes: Optional[ReductionAxes] = None,
                          precomputed_scale: Optional[torch.Tensor] = None) -> CompressedWeight:
    """WC/weight_lowering.py:151-249.  ``tensor`` holds decoded fp32 grid values like the
    reference's torch/numpy path; ``packed`` additionally holds the format's bit patterns."""
    if config.mode == CompressWeightsMode.NVFP4:
        msg = "nvfp4 is not supported."
        raise InternalError(msg)
    cw, _ = _float(weight, config, reduction_axes, precomputed_scale, dq=False)
    return cw


def do_float_dequantization(compressed_weight: CompressedWeight, reduction_axis: int = -1) -> torch.Tensor:
    """WC/weight_lowering.py:131-148."""
    scale = compressed_weight.scale
    if compressed_weight.global_scale is not None:
        scale = scale * compressed_weight.global_scale
    d = compressed_weight.get_unscaled_tensor() * scale
    if reduction_axis != -1:
        d = ungroup_weights(d, reduction_axis)
    return d


def float_quantize_dequantize_weight(weight: torch.Tensor, config: WeightCompressionConfig,
                                     reduction_axes: Optional[ReductionAxes] = None,
                                     precomputed_scale: Optional[torch.Tensor] = None,
                                     return_compressed_weight: Optional[bool] = False):
    """WC/weight_lowering.py:252-289."""
    cw, dq = _float(weight, config, reduction_axes, precomputed_scale, dq=True)
    if return_compressed_weight:
        return dq, cw
    return dq


# ------------------------------------------------------------------------------------------------
# entry point of the per-weight loop
# ------------------------------------------------------------------------------------------------
def compress_weight(weight: torch.Tensor, reduction_axes: ReductionAxes, config: WeightCompressionConfig,
                    precomputed_compressed_weight: Optional[CompressedWeight] = None, *,
                    pack: bool = False) -> CompressedWeight:
    """WC/weight_lowering.py:377-407.

    ``pack=False`` returns what the reference returns (unpacked codes / decoded values).
    ``pack=True`` is the storage path used when a model is transformed: codes leave the kernel
    already nibble-packed (INT4 with the +8 offset, flat order, even index in the low nibble),
    which replaces the reference's separate range check, offset and ``pack_uint4/pack_int4``
    passes (src/nncf/torch/quantization/layers.py:1400-1404,1444-1451)."""
    ps = pz = None
    if precomputed_compressed_weight is not None:
        ps, pz = precomputed_compressed_weight.scale, precomputed_compressed_weight.zero_point
    if not pack:
        if not config.is_integer:
            return do_float_quantization(weight, config, reduction_axes, ps)
        return do_integer_quantization(weight, config, reduction_axes, ps, pz)
    if config.is_integer and config.is_asym_mode and (ps is None) != (pz is None):
        msg = ("If precomputed quantization parameters are provided, both scale and zero point are required "
               "for asymmetric quantization.")
        raise ValueError(msg)
    ma = _multi_axis(weight, config, reduction_axes)
    if ma is not None:
        # convolution weights: per-channel storage; trailing reduced axes make this a reshape, not a copy
        pre = None if ps is None else CompressedWeight(None, ma.flat_params(ps), ma.flat_params(pz))
        cw = compress_weight(ma.flat, 1, config, pre, pack=True)
        if config.num_bits != 4:
            cw.packed = ma.restore(cw.packed)
        elif ma.perm != list(range(len(ma.perm))):
            msg = "nibble-packed storage of a weight whose reduced axes are not trailing is not supported"
            raise UnsupportedModelError(msg)
        cw.scale, cw.zero_point, cw.scale_f16 = ma.params(cw.scale), ma.params(cw.zero_point), ma.params(cw.scale_f16)
        if getattr(cw, "scale_e8m0", None) is not None:
            cw.scale_e8m0 = ma.params(cw.scale_e8m0)
        cw.grouped_shape = ma.shape
        return cw
    w, axis, gs = _grouped(weight, config, reduction_axes, ps)
    four_bit = config.num_bits == 4
    o = quantize_launch(w, config, axis, gs, ps, pz, want_codes="nibble" if four_bit else "byte",
                        want_scale_f16=True, want_zp_packed=True)
    pshape = _keepdims_shape(w.shape, axis)
    scale = ps if ps is not None else o["scale"].reshape(pshape)
    zp = None
    if config.is_integer and config.is_asym_mode:
        zp = pz if pz is not None else o["zp"].reshape(pshape)
    cw = CompressedWeight(None, scale, zp)
    cw.packed = o["packed"].reshape(-1, 1) if four_bit else o["codes"].reshape(w.shape)
    cw.scale_f16 = o["scale_f16"].reshape(pshape)
    if "zp_packed" in o:
        n_groups = o["scale_f16"].numel()
        cw.zero_point_packed = (o["zp_packed"][: (n_groups + 1) // 2].reshape(-1, 1) if four_bit
                                else o["zp_packed"].reshape(pshape))
    cw.grouped_shape = tuple(w.shape)
    if "scale_e8m0" in o:
        cw.scale_e8m0 = o["scale_e8m0"].reshape(pshape)
    return cw
