"""CPU oracle for the weight-compression hot path (TEST INFRASTRUCTURE ONLY).

This module is a numpy restatement of the arithmetic behind ``nncf.compress_weights``
(nncf 3.2.0).  It exists to check the CUDA kernels: only the tests, the smoke check and
the ``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.  The
product package never does; it fails loudly when its CUDA library is missing.

Parity status: PINNED.  ``tests/golden/make_golden.py`` runs the reference itself
(torch CPU backend) on seeded inputs and stores its outputs; ``tests/test_oracle_golden.py``
checks every function here against those fixtures and against the known-answer vectors
transcribed (numbers only) from the reference's own tests.

Every function cites the reference file:line it restates.  Paths are relative to the
reference project root; ``WC`` abbreviates
``src/nncf/quantization/algorithms/weight_compression``.

All arithmetic is IEEE fp32 unless said otherwise: division is a true division,
rounding is round-half-to-even (``np.round``/``np.rint``), additions of the zero point
are separate fp32 adds.  Reductions (mean, sum, matmul) are order-dependent, so values
derived from them are compared with a tolerance, never bit-for-bit.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

F32 = np.float32
EPS32 = np.finfo(np.float32).eps  # 1.1920929e-07, the reference's fns.finfo(x).eps

# ---------------------------------------------------------------------------------------
# Modes (string values equal nncf.parameters.CompressWeightsMode values,
# src/nncf/parameters.py:72-118)
# ---------------------------------------------------------------------------------------
INT8_SYM, INT8_ASYM = "int8_sym", "int8_asym"
INT4_SYM, INT4_ASYM = "int4_sym", "int4_asym"
NF4, MXFP4, FP4 = "nf4", "mxfp4", "fp4"
FP8_E4M3, MXFP8_E4M3 = "fp8_e4m3", "mxfp8_e4m3"

INTEGER_MODES = (INT8_SYM, INT8_ASYM, INT4_SYM, INT4_ASYM)
FLOAT_MODES = (NF4, MXFP4, FP4, FP8_E4M3, MXFP8_E4M3)


def num_bits(mode: str) -> int:
    """WC/config.py:52-72."""
    return 8 if mode in (INT8_SYM, INT8_ASYM, FP8_E4M3, MXFP8_E4M3) else 4


def is_asym(mode: str) -> bool:
    """WC/config.py:74-76."""
    return mode in (INT4_ASYM, INT8_ASYM)


def is_integer(mode: str) -> bool:
    """WC/config.py:78-93."""
    return mode in INTEGER_MODES


# ---------------------------------------------------------------------------------------
# Code books (WC/constants.py:17-36, 39-58, 84-106) -- format definitions, fp32 literals.
# ---------------------------------------------------------------------------------------
NF4_LEVELS = np.array(
    [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
     -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
     0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
     0.7229568362236023, 1.0], dtype=F32)
# Decision boundaries between NF4 levels.  The reference hard-codes these 15 literals
# (aligned with OpenVINO) instead of recomputing midpoints.
NF4_BOUNDS = np.array(
    [-0.84809643, -0.6106329, -0.45999527, -0.33967942, -0.2346074, -0.13791174, -0.045525018,
     0.03979015, 0.120255254, 0.20352125, 0.29201376, 0.38931254, 0.5016634, 0.6427869,
     0.8614784], dtype=F32)
# 15 E2M1 values: a single (negative) zero.
E2M1_LEVELS = np.array([-6.0, -4.0, -3.0, -2.0, -1.5, -1.0, -0.5, -0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0],
                       dtype=F32)
E2M1_BOUNDS = ((E2M1_LEVELS[1:] + E2M1_LEVELS[:-1]) / 2).astype(F32)
FP_MAX = {NF4: 1.0, MXFP4: 6.0, FP4: 6.0, FP8_E4M3: 448.0, MXFP8_E4M3: 448.0}  # WC/constants.py:109-113


def e4m3_decode_table() -> np.ndarray:
    """Magnitudes of the 128 non-negative E4M3 (fn) bit patterns; 0x7F is NaN.

    Equals the table in WC/fp8_conversion.py:19-40, generated from the format definition
    (bias 7, 3 mantissa bits, subnormals at exponent field 0).
    """
    out = np.empty(128, dtype=np.float64)
    for bits in range(128):
        e, m = bits >> 3, bits & 7
        out[bits] = (m / 8.0) * 2.0 ** -6 if e == 0 else (1.0 + m / 8.0) * 2.0 ** (e - 7)
    out[127] = np.nan
    return out.astype(F32)


E4M3_TABLE = e4m3_decode_table()


# ---------------------------------------------------------------------------------------
# Group reshape (WC/weight_lowering.py:40-81, 410-425)
# ---------------------------------------------------------------------------------------
class InvalidGroupSize(ValueError):
    """Stands for nncf.errors.InvalidGroupSizeError."""


def reshape_for_groups(weight: np.ndarray, reduction_axis, group_size: int):
    """[a1, r, a2] -> [a1, r // gs, gs, a2]; returns the new reduction axis.

    WC/weight_lowering.py:57-81.  Raises when r is not divisible by the group size.
    """
    assert group_size != -1
    if isinstance(reduction_axis, (tuple, list)):
        if len(reduction_axis) != 1:
            raise ValueError("group-wise quantization expects a single reduction axis")
        reduction_axis = reduction_axis[0]
    r = weight.shape[reduction_axis]
    if r % group_size != 0:
        raise InvalidGroupSize(f"Channel size {r} should be divisible by size of group {group_size}.")
    reduction_axis = reduction_axis % weight.ndim
    shape = list(weight.shape)
    shape[reduction_axis:reduction_axis + 1] = (r // group_size, group_size)
    return weight.reshape(shape), reduction_axis + 1


# ---------------------------------------------------------------------------------------
# Integer quantisation parameters
# ---------------------------------------------------------------------------------------
def scale_zero_point(lo: np.ndarray, hi: np.ndarray, level_low: int, level_high: int):
    """Asymmetric scale and zero point.  src/nncf/quantization/fake_quantize.py:322-350
    (narrow_range=False).

    scale = (hi - lo) / (levels - 1), |scale| < eps -> eps,
    zp = clip(int32(level_low - round(lo / scale)), level_low, level_high).
    """
    levels = level_high - level_low + 1
    scale = ((hi - lo) / F32(levels - 1)).astype(F32)
    scale = np.where(np.abs(scale) < EPS32, F32(EPS32), scale).astype(F32)
    zp = F32(level_low) - np.round(lo / scale)
    zp = np.clip(zp.astype(np.int32), level_low, level_high)
    return scale, zp


def signed_scale(weight: np.ndarray, axis, bits: int = 4) -> np.ndarray:
    """Symmetric signed scale.  WC/weight_lowering.py:629-649.

    scale = where(|min| >= max, |min|, -max) / 2^(bits-1); negative when the positive
    extreme dominates, so that extreme maps to the lowest code.
    """
    factor = F32(2 ** (bits - 1))
    abs_min = np.abs(np.min(weight, axis=axis, keepdims=True))
    w_max = np.max(weight, axis=axis, keepdims=True)
    scale = np.where(abs_min >= w_max, abs_min, -w_max).astype(F32)
    scale = scale / factor
    return np.where(np.abs(scale) < EPS32, F32(EPS32), scale).astype(F32)


def integer_params(weight: np.ndarray, axis, mode: str):
    """WC/weight_lowering.py:292-326.  Returns (scale fp32, zero_point int32 | None)."""
    assert is_integer(mode)
    w = weight.astype(F32)
    bits = num_bits(mode)
    if is_asym(mode):
        lo = np.min(w, axis=axis, keepdims=True)
        hi = np.max(w, axis=axis, keepdims=True)
        return scale_zero_point(lo, hi, 0, 2 ** bits - 1)
    return signed_scale(w, axis, bits), None


def integer_codes(weight: np.ndarray, mode: str, scale: np.ndarray, zero_point=None) -> np.ndarray:
    """q = clip(round(w / scale [+ float(zp)])).  WC/weight_lowering.py:652-684."""
    w = weight.astype(F32)
    s = scale.astype(F32)
    bits = num_bits(mode)
    asym = is_asym(mode)
    lo = 0 if asym else -(2 ** (bits - 1))
    hi = 2 ** bits - 1 if asym else 2 ** (bits - 1) - 1
    q = (w / s).astype(F32)
    if zero_point is not None:
        q = (q + zero_point.astype(F32)).astype(F32)
    q = np.round(q)
    return np.clip(q, lo, hi).astype(np.uint8 if asym else np.int8)


@dataclass
class Compressed:
    """Stands for WC/parameters.py:19-49 CompressedWeight (tensor, scale, zero_point)."""

    tensor: Optional[np.ndarray] = None
    scale: Optional[np.ndarray] = None
    zero_point: Optional[np.ndarray] = None


def do_integer_quantization(weight, mode, group_size=-1, reduction_axis=None, scale=None, zero_point=None):
    """WC/weight_lowering.py:451-508."""
    assert is_integer(mode)
    if is_asym(mode) and (scale is None) != (zero_point is None):
        raise ValueError("both scale and zero point are required for asymmetric quantization")
    if group_size != -1 and reduction_axis is not None:
        weight, reduction_axis = reshape_for_groups(weight, reduction_axis, group_size)
    w = weight.astype(F32)
    s, z = scale, zero_point
    if s is None or (is_asym(mode) and z is None):
        if reduction_axis is None:
            raise ValueError("Reduction axes are required for computing the scale and (zero point) vectors.")
        s, z = integer_params(w, reduction_axis, mode)
    return Compressed(integer_codes(w, mode, s, z), s, z)


def do_integer_dequantization(cw: Compressed) -> np.ndarray:
    """(int32(q) - zp) as scale dtype, times scale.  WC/weight_lowering.py:428-448."""
    t = cw.tensor
    d = t.astype(np.int32) - cw.zero_point if cw.zero_point is not None else t
    return (d.astype(cw.scale.dtype) * cw.scale).astype(cw.scale.dtype)


def integer_quantize_dequantize(weight, mode, group_size=-1, reduction_axis=None, scale=None, zero_point=None):
    """WC/weight_lowering.py:511-554 (reference branch).  Returns (dq, Compressed)."""
    cw = do_integer_quantization(weight, mode, group_size, reduction_axis, scale, zero_point)
    return do_integer_dequantization(cw), cw


def integer_quantization_error(weight, reduction_axis, mode, group_size=-1, reduction="max_mean") -> float:
    """WC/weight_lowering.py:329-374."""
    if reduction not in ("max_mean", "frobenius"):
        raise ValueError(f"Unsupported aggregation mode: {reduction}.")
    w = weight.astype(F32)
    dq, _ = integer_quantize_dequantize(w, mode, group_size, reduction_axis)
    dq = dq.reshape(w.shape)
    if reduction == "max_mean":
        return float(np.max(np.mean((dq - w) ** 2, axis=reduction_axis)))
    return float(np.linalg.norm((dq - w).ravel()))


# ---------------------------------------------------------------------------------------
# Float (code-book) quantisation
# ---------------------------------------------------------------------------------------
def float_params(weight: np.ndarray, axis, mode: str) -> np.ndarray:
    """Scale for NF4 / FP4 / MXFP4 / FP8 / MXFP8.  WC/weight_lowering.py:84-128.

    scale = max|w| (/ format max unless NF4), eps guard, and for MX modes
    2^clip(ceil(log2(scale)), -127, 127) with log2 evaluated in fp32.
    """
    w = weight.astype(F32)
    scale = np.max(np.abs(w), axis=axis, keepdims=True)
    if mode != NF4:
        scale = (scale / F32(FP_MAX[mode])).astype(F32)
    scale = np.where(np.abs(scale) < EPS32, F32(EPS32), scale).astype(F32)
    if mode in (MXFP4, MXFP8_E4M3):
        e = np.clip(np.ceil(np.log2(scale)), -127, 127).astype(F32)
        scale = (F32(2) ** e).astype(F32)
    return scale


def f16_bits_to_e4m3_bits(h: np.ndarray) -> np.ndarray:
    """fp16 bit pattern -> E4M3 bit pattern, round-to-nearest-even, no infinities:
    fp16 NaN/Inf and anything that rounds past 448 become NaN (0x7F), fp16 subnormals and
    magnitudes below half the smallest E4M3 subnormal become signed zero.
    Restates the conversion of WC/fp8_conversion.py:43-208 as a plain rounding rule.
    """
    h = h.astype(np.uint16)
    sign = ((h >> 8) & 0x80).astype(np.uint8)
    e16 = ((h >> 10) & 0x1F).astype(np.int32)
    m16 = (h & 0x3FF).astype(np.int32)
    out = np.zeros(h.shape, dtype=np.int32)
    naninf = e16 == 31
    normal = (e16 != 0) & ~naninf
    e8 = e16 - 8  # rebias 15 -> 7
    # significand with hidden one, 11 bits: value = sig * 2^(e8 - 7 - 10)
    sig = m16 | 0x400
    # number of low bits to drop: 7 for a normal result, more for a subnormal one
    drop = np.where(e8 >= 1, 7, 7 + (1 - e8))
    drop = np.minimum(drop, 31)
    kept = sig >> drop
    rem = sig & ((1 << drop) - 1)
    half = 1 << (drop - 1)
    up = (rem > half) | ((rem == half) & ((kept & 1) == 1))
    kept = kept + up.astype(np.int32)
    # normal result: kept in [8, 16]; 16 means mantissa overflow -> exponent + 1
    e_res = np.where(e8 >= 1, e8, 0)
    bits_norm = np.where(kept >= 16, ((e_res + 1) << 3), (e_res << 3) | (kept & 7))
    # subnormal result: kept in [0, 8]; 8 lands on the smallest normal (exp field 1, mant 0) = bits 8
    bits_sub = kept
    bits = np.where(e8 >= 1, bits_norm, bits_sub)
    bits = np.where(bits >= 0x7F, 0x7F, bits)
    out = np.where(normal, bits, out)
    out = np.where(naninf, 0x7F, out)
    return (out.astype(np.uint8) | sign).astype(np.uint8)


def fp32_to_e4m3_values(x: np.ndarray) -> np.ndarray:
    """fp32 -> fp16 (RNE) -> E4M3 (RNE) -> decoded fp32.  WC/fp8_conversion.py:211-228."""
    with np.errstate(over="ignore"):
        h = x.astype(F32).astype(np.float16).view(np.uint16)
    b = f16_bits_to_e4m3_bits(h)
    mag = E4M3_TABLE[(b & 0x7F).astype(np.int32)]
    return np.where((b & 0x80) != 0, -mag, mag).astype(F32)


def float_codebook_indexes(norm: np.ndarray, mode: str) -> np.ndarray:
    """Index into the 16-entry NF4 table or the 15-entry E2M1 table.

    WC/weight_lowering.py:570-585: searchsorted(bounds, x, side='left') - a value equal to
    a boundary goes to the lower level - and for E2M1 the nearest of (idx, idx+1) with
    ties resolved towards the odd index of the 15-entry table (= IEEE ties-to-even in E2M1).
    """
    if mode == NF4:
        return np.searchsorted(NF4_BOUNDS, norm, side="left")
    idx = np.searchsorted(E2M1_BOUNDS, norm, side="left")
    nxt = np.clip(idx + 1, 0, E2M1_LEVELS.size - 1)
    dl = np.abs(norm - E2M1_LEVELS[idx])
    dr = np.abs(norm - E2M1_LEVELS[nxt])
    right = (dr < dl) | ((dl == dr) & ((nxt + 1) % 2 == 0))
    return np.where(right, nxt, idx)


def float_quantized_values(norm: np.ndarray, mode: str) -> np.ndarray:
    """Normalised weight -> fp32 value on the format's grid.  WC/weight_lowering.py:557-586."""
    if mode in (FP8_E4M3, MXFP8_E4M3):
        return fp32_to_e4m3_values(norm)
    levels = NF4_LEVELS if mode == NF4 else E2M1_LEVELS
    return levels[float_codebook_indexes(norm, mode)]


def do_float_quantization(weight, mode, group_size=-1, reduction_axis=None, scale=None) -> Compressed:
    """WC/weight_lowering.py:195-249 (torch/numpy branch: tensor = decoded fp32 grid values)."""
    assert mode in FLOAT_MODES
    if group_size != -1 and reduction_axis is not None:
        weight, reduction_axis = reshape_for_groups(weight, reduction_axis, group_size)
    w = weight.astype(F32)
    s = scale if scale is not None else float_params(w, reduction_axis, mode)
    norm = (w / s.astype(F32)).astype(F32)  # WC/weight_lowering.py:613-626
    return Compressed(float_quantized_values(norm, mode), s)


def float_quantize_dequantize(weight, mode, group_size=-1, reduction_axis=None, scale=None):
    """WC/weight_lowering.py:252-289 + 131-148.  Returns (dq, Compressed)."""
    cw = do_float_quantization(weight, mode, group_size, reduction_axis, scale)
    return (cw.tensor * cw.scale).astype(F32), cw


def nibble_code_nf4(values: np.ndarray) -> np.ndarray:
    """Table index 0..15 of an NF4 grid value (storage choice of this build)."""
    return np.searchsorted(NF4_LEVELS, values, side="left").astype(np.uint8)


def nibble_code_e2m1(values: np.ndarray) -> np.ndarray:
    """E2M1 bit pattern s|e1 e0|m of a grid value: sign*8 + index of |v| in
    {0, .5, 1, 1.5, 2, 3, 4, 6}.  Zero is stored as +0 (code 0)."""
    mags = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=F32)
    idx = np.searchsorted(mags, np.abs(values), side="left").astype(np.uint8)
    neg = (values < 0).astype(np.uint8)
    return (neg * 8 + idx).astype(np.uint8)


def e8m0_code(scale: np.ndarray) -> np.ndarray:
    """Biased exponent byte of a power-of-two scale (E8M0: value = 2^(code - 127))."""
    return (np.log2(scale.astype(np.float64)).round().astype(np.int32) + 127).astype(np.uint8)


# ---------------------------------------------------------------------------------------
# Entry point (WC/weight_lowering.py:377-407)
# ---------------------------------------------------------------------------------------
def compress_weight(weight, reduction_axis, mode, group_size=-1, scale=None, zero_point=None) -> Compressed:
    if is_integer(mode):
        return do_integer_quantization(weight, mode, group_size, reduction_axis, scale, zero_point)
    return do_float_quantization(weight, mode, group_size, reduction_axis, scale)


def stored_form(weight: np.ndarray, mode: str, group_size: int = -1, rows_per_chunk: int = 8192) -> dict:
    """What the reference's per-weight loop leaves behind for an [out, in] weight (reduction over the
    last axis): ``compress_weight`` (WC/weight_lowering.py:377-407) followed by the decompressor's
    ``pack_weight`` (src/nncf/torch/quantization/layers.py:1325-1332, 1358-1362, 1400-1404, 1444-1451).
    Returns flat arrays: ``packed`` (4-bit modes: two codes per byte, INT4_SYM offset by 8; 8-bit modes:
    one byte per code), ``scale`` fp32 [groups], ``zero_point`` int32 [groups] (asymmetric modes) and
    ``scale_e8m0`` (MX modes).  NF4 / E2M1 nibbles are this build's storage choice (the reference's torch
    path has none).  Rows are independent, so the weight is processed in chunks of rows to bound memory."""
    weight = np.asarray(weight)
    assert weight.ndim == 2
    out: dict = {"packed": [], "scale": [], "zero_point": [], "scale_e8m0": []}
    for r0 in range(0, weight.shape[0], rows_per_chunk):
        w = np.ascontiguousarray(weight[r0:r0 + rows_per_chunk]).astype(F32)
        cw = compress_weight(w, 1, mode, group_size)
        if is_integer(mode):
            if num_bits(mode) == 4:
                codes = pack_int4(cw.tensor) if mode == INT4_SYM else pack_uint4(cw.tensor)
            else:
                codes = cw.tensor
        elif mode in (FP8_E4M3, MXFP8_E4M3):
            # E4M3 bytes: the quotient rounded to fp16, then to E4M3 (WC/fp8_conversion.py:211-228)
            grouped = w if group_size == -1 else reshape_for_groups(w, 1, group_size)[0]
            with np.errstate(over="ignore"):
                h = (grouped / cw.scale).astype(F32).astype(np.float16).view(np.uint16)
            codes = f16_bits_to_e4m3_bits(h)
        else:
            codes = pack_uint4(nibble_code_nf4(cw.tensor) if mode == NF4 else nibble_code_e2m1(cw.tensor))
        out["packed"].append(np.ascontiguousarray(codes).reshape(-1))
        out["scale"].append(cw.scale.reshape(-1))
        if cw.zero_point is not None:
            out["zero_point"].append(cw.zero_point.reshape(-1).astype(np.int32))
        if mode in (MXFP4, MXFP8_E4M3):
            out["scale_e8m0"].append(e8m0_code(cw.scale).reshape(-1))
    return {k: np.concatenate(v) for k, v in out.items() if v}


# ---------------------------------------------------------------------------------------
# Nibble packing and run-time decompression
# (src/nncf/torch/quantization/quantize_functions.py:389-473)
# ---------------------------------------------------------------------------------------
def pack_uint4(codes: np.ndarray) -> np.ndarray:
    """Flat order; even index -> low nibble, odd -> high nibble; result shape [N/2, 1]."""
    assert codes.dtype == np.uint8
    p = np.ascontiguousarray(codes).reshape(-1, 2)
    return ((p[:, 0:1] & 15) | (p[:, 1:2] << 4)).astype(np.uint8)


def pack_int4(codes: np.ndarray) -> np.ndarray:
    assert codes.dtype == np.int8
    return pack_uint4((codes + 8).astype(np.uint8))


def unpack_uint4(packed: np.ndarray) -> np.ndarray:
    return np.stack((packed & 15, packed >> 4), axis=-1)


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    return unpack_uint4(packed).astype(np.int8) - 8


def decompress_asymmetric(codes, scale_f16, zero_point):
    """(x.f16 - zp.f16) * scale.f16, all in fp16.  quantize_functions.py:389-401."""
    return ((codes.astype(np.float16) - zero_point.astype(np.float16)) * scale_f16).astype(np.float16)


def decompress_symmetric(codes, scale_f16):
    """x.f16 * scale.f16.  quantize_functions.py:404-414."""
    return (codes.astype(np.float16) * scale_f16).astype(np.float16)


# ---------------------------------------------------------------------------------------
# Statistic reducers (src/nncf/common/tensor_statistics/collectors.py:468-540, 924-936)
# ---------------------------------------------------------------------------------------
def mean_reducer(x: np.ndarray, channel_axis: int = -1) -> np.ndarray:
    """Mean over every axis but the channel axis, fp32 accumulate, result in x.dtype
    (collectors.py:512-516 with the axes of WC/torch_backend.py:147-153)."""
    axes = tuple(a for a in range(x.ndim) if a != channel_axis % x.ndim)
    return np.mean(x.astype(np.float64), axis=axes).astype(x.dtype)


def variance_reducers(x: np.ndarray, axes) -> tuple[float, float]:
    """(mean of variance, max of variance); collectors.py:519-532.  fns.var is the
    population variance (ddof=0) on the numpy backend and unbiased on torch
    (src/nncf/tensor/functions/torch_numeric.py: var with correction=ddof, default 0)."""
    v = np.var(x.astype(np.float64), axis=axes)
    return float(np.mean(v)), float(np.max(v))


def mean_abs_max_reducer(x: np.ndarray, axes) -> float:
    """collectors.py:535-540."""
    return float(np.mean(np.max(np.abs(x.astype(np.float64)), axis=axes)))


def hawq_trace_step(acc: float, x: np.ndarray) -> float:
    """collectors.py:929-933: container = (container + sum(x*x)) / x.size."""
    return (acc + float(np.sum(x.astype(np.float64) ** 2))) / x.size


# ---------------------------------------------------------------------------------------
# process_stats (WC/activation_stats.py:20-57)
# ---------------------------------------------------------------------------------------
def process_stats(mean_values: Sequence[np.ndarray], shape_values: Sequence[tuple], subset_size: int,
                  act_ch_axis: int = -1):
    """Returns (s [..., hidden], X [..., hidden, n_kept])."""
    X = np.stack(mean_values)
    X_full = np.moveaxis(X, 0, -1)
    n = X_full.shape[-1]
    if n > subset_size and subset_size > 0:
        lens = []
        for shp in shape_values:
            shp = tuple(shp)
            rest = shp[:act_ch_axis] + shp[act_ch_axis % len(shp) + 1:]
            lens.append(int(np.prod(rest, dtype=np.int64)) if rest else 1)
        step = n // subset_size
        order = [i for i, _ in sorted(enumerate(lens), key=lambda p: -p[1])][::step]
        Xs = X_full[..., order]
    else:
        Xs = X_full
    s = np.max(np.abs(X_full), axis=-1)
    return s, Xs


# ---------------------------------------------------------------------------------------
# ScaleEstimation (WC/scale_estimation.py:160-409)
# ---------------------------------------------------------------------------------------
def _qdq(weight_g, mode, scale, zp):
    """Quantise-dequantise an already grouped weight with given parameters."""
    if is_integer(mode):
        dq, cw = integer_quantize_dequantize(weight_g, mode, scale=scale, zero_point=zp)
    else:
        dq, cw = float_quantize_dequantize(weight_g, mode, scale=scale)
    return dq, cw.tensor


def _target_zero_mask(codes, zp):
    """WC/scale_estimation.py:380-393."""
    t = codes
    if zp is not None:
        t = codes.astype(zp.dtype) - zp
    return t, np.isclose(t, 0)


def _estimate_scales(weight, target, zero_mask, importance):
    """sum_gs |w| / (|target| + zero_mask) * importance.  WC/scale_estimation.py:396-409."""
    ideal = np.abs(weight) / (np.abs(target).astype(F32) + zero_mask)
    return np.sum((ideal * importance).astype(F32), axis=-1, keepdims=True, dtype=F32)


def scale_estimation(s: np.ndarray, X: np.ndarray, weight: np.ndarray, reduction_axis: int, mode: str,
                     group_size: int, initial_steps: int = 5, scale_steps: int = 10,
                     weight_penalty: float = -1.0):
    """ScaleEstimation.calculate_quantization_params (WC/scale_estimation.py:160-377)
    after ``process_stats``: ``s`` [hidden], ``X`` [hidden, n].  2-D weights only.

    Returns (scale, zp|None) in the shapes the reference returns.
    """
    X = X.astype(F32)
    weight = weight.astype(F32)
    transposed = False
    if reduction_axis == 0:
        weight = np.moveaxis(weight, -1, -2)
        reduction_axis = weight.ndim - 1
        transposed = True
    gs = group_size if group_size != -1 else weight.shape[reduction_axis]

    if is_integer(mode):
        q_w, cw = integer_quantize_dequantize(weight, mode, gs, reduction_axis)
        zp = cw.zero_point.astype(cw.scale.dtype) if cw.zero_point is not None else None
    else:
        q_w, cw = float_quantize_dequantize(weight, mode, gs, reduction_axis)
        zp = None
    scale = cw.scale
    codes = cw.tensor

    s_g, _ = reshape_for_groups(s[None, :].astype(F32), reduction_axis, gs)   # [1, G, gs]
    w_g, _ = reshape_for_groups(weight, reduction_axis, gs)                  # [out, G, gs]
    importance = (np.ones_like(w_g) * s_g).astype(F32)
    target, zero_mask = _target_zero_mask(codes, zp)
    importance = np.where(zero_mask, F32(0), importance).astype(F32)
    denom = np.sum(importance, axis=-1, keepdims=True, dtype=F32)
    importance = (importance / (denom + F32(EPS32))).astype(F32)

    X_g, _ = reshape_for_groups(X, -2 % X.ndim, gs)                            # [G, gs, n]
    fp_outs = np.matmul(np.moveaxis(w_g, -2, -3), X_g)                         # [G, out, n]
    q_outs = np.matmul(np.moveaxis(q_w, -2, -3), X_g)
    diffs = np.moveaxis(np.mean((fp_outs - q_outs) ** 2, axis=-1), -1, -2)     # [out, G]
    if weight_penalty > 0.0:
        diffs = diffs + weight_penalty * np.mean((q_w - w_g) ** 2, axis=-1)
    best = diffs
    result = scale
    sign = scale / np.abs(scale)
    zero_scale = F32(0.001)
    zmask = zero_scale * zero_mask.astype(F32)

    def score(cand):
        dq, _ = _qdq(w_g, mode, cand, zp)
        qo = np.matmul(np.moveaxis(dq, -2, -3), X_g)
        d = np.moveaxis(np.mean((fp_outs - qo) ** 2, axis=-1), -1, -2)
        if weight_penalty > 0.0:
            d = d + weight_penalty * np.mean((dq - w_g) ** 2, axis=-1)
        return d

    for i in range(initial_steps):
        cand = (_estimate_scales(w_g, target, zmask, importance) * sign).astype(F32)
        d = score(cand)
        keep = (d > best).astype(F32)
        best = keep * best + (F32(1) - keep) * d
        k3 = keep[..., None]
        result = (k3 * result + (F32(1) - k3) * cand).astype(F32)
        if i < initial_steps - 1:
            _, codes = _qdq(w_g, mode, result, zp)
            target, zm = _target_zero_mask(codes, zp)
            zmask = zero_scale * zm.astype(F32)

    for step in range(scale_steps):
        factor = 1.0 - 0.05 * step
        scaled = (F32(factor) * scale).astype(F32)
        _, codes = _qdq(w_g, mode, scaled, zp)
        target, zm = _target_zero_mask(codes, zp)
        zmask = zero_scale * zm.astype(F32)
        cand = (_estimate_scales(w_g, target, zmask, importance) * sign).astype(F32)
        d = score(cand)
        keep = (d > best).astype(F32)
        best = keep * best + (F32(1) - keep) * d
        k3 = keep[..., None]
        result = (k3 * result + (F32(1) - k3) * cand).astype(F32)

    if group_size == -1:
        result = np.squeeze(result, axis=-2)
        if zp is not None:
            zp = np.squeeze(zp, axis=-2)
    if transposed:
        if group_size == -1:
            result = np.moveaxis(result, -1, -2)
            zp = np.moveaxis(zp, -1, -2) if zp is not None else None
        else:
            result = np.moveaxis(result, (-1, -2, -3), (-2, -3, -1))
            zp = np.moveaxis(zp, (-1, -2, -3), (-2, -3, -1)) if zp is not None else None
    return result, zp


# ---------------------------------------------------------------------------------------
# AWQ (WC/awq.py:243-366)
# ---------------------------------------------------------------------------------------
FP16_MAX = 65504.0
FP16_OVERFLOW_MARGIN = 0.25  # WC/awq.py module constants


def awq_data_free_scale(weight: np.ndarray, axis: int) -> np.ndarray:
    """1 / max(mean|W| over `axis`, eps).  WC/awq.py:363-366."""
    m = np.maximum(np.mean(np.abs(weight.astype(F32)), axis=axis, dtype=F32), F32(EPS32))
    return (F32(1) / m).astype(F32)


def awq_data_aware_scale(s: np.ndarray, X: np.ndarray, weight: np.ndarray, reduction_axis: int, mode: str,
                         group_size: int, percent_to_apply: float = 0.002, alpha_min: float = 0.0,
                         alpha_max: float = 1.0, steps: int = 100, prev_weight=None, prev_s_max=None):
    """AWQ._data_aware_step for a 2-D weight (WC/awq.py:243-357) after process_stats.

    ``s`` [hidden], ``X`` [hidden, n]; returns the per-input-channel scale [hidden].
    ``prev_weight``/``prev_s_max``: merge-node weight and max of its activation magnitude
    for the fp16-overflow clamp (:315-335).
    """
    s = s.astype(F32)
    X = X.astype(F32)
    weight = weight.astype(F32)
    alpha_step = (alpha_max - alpha_min) / steps
    hidden = s.shape[-1]
    prev_w = None
    prev_rdim = None
    if prev_weight is not None and prev_s_max is not None:
        prev_w = np.mean(np.abs(prev_weight.astype(F32)), axis=reduction_axis, dtype=F32)
        prev_rdim = prev_weight.shape[reduction_axis]
    top_k = max(int(hidden * percent_to_apply), 1)
    order = np.argsort(-s, kind="stable")[:top_k]
    gs = group_size if group_size != -1 else hidden
    groups = sorted({int(i) // gs for i in order})
    if reduction_axis == 0:
        weight = np.moveaxis(weight, -1, -2)
    scale = np.ones(hidden, dtype=F32)
    for gi in groups:
        off = gi * gs
        gscale = s[off:off + gs]
        gweight = weight[:, off:off + gs]
        gacts = X[off:off + gs, :]
        a_min = F32(np.quantile(gscale, 0.1))
        gscale = np.clip(gscale, a_min, F32(1e2)).astype(F32)
        fp_out = np.matmul(gweight, gacts)
        min_diff = np.max(np.abs(fp_out))
        best = None
        alpha = alpha_min
        for _ in range(steps):
            cur = (gscale ** F32(alpha)).astype(F32)
            if prev_w is not None:
                threshold = FP16_OVERFLOW_MARGIN * FP16_MAX
                mags = (prev_w[off:off + gs] / cur) * F32(prev_s_max) * prev_rdim
                if mags.max() >= threshold:
                    clamped = prev_w[off:off + gs] * F32(prev_s_max) * prev_rdim / threshold
                    cur = np.where(mags < threshold, cur, clamped).astype(F32)
            wq = (gweight * cur).astype(F32)
            if is_integer(mode):
                dq, _ = integer_quantize_dequantize(wq, mode, -1, -1)
            else:
                dq, _ = float_quantize_dequantize(wq, mode, -1, -1)
            sacts = gacts / cur[:, None]
            cur_out = np.matmul(dq, sacts)
            cur_diff = np.mean(np.abs(cur_out - fp_out))
            if cur_diff < min_diff:
                min_diff = cur_diff
                best = cur
            alpha += alpha_step
        if best is not None:
            scale[off:off + gs] = best
    return scale


# ---------------------------------------------------------------------------------------
# GPTQ (WC/gptq.py:200-379)
# ---------------------------------------------------------------------------------------
def gptq_hessian(inputs: Sequence[np.ndarray]) -> np.ndarray:
    """Running-rescaled H = sum (2/n) X^T X for a 2-D weight.  WC/gptq.py:200-242.

    A [b, T, C] activation counts as b samples; a 2-D [T, C] one as a single sample.
    """
    C = inputs[0].shape[-1]
    H = np.zeros((C, C), dtype=F32)
    n = 0
    for inp in inputs:
        b = inp.shape[0] if inp.ndim == 3 else 1
        x = inp.reshape(-1, C).T
        H *= F32(n / (n + b))
        n += b
        x = x.astype(F32) * F32(math.sqrt(2 / n))
        H += x @ x.T
    return H


def gptq_hinv(H: np.ndarray, weight: np.ndarray, damp_percent: float):
    """Dead columns, damping and the upper Cholesky factor of H^-1.  WC/gptq.py:269-295.
    Mutates H and weight like the reference."""
    dead = np.diag(H) == 0
    H[dead, dead] = 1
    weight[:, dead] = 0
    damp = F32(damp_percent) * np.mean(np.diag(H), dtype=F32)
    idx = np.arange(H.shape[0])
    H[idx, idx] += damp
    # fp32 LAPACK, like the reference's torch.linalg.cholesky / cholesky_inverse / cholesky(upper)
    from scipy.linalg import lapack

    L, info = lapack.spotrf(H.astype(F32), lower=1)
    assert info == 0, "Hessian is not positive definite"
    Hinv, info = lapack.spotri(L, lower=1)
    assert info == 0
    Hinv = np.tril(Hinv) + np.tril(Hinv, -1).T
    U, info = lapack.spotrf(Hinv.astype(F32), lower=0)
    assert info == 0
    U = np.triu(U)
    return U.astype(F32)


def gptq_quantize(weight: np.ndarray, hinv: np.ndarray, mode: str, group_size: int, block_size: int = 128,
                  se_stats=None):
    """Blocked column sweep with error feedback.  WC/gptq.py:297-379.

    ``se_stats`` = (s [C], X [C, n]) after ``process_stats``: GPTQ(scale_estimation=True), i.e. 4-bit integer
    groups take their parameters from ``scale_estimation`` on the group's slice of the statistics and of the
    tensor-level weight (WC/gptq.py:319-327; the reference slices the raw activations, reduces them with
    ``activations_to_wc_statistics`` :382-396 and lets calculate_quantization_params run process_stats with
    its default subset of 32, which commutes with the slicing).

    ``weight`` [out, C] fp32 (mutated), ``hinv`` upper factor [C, C].  Scales are taken at
    each group start from the *tensor-level* weight (updated at block ends only), exactly as
    the reference indexes ``weight_tensor`` (:312-335) rather than the in-block copy.
    Returns (dequantised weight, scales [out, G, 1], zero points or None).
    """
    out_ch, C = weight.shape
    gs = group_size if group_size != -1 else C
    scales, zps = [], []
    Q = np.zeros_like(weight)
    for i1 in range(0, C, block_size):
        i2 = min(i1 + block_size, C)
        Wb = weight[:, i1:i2].copy()
        Eb = np.zeros_like(Wb)
        Hb = hinv[i1:i2, i1:i2]
        for i in range(i2 - i1):
            col = Wb[:, i]
            d = Hb[i, i]
            if (i1 + i) % gs == 0:
                grp = weight[:, i1 + i:i1 + i + gs]
                if is_integer(mode) and se_stats is not None and num_bits(mode) == 4:
                    c0 = i1 + i
                    sc, zp = scale_estimation(se_stats[0][c0:c0 + gs], se_stats[1][c0:c0 + gs], grp, 1, mode, -1)
                    zps.append(zp)
                elif is_integer(mode):
                    sc, zp = integer_params(grp, 1, mode)
                    zps.append(zp)
                else:
                    sc = float_params(grp, 1, mode)
                scales.append(sc)
            if is_integer(mode):
                q, _ = integer_quantize_dequantize(col[:, None], mode, scale=scales[-1], zero_point=zps[-1])
            else:
                q, _ = float_quantize_dequantize(col[:, None], mode, scale=scales[-1])
            q = q.ravel()
            Q[:, i1 + i] = q
            err = ((col - q) / d).astype(F32)
            Wb[:, i:] -= np.outer(err, Hb[i, i:]).astype(F32)
            Eb[:, i] = err
        weight[:, i2:] -= (Eb @ hinv[i1:i2, i2:]).astype(F32)
    S = np.stack(scales, axis=1)
    Z = np.stack(zps, axis=1) if is_asym(mode) else None
    if group_size == -1:
        S = np.squeeze(S, axis=-1)
        Z = np.squeeze(Z, axis=-1) if Z is not None else None
    return Q, S, Z


# ---------------------------------------------------------------------------------------
# LoRA correction (WC/lora_correction.py:139-271)
# ---------------------------------------------------------------------------------------
def lora_correction_adapters(weight: np.ndarray, fq_weight: np.ndarray, mean_values: Sequence[np.ndarray],
                             shape_values: Sequence[tuple], group_size: int, rank: int = 8, num_iterations: int = 3,
                             apply_regularization: bool = True, subset_size: int = 128):
    """The two low-rank adapters of one layer, with the reference's own dense routines: full SVD of the weighted
    residual for the start (:212-216), then alternating least squares with QR-type solvers (:222-269).
    ``weight`` / ``fq_weight`` [O, H] (reduction axis 1); returns (lora_A [R, H], lora_B [O, R]) in fp32."""
    residual = (weight.astype(np.float32) - fq_weight.astype(np.float32)).T.copy()      # [H, O]
    s, X = process_stats(mean_values, shape_values, subset_size)                         # [H], [H, SS]
    s = s.astype(np.float32).copy()
    X = X.astype(np.float32).T                                                           # [SS, H]
    svd_residual = residual
    if group_size > 0:
        # :197-209: activation magnitudes normalised per quantisation group (sum to one, then largest = one)
        for i in range(s.shape[0] // group_size):
            sl = slice(i * group_size, (i + 1) * group_size)
            s[sl] = s[sl] / np.sum(s[sl])
            s[sl] = s[sl] / np.max(s[sl])
        svd_residual = residual * s[:, None]
    U_full, S_full, V_full = np.linalg.svd(svd_residual, full_matrices=False)
    U = U_full[:, :rank]
    V = np.diag(S_full[:rank]) @ V_full[:rank, :]
    noise = X @ residual
    for _ in range(num_iterations):
        XU = X @ U
        if not apply_regularization:
            V = np.linalg.lstsq(XU, noise, rcond=None)[0]
        else:
            V = np.linalg.lstsq(np.concatenate([U, XU], axis=0), np.concatenate([residual, noise], axis=0), rcond=None)[0]
        VI = np.linalg.pinv(V)
        noiseVI = noise @ VI
        if not apply_regularization:
            U = np.linalg.lstsq(X, noiseVI, rcond=None)[0]
        else:
            E = np.eye(U.shape[0], dtype=U.dtype)
            U = np.linalg.lstsq(np.concatenate([E, X], axis=0), np.concatenate([residual @ VI, noiseVI], axis=0),
                                rcond=None)[0]
    return U.T.astype(np.float32), V.T.astype(np.float32)
