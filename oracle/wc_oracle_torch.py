"""Multi-threaded CPU baseline for the data-free integer path (TEST / BENCH INFRASTRUCTURE ONLY).

The reference's torch backend executes weight compression as a chain of whole-tensor torch
operations on the host cores.  This module restates that chain for the integer modes with the
same operations in the same order, so that the benchmark's ``cpu_baseline`` / ``--impl reference``
arm times what the reference would do on the same machine with all host threads.  It is
checked against the numpy oracle (``wc_oracle``) in the CPU test-suite, which in turn is pinned
to golden outputs of the reference itself.  Parity status: pinned (through ``wc_oracle``).
"""

from __future__ import annotations

import torch

EPS32 = torch.finfo(torch.float32).eps


def compress_weight_int(weight: torch.Tensor, mode: str, group_size: int):
    """[out, in] weight, reduction over the last axis.
    WC/weight_lowering.py:451-508 -> :292-326 (parameters; :629-649 signed scale or
    src/nncf/quantization/fake_quantize.py:322-350) -> :652-684 (codes), where WC is
    src/nncf/quantization/algorithms/weight_compression.  Returns (codes, scale, zero_point)."""
    bits = 8 if mode.startswith("int8") else 4
    asym = mode.endswith("asym")
    w = weight
    if group_size != -1:
        w = w.reshape(w.shape[0], w.shape[1] // group_size, group_size)
    if w.dtype != torch.float32:
        w = w.to(torch.float32)
    axis = w.ndim - 1
    zp = None
    if asym:
        lo = torch.amin(w, dim=axis, keepdim=True)
        hi = torch.amax(w, dim=axis, keepdim=True)
        levels = 2 ** bits
        scale = ((hi - lo) / (levels - 1)).to(torch.float32)
        scale = torch.where(torch.abs(scale) < EPS32, EPS32, scale)
        zp = 0 - torch.round(lo / scale)
        zp = torch.clip(zp.to(torch.int32), 0, levels - 1)
    else:
        factor = 2 ** (bits - 1)
        w_abs_min = torch.abs(torch.amin(w, dim=axis, keepdim=True))
        w_max = torch.amax(w, dim=axis, keepdim=True)
        scale = torch.where(w_abs_min >= w_max, w_abs_min, -w_max)
        scale /= factor
        scale = torch.where(torch.abs(scale) < EPS32, EPS32, scale)
    q = w / scale
    if zp is not None:
        q += zp.to(torch.float32)
    q = torch.round(q)
    lo_l, hi_l = (0, 2 ** bits - 1) if asym else (-(2 ** (bits - 1)), 2 ** (bits - 1) - 1)
    codes = torch.clip(q, lo_l, hi_l).to(torch.uint8 if asym else torch.int8)
    return codes, scale, zp


def pack_weight(codes: torch.Tensor, mode: str) -> torch.Tensor:
    """The decompressor's pack step: range check, +8 for signed int4, nibble pack
    (src/nncf/torch/quantization/layers.py:1325-1332,1400-1404,1444-1451 and
    src/nncf/torch/quantization/quantize_functions.py:417-461)."""
    bits = 8 if mode.startswith("int8") else 4
    asym = mode.endswith("asym")
    lo, hi = (0, 2 ** bits - 1) if asym else (-(2 ** (bits - 1)), 2 ** (bits - 1) - 1)
    if torch.any((codes < lo) | (codes > hi)):
        raise ValueError("codes out of range")
    if bits == 8:
        return codes
    t = codes
    if not asym:
        t = (t + 8).to(torch.uint8)
    t = t.contiguous().reshape(-1, 2)
    return torch.bitwise_and(t[..., ::2], 15) | t[..., 1::2] << 4


def compress_and_pack(weight: torch.Tensor, mode: str, group_size: int):
    """What the reference's per-weight loop body costs: compress, fp16 scale buffer, pack."""
    codes, scale, zp = compress_weight_int(weight, mode, group_size)
    packed = pack_weight(codes, mode)
    scale16 = scale.to(torch.float16)
    zp_packed = None
    if zp is not None:
        zp_packed = pack_weight(zp.to(torch.uint8), "int4_asym" if mode.startswith("int4") else "int8_asym") \
            if (mode.startswith("int8") or zp.numel() % 2 == 0) else zp.to(torch.uint8)
    return packed, scale16, zp_packed
