"""Weight decompressor modules: the stored form of a compressed weight and its run-time
decompression, mirroring src/nncf/torch/quantization/layers.py:1305-1460
(INT8/INT4 Symmetric/Asymmetric WeightsDecompressor: same constructor arguments, buffers ``_scale``
fp16 and ``_zero_point`` packed, ``pack_weight`` with the reference's range checks and error type).
``forward`` is one ``nncfb_decompress`` launch instead of the reference's unpack / stack / reshape /
cast / subtract / multiply chain.  NF4 and MXFP4 / FP4 decompressors have no counterpart in the
reference's torch backend (it rejects those modes); they follow the same pattern."""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import _lib
from .parameters import CompressWeightsMode


def pack_uint4(tensor: torch.Tensor) -> torch.Tensor:
    """quantize_functions.py:417-433: flat order, even index in the low nibble; result [N/2, 1]."""
    if tensor.dtype != torch.uint8:
        from .errors import ValidationError

        msg = f"Invalid tensor dtype {tensor.type}. torch.uint8 type is supported."
        raise ValidationError(msg)
    t = tensor.contiguous().reshape(-1)
    out = torch.empty(t.numel() // 2, dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        _lib.check(_lib.lib.nncfb_pack_nibbles(_lib.ptr(t), t.numel(), 0, _lib.ptr(out), _lib.stream_handle(t.device)))
    return out.reshape(-1, 1)


def pack_int4(tensor: torch.Tensor) -> torch.Tensor:
    """quantize_functions.py:447-461: +8 then pack."""
    if tensor.dtype != torch.int8:
        from .errors import ValidationError

        msg = f"Invalid tensor dtype {tensor.type}. torch.int8 type is supported."
        raise ValidationError(msg)
    t = tensor.contiguous().reshape(-1)
    out = torch.empty(t.numel() // 2, dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        _lib.check(_lib.lib.nncfb_pack_nibbles(_lib.ptr(t), t.numel(), 8, _lib.ptr(out), _lib.stream_handle(t.device)))
    return out.reshape(-1, 1)


def unpack_uint4(packed: torch.Tensor) -> torch.Tensor:
    """quantize_functions.py:436-444; result [..., 2] uint8."""
    p = packed.contiguous().reshape(-1)
    out = torch.empty(p.numel() * 2, dtype=torch.int8, device=p.device)
    with torch.cuda.device(p.device):
        _lib.check(_lib.lib.nncfb_unpack_nibbles(_lib.ptr(p), p.numel(), 0, _lib.ptr(out), _lib.stream_handle(p.device)))
    return out.view(torch.uint8).reshape(*packed.shape, 2)


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """quantize_functions.py:464-473; result [..., 2] int8."""
    p = packed.contiguous().reshape(-1)
    out = torch.empty(p.numel() * 2, dtype=torch.int8, device=p.device)
    with torch.cuda.device(p.device):
        _lib.check(_lib.lib.nncfb_unpack_nibbles(_lib.ptr(p), p.numel(), 8, _lib.ptr(out), _lib.stream_handle(p.device)))
    return out.reshape(*packed.shape, 2)


class BaseWeightsDecompressor(nn.Module):
    mode: CompressWeightsMode

    def __init__(self, compressed_weight_shape, result_shape, result_dtype):
        super().__init__()
        self.compressed_weight_shape = tuple(compressed_weight_shape) if compressed_weight_shape is not None else None
        self.result_shape = tuple(result_shape) if result_shape is not None else None
        self.result_dtype = result_dtype

    def _decompress(self, x: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor],
                    group_size: int, n: int) -> torch.Tensor:
        out_dtype = self.result_dtype if self.result_dtype is not None else torch.float16
        kdtype = out_dtype if out_dtype in (torch.float32, torch.float16, torch.bfloat16) else torch.float32
        out = torch.empty(n, dtype=kdtype, device=x.device)
        with torch.cuda.device(x.device):
            _lib.check(_lib.lib.nncfb_decompress(
                _lib.ptr(x.contiguous()), _lib.MODE_IDS[self.mode.value], n, group_size, _lib.ptr(scale.contiguous()),
                _lib.ptr(zero_point.contiguous()) if zero_point is not None else None, _lib.ptr(out),
                _lib.DTYPE_IDS[kdtype], _lib.stream_handle(x.device)))
        return out if kdtype == out_dtype else out.to(out_dtype)

    def _group_size(self, scale_shape, full_shape) -> int:
        """Elements sharing a scale, from the scale's keepdims shape over the (grouped) weight shape."""
        gs = 1
        for s, w in zip(scale_shape, full_shape):
            if s == 1 and w != 1:
                gs *= w
        return gs

    def pack_weight(self, weight: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class INT8AsymmetricWeightsDecompressor(BaseWeightsDecompressor):
    """layers.py:1305-1338."""

    mode = CompressWeightsMode.INT8_ASYM

    def __init__(self, scale: torch.Tensor, zero_point: torch.Tensor, result_dtype: Optional[torch.dtype] = None,
                 zero_point_is_stored: bool = False):
        """``zero_point_is_stored``: ``zero_point`` is already the uint8 buffer (written by the compression kernel),
        so the range check and cast of ``pack_weight`` are not repeated."""
        super().__init__(None, None, result_dtype)
        self.register_buffer("_scale", scale.to(torch.float16))
        self.register_buffer("_zero_point", zero_point if zero_point_is_stored else self.pack_weight(zero_point))

    def pack_weight(self, weight: torch.Tensor) -> torch.Tensor:
        if torch.is_floating_point(weight):
            msg = f"Invalid weight dtype {weight.type}. Integer types are supported."
            raise ValueError(msg)
        if torch.any((weight < 0) | (weight > 255)):
            msg = "Weight values are not in [0, 255]."
            raise ValueError(msg)
        return weight.to(torch.uint8)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gs = self._group_size(self._scale.shape, x.shape)
        return self._decompress(x, self._scale, self._zero_point, gs, x.numel()).reshape(x.shape)


class INT8SymmetricWeightsDecompressor(BaseWeightsDecompressor):
    """layers.py:1341-1368."""

    mode = CompressWeightsMode.INT8_SYM

    def __init__(self, scale: torch.Tensor, result_dtype: Optional[torch.dtype] = None):
        super().__init__(None, None, result_dtype)
        self.register_buffer("_scale", scale.to(torch.float16))

    def pack_weight(self, weight: torch.Tensor) -> torch.Tensor:
        if torch.any((weight < -128) | (weight > 127)):
            msg = "Weight values are not in [-128, 127]."
            raise ValueError(msg)
        return weight.to(torch.int8)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gs = self._group_size(self._scale.shape, x.shape)
        return self._decompress(x, self._scale, None, gs, x.numel()).reshape(x.shape)


class INT4AsymmetricWeightsDecompressor(BaseWeightsDecompressor):
    """layers.py:1371-1416."""

    mode = CompressWeightsMode.INT4_ASYM

    def __init__(self, scale, zero_point, compressed_weight_shape, result_shape=None, result_dtype=None,
                 zero_point_shape=None):
        """``zero_point_shape``: given when ``zero_point`` is already nibble-packed ([n / 2, 1] uint8, written by the
        compression kernel); it is then the shape of the unpacked zero points."""
        super().__init__(compressed_weight_shape, result_shape, result_dtype)
        self.register_buffer("_scale", scale.to(torch.float16))
        if zero_point_shape is not None:
            self.zero_point_shape = tuple(zero_point_shape)
            self.register_buffer("_zero_point", zero_point)
        else:
            self.zero_point_shape = tuple(zero_point.shape)
            self.register_buffer("_zero_point", self.pack_weight(zero_point))

    def pack_weight(self, weight: torch.Tensor) -> torch.Tensor:
        if torch.any((weight < 0) | (weight > 15)):
            msg = "Weight values are not in [0, 15]."
            raise ValueError(msg)
        return pack_uint4(weight.to(torch.uint8))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n = 1
        for d in self.compressed_weight_shape:
            n *= d
        gs = self._group_size(self._scale.shape, self.compressed_weight_shape)
        out = self._decompress(x, self._scale, self._zero_point, gs, n)
        return out.reshape(self.result_shape if self.result_shape is not None else self.compressed_weight_shape)


class INT4SymmetricWeightsDecompressor(BaseWeightsDecompressor):
    """layers.py:1419-1460."""

    mode = CompressWeightsMode.INT4_SYM

    def __init__(self, scale, compressed_weight_shape, result_shape=None, result_dtype=None):
        super().__init__(compressed_weight_shape, result_shape, result_dtype)
        self.register_buffer("_scale", scale.to(torch.float16))

    def pack_weight(self, weight: torch.Tensor) -> torch.Tensor:
        if torch.is_floating_point(weight):
            msg = f"Invalid weight dtype {weight.type}. Integer types are supported."
            raise ValueError(msg)
        if torch.any((weight < -8) | (weight > 7)):
            msg = "Tensor values are not in [-8, 7]."
            raise ValueError(msg)
        return pack_int4(weight.to(torch.int8))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n = 1
        for d in self.compressed_weight_shape:
            n *= d
        gs = self._group_size(self._scale.shape, self.compressed_weight_shape)
        out = self._decompress(x, self._scale, None, gs, n)
        return out.reshape(self.result_shape if self.result_shape is not None else self.compressed_weight_shape)


class FloatCodebookWeightsDecompressor(BaseWeightsDecompressor):
    """NF4 / FP4 (fp32 scale) and MXFP4 (E8M0 scale byte) weights stored as nibble codes.  No reference
    counterpart in the torch backend; decoded value times scale in fp32, then the cast."""

    def __init__(self, mode: CompressWeightsMode, scale: torch.Tensor, compressed_weight_shape, result_shape=None,
                 result_dtype=None):
        super().__init__(compressed_weight_shape, result_shape, result_dtype)
        self.mode = CompressWeightsMode(mode)
        self.register_buffer("_scale", scale)  # fp32, or uint8 exponent bytes for MXFP4

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        n = 1
        for d in self.compressed_weight_shape:
            n *= d
        gs = self._group_size(self._scale.shape, self.compressed_weight_shape)
        out = self._decompress(x, self._scale, None, gs, n)
        return out.reshape(self.result_shape if self.result_shape is not None else self.compressed_weight_shape)


class SQMultiply(nn.Module):
    """Per-channel activation scale inserted by AWQ where it cannot be folded into a preceding weight
    (layers.py:1463-1486)."""

    def __init__(self, scale_shape):
        super().__init__()
        self._scale_value = nn.Parameter(torch.empty(scale_shape), requires_grad=False)

    @property
    def scale(self) -> torch.Tensor:
        return self._scale_value

    @scale.setter
    def scale(self, value: torch.Tensor) -> None:
        self._scale_value.data = value

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.mul(x, self._scale_value)
