"""Value types that cross the boundary of the hot path, mirroring
WC/config.py:27-135 (WeightCompressionConfig), WC/parameters.py:19-49 (CompressedWeight) and
src/nncf/common/tensor_statistics/statistics.py:260-300 (WCTensorStatistic), where WC is
src/nncf/quantization/algorithms/weight_compression of the reference.  Tensors are plain
``torch.Tensor`` objects on a CUDA device: there is no tensor-dispatch layer."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .errors import ValidationError
from .parameters import CompressWeightsMode

_M = CompressWeightsMode
_FLOAT_MODES = (_M.NF4, _M.MXFP4, _M.MXFP8_E4M3, _M.FP8_E4M3, _M.FP4, _M.NVFP4, _M.CODEBOOK, _M.ADAPTIVE_CODEBOOK,
                _M.CB4)


@dataclass
class WeightCompressionConfig:
    """How to compress one weight.  ``group_size == -1`` means one scale per output channel."""

    mode: CompressWeightsMode = CompressWeightsMode.INT8_ASYM
    group_size: int = -1

    def __post_init__(self) -> None:
        self.mode = CompressWeightsMode(self.mode)
        if self.group_size == 0 or self.group_size < -1:
            msg = f"Invalid group_size={self.group_size}. Group size must be a positive integer or -1."
            raise ValidationError(msg)

    @property
    def num_bits(self) -> int:
        return 8 if self.mode in (_M.INT8_SYM, _M.INT8_ASYM, _M.FP8_E4M3, _M.MXFP8_E4M3) else 4

    @property
    def is_asym_mode(self) -> bool:
        return self.mode in (_M.INT4_ASYM, _M.INT8_ASYM)

    @property
    def is_integer(self) -> bool:
        return self.mode not in _FLOAT_MODES

    @property
    def is_codebook(self) -> bool:
        return self.mode in (_M.CODEBOOK, _M.CB4, _M.ADAPTIVE_CODEBOOK)

    def __hash__(self) -> int:
        return hash((self.mode.value, self.group_size))


@dataclass
class CompressedWeight:
    """Compressed weight and its decompression parameters.

    ``tensor``: integer codes (int8 / uint8) for integer modes, decoded fp32 grid values for
    float modes - the same content the reference's torch path returns.  The remaining fields are
    additions of this build: ``packed`` (nibble-packed / byte codes as stored in a model),
    ``scale_e8m0`` (exponent byte of MX scales), ``scale_f16`` (the decompressor's fp16 scale
    buffer), ``zero_point_packed`` (the decompressor's zero-point buffer: uint8, nibble-packed for 4-bit modes) and
    ``grouped_shape`` (shape of the codes before packing)."""

    tensor: Optional[torch.Tensor] = None
    scale: Optional[torch.Tensor] = None
    zero_point: Optional[torch.Tensor] = None
    codebook: Optional[torch.Tensor] = None
    global_scale: Optional[torch.Tensor] = None
    packed: Optional[torch.Tensor] = None
    scale_e8m0: Optional[torch.Tensor] = None
    scale_f16: Optional[torch.Tensor] = None
    zero_point_packed: Optional[torch.Tensor] = None
    grouped_shape: Optional[tuple] = None

    def get_unscaled_tensor(self) -> Optional[torch.Tensor]:
        if self.tensor is not None and self.codebook is not None:
            return self.codebook[self.tensor]
        return self.tensor


@dataclass
class WCTensorStatistic:
    """Per-sample activation means and the shapes they were reduced from."""

    mean_values: list = field(default_factory=list)
    shape_values: list = field(default_factory=list)


@dataclass
class WeightCompressionParameters:
    """What to compress and how (WC/config.py:139-167), keyed by module instead of graph node."""

    weight_name: str
    module: torch.nn.Module
    weight_attr: str
    reduction_axes: tuple
    compression_config: Optional[WeightCompressionConfig] = None
    is_embedding: bool = False
    order: int = 0
    # other modules that hold the very same Parameter (tied weights, e.g. lm_head.weight is embed_tokens.weight):
    # the weight is compressed once and every holder gets the decompressor over the one packed tensor
    shared_modules: list = field(default_factory=list)

    @property
    def weight(self) -> torch.Tensor:
        return getattr(self.module, self.weight_attr)

    @property
    def weight_shape(self) -> tuple:
        return tuple(self.weight.shape)

    @property
    def num_weights(self) -> int:
        return int(self.weight.numel())
