"""Public enums and option dataclasses, mirroring the reference's API surface for
``nncf.compress_weights`` (src/nncf/parameters.py:72-209,
src/nncf/quantization/advanced_parameters.py:288-452).  Member names and string values are
the reference's so that user code switches over by changing the import."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum


class _StrEnum(str, Enum):
    def __str__(self) -> str:  # same printing as enum.StrEnum
        return str(self.value)


class CompressWeightsMode(_StrEnum):
    INT8_SYM = "int8_sym"
    INT8_ASYM = "int8_asym"
    INT4_SYM = "int4_sym"
    INT4_ASYM = "int4_asym"
    NF4 = "nf4"
    CB4 = "cb4"
    MXFP4 = "mxfp4"
    MXFP8_E4M3 = "mxfp8_e4m3"
    FP8_E4M3 = "fp8_e4m3"
    FP4 = "fp4"
    NVFP4 = "nvfp4"
    CODEBOOK = "codebook"
    ADAPTIVE_CODEBOOK = "adaptive_codebook"


class CompressionFormat(_StrEnum):
    DQ = "dequantize"
    FQ = "fake_quantize"
    FQ_LORA = "fake_quantize_with_lora"
    FQ_LORA_NLS = "fake_quantize_with_lora_nls"


class BackupMode(_StrEnum):
    NONE = "none"
    INT8_SYM = "int8_sym"
    INT8_ASYM = "int8_asym"
    MXFP8_E4M3 = "mxfp8_e4m3"
    FP8_E4M3 = "fp8_e4m3"


class SensitivityMetric(_StrEnum):
    WEIGHT_QUANTIZATION_ERROR = "weight_quantization_error"
    HESSIAN_INPUT_ACTIVATION = "hessian_input_activation"
    MEAN_ACTIVATION_VARIANCE = "mean_activation_variance"
    MAX_ACTIVATION_VARIANCE = "max_activation_variance"
    MEAN_ACTIVATION_MAGNITUDE = "mean_activation_magnitude"


class GroupSizeFallbackMode(_StrEnum):
    """src/nncf/quantization/advanced_parameters.py: what to do with a weight whose
    channel size is not divisible by the group size."""

    ERROR = "error"
    IGNORE = "ignore"
    ADJUST = "adjust"


@dataclass
class AdvancedAWQParameters:
    """advanced_parameters.py: AWQ defaults (subset 32, 0.2 % of channels, alpha in [0, 1], 100 steps)."""

    subset_size: int = 32
    percent_to_apply: float = 0.002
    alpha_min: float = 0.0
    alpha_max: float = 1.0
    steps: int = 100
    prefer_data_aware_scaling: bool = True


@dataclass
class AdvancedScaleEstimationParameters:
    subset_size: int = 64
    initial_steps: int = 5
    scale_steps: int = 5
    weight_penalty: float = -1.0


@dataclass
class AdvancedGPTQParameters:
    damp_percent: float = 0.1
    block_size: int = 128
    subset_size: int = 128


@dataclass
class AdvancedLoraCorrectionParameters:
    """src/nncf/quantization/advanced_parameters.py:360-382."""
    adapter_rank: int = 8
    num_iterations: int = 3
    apply_regularization: bool = True
    subset_size: int = 128
    use_int8_adapters: bool = True


@dataclass
class AdvancedCompressionParameters:
    statistics_path: str | None = None
    group_size_fallback_mode: GroupSizeFallbackMode | None = None
    min_adjusted_group_size: int = 32
    awq_params: AdvancedAWQParameters = field(default_factory=AdvancedAWQParameters)
    scale_estimation_params: AdvancedScaleEstimationParameters = field(
        default_factory=AdvancedScaleEstimationParameters)
    gptq_params: AdvancedGPTQParameters = field(default_factory=AdvancedGPTQParameters)
    lora_correction_params: AdvancedLoraCorrectionParameters = field(default_factory=AdvancedLoraCorrectionParameters)
