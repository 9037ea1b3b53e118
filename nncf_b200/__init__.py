"""nncf_b200: a B200 (sm_100a) implementation of the hot path behind ``nncf.compress_weights``.

The package mirrors the reference's weight-compression interface (same names and argument
meaning) and executes the arithmetic with hand-written CUDA kernels through a C ABI
(``libnncf_b200.so``, declared in ``include/nncf_b200.h``).  There is no CPU fallback: importing
the package without the built library raises ``LibraryNotBuiltError``.
"""

from .errors import (InternalError, InvalidGroupSizeError, LibraryNotBuiltError, ParameterNotSupportedError,
                     UnsupportedModelError, ValidationError)
from .parameters import (AdvancedAWQParameters, AdvancedCompressionParameters, AdvancedGPTQParameters,
                         AdvancedLoraCorrectionParameters, AdvancedScaleEstimationParameters, BackupMode, CompressionFormat, CompressWeightsMode,
                         GroupSizeFallbackMode, SensitivityMetric)
from .config import CompressedWeight, WCTensorStatistic, WeightCompressionConfig, WeightCompressionParameters
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from . import weight_lowering
from .weight_lowering import compress_weight
from .compress_api import Dataset, compress_weights
from .serialization import (from_reference_state_dict, get_config, gptq_layout, load_from_config, load_safetensors,
                            reference_state_dict, save_safetensors, strip)

__version__ = "0.1.0"
