"""``compress_weights`` for torch models: the drop-in entry point.

Mirrors ``nncf.compress_weights`` (src/nncf/quantization/quantize_model.py:396-696) and the
orchestration of ``WeightCompression`` (src/nncf/quantization/algorithms/weight_compression/
algorithm.py: option validation :140-295, defaults :74-137, which weights get the primary / backup
precision :540-575 and :961-1088, mixed precision :622-650, group-size validation :652-780,
algorithm order in apply_with_parameters :1127-1232, transform_model in torch_backend.py:424-485) for
models made of ``nn.Linear`` and ``nn.Embedding`` layers.  The reference finds weights by tracing the
model into a graph; here they are found as modules (in first-execution order when a dataset sample is
available, else in registration order), which is the same set for transformer-style models.  All tensor
work goes through the CUDA library; the per-weight loop is one batched launch (``CompressionPlan``).

The stored result uses torch parametrizations: ``module.weight`` becomes a parametrized attribute whose
stored tensor is the packed weight and whose parametrization is the decompressor module, so the model
keeps running and ``state_dict()`` carries packed weights, fp16 scales and packed zero points.
"""

from __future__ import annotations

from typing import Any, Callable, Iterable, Optional

import torch
from torch import nn
from torch.nn.utils import parametrize

from .activation_stats import StatisticsCollector, channel_stats
from .awq import AWQ
from .config import CompressedWeight, WCTensorStatistic, WeightCompressionConfig, WeightCompressionParameters
from .decompressors import (FloatCodebookWeightsDecompressor, INT4AsymmetricWeightsDecompressor,
                            INT4SymmetricWeightsDecompressor, INT8AsymmetricWeightsDecompressor,
                            INT8SymmetricWeightsDecompressor)
from .errors import InvalidGroupSizeError, ParameterNotSupportedError, ValidationError
from . import serialization
from .gptq import GPTQ
from .parameters import (AdvancedCompressionParameters, BackupMode, CompressionFormat, CompressWeightsMode,
                         GroupSizeFallbackMode, SensitivityMetric)
from .pipeline import CompressionPlan
from .scale_estimation import ScaleEstimation
from .lora_correction import LoraAdapters, LoraCorrectionAlgorithm, attach_adapters
from .weight_lowering import get_integer_quantization_error

_M = CompressWeightsMode
INT8_MODES = (_M.INT8_SYM, _M.INT8_ASYM)
SUPPORTED_MODES = (_M.INT8_SYM, _M.INT8_ASYM, _M.INT4_SYM, _M.INT4_ASYM, _M.NF4, _M.MXFP4, _M.FP4)


class Dataset:
    """Iterable of calibration items with an optional transform, like nncf.Dataset
    (src/nncf/data/dataset.py:18-136)."""

    def __init__(self, data_source: Iterable, transform_func: Optional[Callable] = None):
        self._data = data_source
        self._transform = transform_func

    def get_inference_data(self, indices=None):
        for i, item in enumerate(self._data):
            if indices is not None and i not in indices:
                continue
            yield self._transform(item) if self._transform else item


# Model-level GPTQ replays repeated blocks (decoder layers) on cached inputs instead of re-running the model's
# prefix for every layer.  False restores the plain form (one partial forward of the whole model per layer and
# calibration item), which computes the same thing and is kept for models the block detection does not fit.
LAYERWISE_REPLAY = True
# With the block replay, run each block ONCE per micro-batch and pause it at every target layer until that layer
# has been quantised, instead of re-running the block from its start for every layer (see _ResumableBlock).
# False restores the re-running form; both give the same compressed model.
RESUMABLE_REPLAY = True


# Where the time of a model-level GPTQ run goes: seconds per phase ("hessians", "inverse_factors", "sweeps",
# "total"; the calibration forward passes are the remainder), filled when COLLECT_TIMERS is set.  Phases are
# bracketed by CUDA events on the current stream and resolved once at the end, so collecting them adds no
# synchronisation.
COLLECT_TIMERS = False
TIMERS: dict = {}


class _PhaseTimer:
    def __init__(self, enabled: bool):
        self.enabled = enabled
        self.pairs: dict = {}
        self.host: dict = {}

    def start(self, key: str):
        if not self.enabled:
            return None
        import time

        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        self.pairs.setdefault(key, []).append((a, b))
        return (b, self.host, key, time.perf_counter())

    @staticmethod
    def stop(handle) -> None:
        if handle is not None:
            import time

            b, host, key, t0 = handle
            b.record()
            host[key] = host.get(key, 0.0) + time.perf_counter() - t0   # time the host spent issuing the phase

    def resolve(self) -> dict:
        torch.cuda.synchronize()
        out = {k: sum(a.elapsed_time(b) for a, b in v) / 1e3 for k, v in self.pairs.items()}
        out.update({"host_" + k: v for k, v in self.host.items()})
        return out


def _run(model: nn.Module, item: Any) -> None:
    if isinstance(item, dict):
        model(**item)
    elif isinstance(item, (tuple, list)):
        model(*item)
    else:
        model(item)


# --------------------------------------------------------------------------------------------------
# validation and defaults
# --------------------------------------------------------------------------------------------------
def check_user_compression_configuration(mode, subset_size, dataset, ratio, group_size, all_layers, awq,
                                         scale_estimation, gptq, lora_correction, sensitivity_metric, backup_mode,
                                         compression_format, advanced_parameters) -> None:
    """algorithm.py:140-295 and the torch-specific guards of quantize_model.py:497-533."""
    if mode not in SUPPORTED_MODES:
        msg = f"Torch backend does not support {mode.value} mode for weight compression."
        raise ParameterNotSupportedError(msg)
    if lora_correction:
        # the rules of the one reference backend that has the option (quantize_model.py:594-615)
        if dataset is None:
            msg = "Scale estimation, GPTQ or Lora Correction algorithm is defined, but dataset is None."
            raise ParameterNotSupportedError(msg)
        if gptq:
            msg = "Simultaneous use of Lora correction and GPTQ algorithms is not supported. Select one of them."
            raise ParameterNotSupportedError(msg)
        if mode not in (_M.INT4_SYM, _M.INT4_ASYM, _M.NF4):
            msg = f"Lora Correction algorithm is defined, but mode {mode.value} is not one of int4_sym, int4_asym, nf4."
            raise ParameterNotSupportedError(msg)
    if compression_format != CompressionFormat.DQ:
        msg = f"{compression_format.value} compression format is not supported: only the default DQ format is."
        raise ParameterNotSupportedError(msg)
    if advanced_parameters and advanced_parameters.statistics_path:
        msg = "Torch does not support statistics caching."
        raise ParameterNotSupportedError(msg)
    if mode in INT8_MODES:
        if (ratio and ratio != 1) or (group_size and group_size != -1):
            msg = ("INT8 modes require per-channel quantization of all layers in 8 bit. "
                   "Default values of `ratio` (1) and `group_size` (-1) cannot be overridden.")
            raise ParameterNotSupportedError(msg)
        unsupported = {"all_layers": all_layers, "sensitivity_metric": sensitivity_metric, "dataset": dataset,
                       "awq": awq, "scale_estimation": scale_estimation, "gptq": gptq,
                       "lora_correction": lora_correction, "backup_mode": backup_mode}
        bad = [k for k, v in unsupported.items() if v is not None]
        if bad:
            msg = f"INT8 modes do not support {', '.join(bad)} option(s). Set them to None."
            raise ParameterNotSupportedError(msg)
    if ratio is not None and not (0 <= ratio <= 1):
        msg = f"The ratio should be between 0 and 1, but ratio={ratio} is specified."
        raise ValidationError(msg)
    sizes = [subset_size]
    if advanced_parameters:
        sizes += [advanced_parameters.awq_params.subset_size, advanced_parameters.scale_estimation_params.subset_size,
                  advanced_parameters.gptq_params.subset_size, advanced_parameters.lora_correction_params.subset_size]
        if advanced_parameters.lora_correction_params.adapter_rank <= 0:
            rank = advanced_parameters.lora_correction_params.adapter_rank
            msg = f"The lora adapter rank should be positive, but rank={rank} is given."
            raise ValidationError(msg)
    for size in sizes:
        if size <= 0:
            msg = f"The subset_size value should be positive, but subset_size={size} is given."
            raise ValidationError(msg)
    if ratio and dataset is None and sensitivity_metric is not None and \
            sensitivity_metric != SensitivityMetric.WEIGHT_QUANTIZATION_ERROR:
        msg = (f"Mixed precision selection with sensitivity metric={sensitivity_metric.value} "
               "requires a dataset, but it's not provided.")
        raise ValidationError(msg)
    if mode == _M.MXFP4 and group_size not in (None, 32):
        msg = f"MXFP4 and MXFP8_E4M3 types only support group size of 32, group size of {group_size} is given"
        raise ValidationError(msg)
    if (awq or scale_estimation or gptq) and dataset is None and not (awq and not scale_estimation and not gptq):
        msg = "Scale estimation and GPTQ require a dataset."
        raise ValidationError(msg)


def get_weight_compression_configuration(mode, dataset, ratio, group_size, all_layers, awq, scale_estimation, gptq,
                                         sensitivity_metric, backup_mode, advanced_parameters) -> dict:
    """algorithm.py:74-137."""
    if group_size is None:
        group_size = -1 if mode in INT8_MODES else (32 if mode == _M.MXFP4 else 128)
    if backup_mode is None:
        if mode == _M.MXFP4:
            backup_mode = BackupMode.MXFP8_E4M3
        elif mode == _M.FP4:
            backup_mode = BackupMode.FP8_E4M3
        else:
            backup_mode = BackupMode.INT8_ASYM
    if sensitivity_metric is None:
        sensitivity_metric = (SensitivityMetric.WEIGHT_QUANTIZATION_ERROR if dataset is None
                              else SensitivityMetric.MAX_ACTIVATION_VARIANCE)
    return {"mode": mode, "ratio": ratio or 1, "group_size": group_size, "all_layers": all_layers or False,
            "awq": awq or False, "scale_estimation": scale_estimation or False, "gptq": gptq or False,
            "sensitivity_metric": sensitivity_metric, "backup_mode": backup_mode,
            "advanced_parameters": advanced_parameters or AdvancedCompressionParameters()}


def _backup_config(backup_mode: BackupMode, group_size: int = -1) -> Optional[WeightCompressionConfig]:
    """algorithm.py:577-603."""
    if backup_mode == BackupMode.NONE:
        return None
    if backup_mode == BackupMode.FP8_E4M3:
        return WeightCompressionConfig(_M.FP8_E4M3, group_size)
    if backup_mode == BackupMode.MXFP8_E4M3:
        return WeightCompressionConfig(_M.MXFP8_E4M3, 32)
    if backup_mode == BackupMode.INT8_SYM:
        return WeightCompressionConfig(_M.INT8_SYM, -1)
    return WeightCompressionConfig(_M.INT8_ASYM, -1)


# --------------------------------------------------------------------------------------------------
# weights of the model
# --------------------------------------------------------------------------------------------------
def _execution_order(model: nn.Module, sample: Any) -> dict:
    """First-call order of the leaf modules during one forward pass.  The same pass numbers the distinct input
    tensors of the Linear layers (``_LAST_INPUTS``: module id -> number; a layer called with the very tensor the
    Linear before it was called with gets the same number), so that layers fed by one tensor - q / k / v,
    gate / up - can be grouped later without running the model again.  Only the latest input is kept alive."""
    order: dict = {}
    handles = []
    _LAST_INPUTS.clear()
    state = {"last": None, "number": 0}

    def hook(mod, args):
        order.setdefault(id(mod), len(order))
        if isinstance(mod, nn.Linear) and args and isinstance(args[0], torch.Tensor) and id(mod) not in _LAST_INPUTS:
            if args[0] is not state["last"]:
                state["last"] = args[0]
                state["number"] += 1
            _LAST_INPUTS[id(mod)] = state["number"]

    for m in model.modules():
        if isinstance(m, (nn.Linear, nn.Embedding)):
            handles.append(m.register_forward_pre_hook(hook))
    try:
        with torch.no_grad():
            _run(model, sample)
    finally:
        for h in handles:
            h.remove()
        state["last"] = None
    return order


_LAST_INPUTS: dict = {}


def get_weight_compression_parameters(model: nn.Module, ignored_scope: Optional[Iterable[str]] = None,
                                      sample: Any = None) -> list[WeightCompressionParameters]:
    """All Linear (matmul) and Embedding weights in execution order (algorithm.py:961-1088 for the
    two layer kinds handled here; reduction axis = last for both, src/nncf/torch/model_graph_manager.py:350-383).
    A Parameter held by several modules (tied embeddings) appears once, under the module that runs first, like
    the reference's de-duplication by weight name (algorithm.py:992-1007); the other holders are listed in
    ``shared_modules``.  The returned list carries ``is_last_layer_skipped`` (algorithm.py:1003-1006): True
    when the last layer in execution order was dropped as such a duplicate."""
    ignored = set(ignored_scope or [])
    order = _execution_order(model, sample) if sample is not None else {}
    params = []
    for idx, (name, m) in enumerate(model.named_modules(remove_duplicate=False)):
        if not isinstance(m, (nn.Linear, nn.Embedding)) or name in ignored:
            continue
        if m.weight.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            continue
        params.append(WeightCompressionParameters(
            weight_name=name, module=m, weight_attr="weight", reduction_axes=(1,),
            is_embedding=isinstance(m, nn.Embedding), order=order.get(id(m), 10 ** 9 + idx)))
    params.sort(key=lambda p: p.order)
    unique: list = _ParameterList()
    by_weight: dict = {}
    seen_modules: set = set()
    for i, p in enumerate(params):
        if id(p.module) in seen_modules:   # the same module registered under two names
            continue
        seen_modules.add(id(p.module))
        first = by_weight.get(id(p.module.weight))
        if first is not None:
            first.shared_modules.append(p.module)
            unique.is_last_layer_skipped = i == len(params) - 1
            continue
        by_weight[id(p.module.weight)] = p
        unique.append(p)
    return unique


class _ParameterList(list):
    is_last_layer_skipped = False


def _ratio_defining(params, mode, all_layers):
    """algorithm.py:540-575."""
    if mode in INT8_MODES:
        return list(params)
    rd = [p for p in params if not p.is_embedding]
    if not all_layers and not getattr(params, "is_last_layer_skipped", False):
        rd = rd[:-1]
    if all_layers:
        rd += [p for p in params if p.is_embedding]
    return rd


# --------------------------------------------------------------------------------------------------
# statistics
# --------------------------------------------------------------------------------------------------
class _ActivationStats:
    """Forward pre-hooks on the Linear layers: per-sample channel means (AWQ / ScaleEstimation) and the
    mixed-precision metrics (collectors.py:519-540, :924-936), all from one pass over each activation."""

    def __init__(self, params, subset_size: int, metric: Optional[SensitivityMetric]):
        self.collectors = {p.weight_name: StatisticsCollector(-1, subset_size) for p in params if not p.is_embedding}
        self.metric = metric
        self.metric_values = {p.weight_name: [] for p in params if not p.is_embedding}
        self.hawq = {p.weight_name: 0.0 for p in params if not p.is_embedding}
        self._handles = []
        for p in params:
            if p.is_embedding:
                continue
            self._handles.append(p.module.register_forward_pre_hook(self._make_hook(p.weight_name)))

    def _make_hook(self, name):
        def hook(mod, args):
            x = args[0]
            col = self.collectors[name]
            if col.num_samples is not None and len(col.stat.mean_values) >= col.num_samples:
                return
            col.register(x)
            if self.metric in (SensitivityMetric.MEAN_ACTIVATION_VARIANCE, SensitivityMetric.MAX_ACTIVATION_VARIANCE):
                # variance over the sequence axis (-2) per batch row, then mean / max
                vals = [channel_stats(row, -1, ("var",))["var"] for row in x.reshape(-1, x.shape[-2], x.shape[-1])]
                v = torch.stack(vals)
                self.metric_values[name].append(float(v.mean()) if self.metric == SensitivityMetric.MEAN_ACTIVATION_VARIANCE
                                                else float(v.max()))
            elif self.metric == SensitivityMetric.MEAN_ACTIVATION_MAGNITUDE:
                vals = [channel_stats(row, -1, ("absmax",))["absmax"] for row in
                        x.reshape(-1, x.shape[-2], x.shape[-1])]
                self.metric_values[name].append(float(torch.stack(vals).mean()))
            elif self.metric == SensitivityMetric.HESSIAN_INPUT_ACTIVATION:
                ss = float(channel_stats(x, -1, ("sumsq",))["sumsq"].sum())
                self.hawq[name] = (self.hawq[name] + ss) / x.numel()
                self.metric_values[name].append(0.0)
        return hook

    def remove(self):
        for h in self._handles:
            h.remove()

    def statistics(self) -> dict:
        return {k: c.stat for k, c in self.collectors.items() if c.stat.mean_values}

    def activation_score(self, name: str) -> float:
        n = max(len(self.metric_values[name]), 1)
        if self.metric == SensitivityMetric.HESSIAN_INPUT_ACTIVATION:
            return self.hawq[name] * 2 / n
        return sum(self.metric_values[name]) / n


# --------------------------------------------------------------------------------------------------
# AWQ pattern: Linear -> (elementwise multiply) -> Linear
# --------------------------------------------------------------------------------------------------
def find_mul_merge_pairs(model: nn.Module, sample: Any, targets: dict) -> dict:
    """{target name: merge module} for every target Linear whose input is the product of a multiply that
    directly consumes another Linear's output (the MatMul -> Multiply -> MatMul pattern of
    awq_patterns.py:20-43, e.g. up_proj -> (* act(gate)) -> down_proj).  Found by following tensor
    identities through one forward pass."""
    from torch.overrides import TorchFunctionMode

    produced_by: dict = {}   # id(output tensor) -> Linear module
    mul_inputs: dict = {}    # id(mul output) -> ids of its tensor operands
    keep = []                # keeps every seen tensor alive so that ids stay unique
    pairs: dict = {}
    by_module = {id(m): n for n, m in targets.items()}

    class Tracer(TorchFunctionMode):
        def __torch_function__(self, func, types, args=(), kwargs=None):
            out = func(*args, **(kwargs or {}))
            if getattr(func, "__name__", "") in ("mul", "__mul__", "multiply", "__rmul__") and isinstance(out, torch.Tensor):
                ids = [id(a) for a in args if isinstance(a, torch.Tensor)]
                mul_inputs[id(out)] = ids
                keep.extend([out, *[a for a in args if isinstance(a, torch.Tensor)]])
            return out

    handles = []

    def post(mod, args, out):
        if isinstance(out, torch.Tensor):
            produced_by[id(out)] = mod
            keep.append(out)

    def pre(mod, args):
        x = args[0]
        name = by_module.get(id(mod))
        if name is None or not isinstance(x, torch.Tensor):
            return
        for src in mul_inputs.get(id(x), []):
            merge = produced_by.get(src)
            if merge is not None and merge is not mod:
                pairs.setdefault(name, merge)

    for m in model.modules():
        if isinstance(m, nn.Linear):
            handles.append(m.register_forward_hook(post))
            handles.append(m.register_forward_pre_hook(pre))
    try:
        with torch.no_grad(), Tracer():
            _run(model, sample)
    finally:
        for h in handles:
            h.remove()
    return pairs


_SM_COUNT: dict = {}


def _sm_count(device: torch.device) -> int:
    if device not in _SM_COUNT:
        _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[device]


# --------------------------------------------------------------------------------------------------
# GPTQ over several ranks
# --------------------------------------------------------------------------------------------------
class _GptqRanks:
    """The three exchange steps of distributed GPTQ.  With ``group`` None every method is the identity."""

    def __init__(self, group: Any):
        self.group = group
        if group is None:
            self.world, self.rank = 1, 0
        else:
            import torch.distributed as dist

            self.dist = dist
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)

    def share(self, items: list) -> list:
        """This rank's calibration items: every world-th one."""
        if self.world == 1:
            return items
        if len(items) < self.world:
            msg = f"{len(items)} calibration items cannot be shared among {self.world} ranks"
            raise ValidationError(msg)
        return items[self.rank::self.world]

    def combine(self, H: torch.Tensor, n_local: int, stat: Optional[WCTensorStatistic]):
        """The Hessian over all ranks' items from the per-rank running averages: each is (2 / n_r) * sum X^T X over
        the rank's n_r samples, the whole is (2 / n) * sum over everything = sum_r (n_r / n) * H_r."""
        if self.world == 1:
            return H, stat
        n = torch.tensor([float(n_local)], dtype=torch.float64, device=H.device)
        self.dist.all_reduce(n, group=self.group)
        H.mul_(float(n_local) / float(n.item()))
        self.dist.all_reduce(H, group=self.group)
        if stat is not None:
            # per-item channel means and shapes, back in the order of the calibration items (item i lives on
            # rank i % world)
            mine = ([m.cpu() for m in stat.mean_values], list(stat.shape_values))
            everyone: list = [None] * self.world
            self.dist.all_gather_object(everyone, mine, group=self.group)
            merged = WCTensorStatistic()
            for i in range(max(len(e[0]) for e in everyone)):
                for means, shapes in everyone:
                    if i < len(means):
                        merged.mean_values.append(means[i].to(H.device))
                        merged.shape_values.append(shapes[i])
            stat = merged
        return H, stat

    def same_factor(self, hinv: torch.Tensor) -> torch.Tensor:
        """Every rank computed the factor from the same Hessian; rank 0's copy is the one all of them use."""
        if self.world > 1:
            dead, info = getattr(hinv, "_dead_columns", None), getattr(hinv, "_cholesky_info", None)
            self.dist.broadcast(hinv, self.dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                                group=self.group)
            hinv._dead_columns, hinv._cholesky_info = dead, info
        return hinv

    def from_owner(self, owner: int, p: WeightCompressionParameters, q, scale, zero_point):
        """Results of one layer's sweep from the rank that ran it: dequantised weight (in the weight's dtype),
        scales and (asymmetric modes) zero points, allocated here on the other ranks."""
        cfg = p.compression_config
        rows, cols = p.weight.shape
        gs = cfg.group_size if cfg.group_size != -1 else cols
        pshape = (rows, cols // gs, 1) if cfg.group_size != -1 else (rows, 1)
        dev = p.weight.device
        if self.rank != owner:
            q = torch.empty((rows, cols), dtype=p.weight.dtype, device=dev)
            scale = torch.empty(pshape, dtype=torch.float32, device=dev)
            zero_point = torch.empty(pshape, dtype=torch.int32, device=dev) if cfg.is_asym_mode else None
        src = self.dist.get_global_rank(self.group, owner)
        for t in (q, scale, zero_point):
            if t is not None:
                self.dist.broadcast(t, src, group=self.group)
        return q, scale, zero_point


# --------------------------------------------------------------------------------------------------
# the entry point
# --------------------------------------------------------------------------------------------------
def compress_weights(
    model: nn.Module,
    mode: CompressWeightsMode = CompressWeightsMode.INT8_ASYM,
    ratio: Optional[float] = None,
    group_size: Optional[int] = None,
    ignored_scope: Optional[Iterable[str]] = None,
    all_layers: Optional[bool] = None,
    dataset: Optional[Dataset] = None,
    sensitivity_metric: Optional[SensitivityMetric] = None,
    *,
    subset_size: int = 128,
    awq: Optional[bool] = None,
    scale_estimation: Optional[bool] = None,
    gptq: Optional[bool] = None,
    lora_correction: Optional[bool] = None,
    backup_mode: Optional[BackupMode] = None,
    compression_format: CompressionFormat = CompressionFormat.DQ,
    advanced_parameters: Optional[AdvancedCompressionParameters] = None,
    process_group: Any = None,
) -> nn.Module:
    """Compress the weights of ``model`` (CUDA, modified in place and returned).  Same keyword API and
    defaults as ``nncf.compress_weights``; ``ignored_scope`` is a collection of module names.

    ``process_group`` (an addition; the reference runs in one process): a ``torch.distributed`` group whose
    ranks each hold a replica of ``model`` on their own GPU and call this function together with the same
    arguments.  GPTQ is then shared out: every rank runs its share of the calibration items through the
    blocks and the partial Hessians are summed with an all-reduce; the inverse factor is computed on every
    rank and taken from rank 0 of the group; layers that share a factor (q / k / v, gate / up) are swept by
    different ranks and broadcast.  Every rank returns the same compressed model.  Other algorithms run
    replicated."""
    import time

    t_call = time.perf_counter()
    mode = CompressWeightsMode(mode)
    check_user_compression_configuration(mode, subset_size, dataset, ratio, group_size, all_layers, awq,
                                         scale_estimation, gptq, lora_correction, sensitivity_metric, backup_mode,
                                         compression_format, advanced_parameters)
    cfg = get_weight_compression_configuration(mode, dataset, ratio, group_size, all_layers, awq, scale_estimation,
                                               gptq, sensitivity_metric, backup_mode, advanced_parameters)
    adv: AdvancedCompressionParameters = cfg["advanced_parameters"]
    items = list(dataset.get_inference_data()) if dataset is not None else []
    sample = items[0] if items else None
    params = get_weight_compression_parameters(model, ignored_scope, sample)
    if not params:
        return model
    if any(not p.weight.is_cuda for p in params):
        msg = "nncf_b200.compress_weights needs the model on a CUDA device: there is no CPU fallback"
        raise ValueError(msg)

    primary = WeightCompressionConfig(mode, cfg["group_size"])
    backup = _backup_config(cfg["backup_mode"], cfg["group_size"])
    ratio_defining = _ratio_defining(params, mode, cfg["all_layers"])
    rd_names = {p.weight_name for p in ratio_defining}
    for p in params:
        p.compression_config = primary if p.weight_name in rd_names else backup

    # group-size fallback / validation (algorithm.py:652-780)
    if primary.group_size != -1:
        failed = [p for p in ratio_defining if p.weight_shape[1] % primary.group_size != 0]
        fb = adv.group_size_fallback_mode
        for p in failed:
            if fb == GroupSizeFallbackMode.IGNORE:
                p.compression_config = None
            elif fb == GroupSizeFallbackMode.ADJUST:
                gs = primary.group_size
                while gs >= adv.min_adjusted_group_size and p.weight_shape[1] % gs != 0:
                    gs //= 2
                p.compression_config = (WeightCompressionConfig(mode, gs) if gs >= adv.min_adjusted_group_size
                                        and p.weight_shape[1] % gs == 0 else backup)
        still = [p for p in ratio_defining if p.compression_config is not None and p.compression_config.group_size != -1
                 and p.weight_shape[1] % p.compression_config.group_size != 0]
        if still:
            names = "\n\t".join(f'"{p.weight_name}" (channel size: {p.weight_shape[1]})' for p in still)
            msg = (f"Failed to apply group-wise quantization with group size value {primary.group_size}.\n"
                   "Ensure that the group size is divisible by the channel size, or consider setting "
                   "`group_size_fallback_mode` to IGNORE or ADJUST. Failed nodes:\n\t" + names)
            raise InvalidGroupSizeError(msg)
        ratio_defining = [p for p in ratio_defining if p.compression_config is not None]

    # statistics (one calibration pass, hooks on every Linear input)
    need_stats = bool(items) and (cfg["awq"] or cfg["scale_estimation"] or bool(lora_correction) or
                                  (cfg["ratio"] < 1 and cfg["sensitivity_metric"] != SensitivityMetric.WEIGHT_QUANTIZATION_ERROR))
    stats: dict = {}
    act = None
    if need_stats:
        metric = cfg["sensitivity_metric"] if cfg["ratio"] < 1 else None
        act = _ActivationStats(params, subset_size, metric)
        try:
            with torch.no_grad():
                for item in items[:subset_size]:
                    _run(model, item)
        finally:
            act.remove()
        stats = act.statistics()

    # mixed precision (algorithm.py:622-650, mixed_precision.py:71-100)
    if cfg["ratio"] < 1 and ratio_defining and mode not in INT8_MODES:
        scores = []
        metric = cfg["sensitivity_metric"]
        for p in ratio_defining:
            if metric == SensitivityMetric.HESSIAN_INPUT_ACTIVATION:
                wscore = get_integer_quantization_error(p.weight, 1, WeightCompressionConfig(), "frobenius")
            else:
                err = get_integer_quantization_error(p.weight, 1, WeightCompressionConfig(), "max_mean")
                wscore = 1 / (err + torch.finfo(p.weight.dtype).eps)
            if metric == SensitivityMetric.WEIGHT_QUANTIZATION_ERROR:
                scores.append(wscore)
            elif p.is_embedding:
                scores.append(0.0)
            else:
                scores.append(wscore * act.activation_score(p.weight_name))
        total = sum(p.num_weights for p in ratio_defining)
        n4 = 0
        chosen = set()
        for i in sorted(range(len(scores)), key=lambda k: scores[k]):
            p = ratio_defining[i]
            if (n4 + p.num_weights) / total >= cfg["ratio"]:
                break
            chosen.add(p.weight_name)
            n4 += p.num_weights
        for p in ratio_defining:
            if p.weight_name not in chosen:
                p.compression_config = backup

    active = [p for p in params if p.compression_config is not None]
    precomputed: dict[str, CompressedWeight] = {}

    # AWQ (awq.py:124-241): Linear -> multiply -> Linear pairs, 4-bit targets only
    if cfg["awq"] and sample is not None:
        four_bit = {p.weight_name: p.module for p in active if p.compression_config.num_bits == 4 and not p.is_embedding}
        pairs = find_mul_merge_pairs(model, sample, four_bit)
        algo = AWQ(adv.awq_params.subset_size, adv.awq_params.percent_to_apply, adv.awq_params.alpha_min,
                   adv.awq_params.alpha_max, adv.awq_params.steps, adv.awq_params.prefer_data_aware_scaling)
        by_module = {id(p.module): p for p in params}
        scales = {}
        for p in active:
            merge = pairs.get(p.weight_name)
            if merge is None or p.weight_name not in stats:
                continue
            mp = by_module.get(id(merge))
            scales[p.weight_name] = algo.apply_to_pair(p, p.module.weight, stats[p.weight_name], merge.weight,
                                                       stats.get(mp.weight_name) if mp is not None else None)
        algo.update_statistics(stats, scales)

    # GPTQ (gptq.py:82-171) or ScaleEstimation (scale_estimation.py:97-158)
    if cfg["gptq"]:
        # with scale_estimation the reference gives the flag to GPTQ instead of running ScaleEstimation separately
        # (WC/algorithm.py: the GPTQ branch excludes the ScaleEstimation branch)
        g = GPTQ(adv.gptq_params.damp_percent, adv.gptq_params.block_size, adv.gptq_params.subset_size,
                 scale_estimation=cfg["scale_estimation"])
        targets = [p for p in active if not p.is_embedding and p.compression_config.mode not in INT8_MODES]
        ranks = _GptqRanks(process_group)
        cal = ranks.share(items[: adv.gptq_params.subset_size])
        if COLLECT_TIMERS:
            torch.cuda.synchronize()
            t_before = time.perf_counter() - t_call
        timer = _PhaseTimer(COLLECT_TIMERS)
        t_total = timer.start("total")

        def quantise_group(group, runners=None, given=None):
            """One Hessian for layers fed by the very same tensor (q/k/v, gate/up), one factorisation, then
            every layer of the group; weights are replaced only after the whole group saw the same inputs."""
            if given is not None:
                H, layer_stat, n_local = given
            else:
                H, layer_stat, n_local = _layer_hessian(runners, group[0].module, g,
                                                        want_statistics=cfg["scale_estimation"], timer=timer)
            H, layer_stat = ranks.combine(H, n_local, layer_stat)
            hinv = None
            # Layers that share the factor are independent from here on, and a sweep is a chain of small dependent
            # launches whose duration hardly depends on the number of rows (up to one 128-row tile per SM).  In one
            # process the layers of a group with the same configuration are therefore stacked row-wise and swept as
            # ONE weight (q / k / v: one chain of 32 blocks instead of three; rows are independent, so the result is
            # the same).  With several ranks each layer of the group is swept by one rank (layer i by rank
            # i mod world) and broadcast; a layer that is alone in its group is swept by every rank for itself, which
            # gives identical bits everywhere without any exchange.
            dev = group[0].weight.device
            shared_out = ranks.world > 1 and len(group) > 1
            stack = (ranks.world == 1 and len(group) > 1 and
                     all(p.compression_config == group[0].compression_config for p in group) and
                     sum(p.weight.shape[0] for p in group) <= 128 * _sm_count(dev))
            units = [group] if stack else [[p] for p in group]
            for idx, unit in enumerate(units):
                w = torch.cat([p.weight.data.float() for p in unit], 0).contiguous() if len(unit) > 1 else \
                    unit[0].weight.data.float().contiguous()
                if hinv is None:
                    h = timer.start("inverse_factors")
                    hinv = ranks.same_factor(g.prepare_hessian_inverse(H, w))
                    timer.stop(h)
                    h_sweeps = timer.start("sweeps")
                q = sc = zp = None
                if not shared_out or idx % ranks.world == ranks.rank:
                    q, sc, zp = g._quantize_weights(unit[0], H, w, hinv=hinv, statistics=layer_stat, check_status=False)
                    q = q.to(unit[0].weight.dtype)
                if shared_out:
                    q, sc, zp = ranks.from_owner(idx % ranks.world, unit[0], q, sc, zp)
                r0 = 0
                for p in unit:
                    r1 = r0 + p.weight.shape[0]
                    precomputed[p.weight_name] = CompressedWeight(None, sc[r0:r1], zp[r0:r1] if zp is not None else None)
                    p._gptq_weight = q[r0:r1]
                    r0 = r1
            timer.stop(h_sweeps)
            g.check_factor(hinv)
            g.check_tensor_core_status(dev)
            for p in group:
                p.module.weight.data = p._gptq_weight.to(p.weight.dtype)
                del p._gptq_weight

        groups = _same_input_groups(model, sample, targets)
        blocks = _decoder_blocks(model, targets) if LAYERWISE_REPLAY else None
        done: set = set()
        if blocks is not None:
            # Layer-wise engine (the role of src/nncf/quantization/algorithms/layerwise/engine.py:33-198): the
            # inputs of the first repeated block are captured once; each block is then replayed on its own on the
            # outputs of the already-quantised block before it, instead of re-running the whole prefix of the
            # model for every layer.
            h = timer.start("capture_block_inputs")
            replay = _BlockReplay(model, blocks, cal)
            timer.stop(h)
            workers = _ReplayWorkers(len(replay.hidden), targets[0].weight.device) if RESUMABLE_REPLAY else None
            try:
                for bi, block in enumerate(blocks):
                    inside = {id(m) for m in block.modules()}
                    mine = [group for group in groups if id(group[0].module) in inside]
                    if workers is not None and mine:
                        run = _ResumableBlock(workers, replay, bi, [group[0].module for group in mine], g,
                                              cfg["scale_estimation"], timer)
                        try:
                            for gi, group in enumerate(mine):
                                quantise_group(group, given=run.hessian(gi))
                                done.update(p.weight_name for p in group)
                            run.finish()
                        finally:
                            run.close()
                        continue
                    for group in mine:
                        quantise_group(group, replay.runners(bi))
                        done.update(p.weight_name for p in group)
                    replay.advance(bi)
            finally:
                if workers is not None:
                    workers.close()
        for group in groups:  # layers outside the repeated blocks (or models without such blocks)
            if group[0].weight_name not in done:
                quantise_group(group, [lambda item=item: _run(model, item) for item in cal])
        timer.stop(t_total)
        if COLLECT_TIMERS:
            TIMERS.clear()
            TIMERS.update(timer.resolve())
            TIMERS["calibration_forward_and_host"] = TIMERS["total"] - sum(
                TIMERS.get(k, 0.0) for k in ("hessians", "inverse_factors", "sweeps"))
            if "block_segments" in TIMERS:
                TIMERS["block_forward"] = TIMERS["block_segments"] - TIMERS.get("hessians", 0.0)
    elif cfg["scale_estimation"]:
        se = adv.scale_estimation_params
        algo = ScaleEstimation(se.subset_size, se.initial_steps, se.scale_steps, se.weight_penalty)
        precomputed.update({k: v for k, v in algo.apply([p for p in active if not p.is_embedding], stats).items()
                            if v.scale is not None})

    if COLLECT_TIMERS and cfg["gptq"]:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        _transform_model(active, precomputed)
        torch.cuda.synchronize()
        TIMERS["find_layers_and_order"] = t_before
        TIMERS["transform_model"] = time.perf_counter() - t0
        return model
    lora = None
    if lora_correction and not cfg["gptq"]:
        # WC/algorithm.py:1187-1195: the statistics as they stand after AWQ
        lora = LoraCorrectionAlgorithm(stats, adv.lora_correction_params)
    _transform_model(active, precomputed, lora)
    return model


def _same_input_groups(model: nn.Module, sample: Any, targets: list) -> list:
    """Consecutive target layers whose forward receives the identical input tensor (taken from the pass that
    established the execution order when there was one, else from a pass of its own)."""
    seen: dict = {}
    if all(id(p.module) in _LAST_INPUTS for p in targets):
        seen = {p.weight_name: _LAST_INPUTS[id(p.module)] for p in targets}
    else:
        keep = []
        handles = []

        def make(name):
            def hook(mod, args):
                seen.setdefault(name, id(args[0]))
                keep.append(args[0])
            return hook

        for p in targets:
            handles.append(p.module.register_forward_pre_hook(make(p.weight_name)))
        try:
            with torch.no_grad():
                _run(model, sample)
        finally:
            for h in handles:
                h.remove()
    groups: list = []
    for p in targets:
        key = seen.get(p.weight_name)
        if groups and key is not None and seen.get(groups[-1][0].weight_name) == key and \
                groups[-1][0].weight_shape[1] == p.weight_shape[1]:
            groups[-1].append(p)
        else:
            groups.append([p])
    _LAST_INPUTS.clear()
    return groups


def _layer_hessian(runners: list, module: nn.Linear, g: GPTQ, want_statistics: bool = False,
                   timer: Optional[_PhaseTimer] = None):
    """Hessian of one Linear's input over the calibration items, with every previously processed layer already
    holding its quantised weight (the semantics of the reference's layer-wise engine,
    src/nncf/quantization/algorithms/layerwise/openvino_iterator.py:183-231).  ``runners``: one callable per
    calibration item that runs the model (or the block that contains ``module``) on it.  Activations are
    consumed as they appear; nothing is stored but, when the sweep refines its scales with ScaleEstimation, the
    per-sample channel means and shapes (what GPTQ.activations_to_wc_statistics would reduce from stored
    inputs).  Returns (H, statistics or None, number of samples seen)."""
    C = module.in_features
    stat = WCTensorStatistic() if want_statistics else None
    H = torch.zeros(C, C, dtype=torch.float32, device=module.weight.device)
    state = {"n": 0, "split": None}

    class _Stop(Exception):
        pass

    def hook(mod, args):
        x = args[0]
        batch = x.shape[0] if x.ndim == 3 else 1
        h = timer.start("hessians") if timer is not None else None
        state["n"] = g.accumulate_hessian(H, x, state["n"], batch)
        _PhaseTimer.stop(h)
        if stat is not None:
            # a micro-batch stacks several calibration items: statistics are per item
            split = state["split"]
            parts = x.split(split, 0) if split is not None and len(split) > 1 and sum(split) == x.shape[0] else [x]
            for part in parts:
                one = g.activations_to_wc_statistics([part])
                stat.mean_values.append(one.mean_values[0])
                stat.shape_values.append(one.shape_values[0])
        raise _Stop

    h = module.register_forward_pre_hook(hook)
    try:
        with torch.no_grad():
            for run in runners:
                state["split"] = getattr(run, "split", None)
                try:
                    run()
                except _Stop:
                    pass
    finally:
        h.remove()
    from . import _lib

    with torch.cuda.device(H.device):
        # a bounded wait of the tensor-core kernel that ran out in ANY of the accumulation steps raises here
        _lib.check(_lib.lib.nncfb_hessian_status(_lib.stream_handle(H.device)))
    return H, stat, state["n"]


def _decoder_blocks(model: nn.Module, targets: list) -> Optional[list]:
    """The repeated blocks of the model: the nn.ModuleList of callable modules that holds the most target
    layers (decoder layers of a transformer).  None when there is no such list."""
    best = None
    target_ids = {id(p.module) for p in targets}
    for mod in model.modules():
        if not isinstance(mod, nn.ModuleList) or len(mod) < 2:
            continue
        if any(type(b).forward is nn.Module.forward for b in mod):  # containers without a forward of their own
            continue
        n = sum(1 for b in mod for m in b.modules() if id(m) in target_ids)
        if n and (best is None or n > best[0]):
            best = (n, list(mod))
    return best[1] if best else None


def _same_value(a: Any, b: Any) -> bool:
    """Whether two call arguments of different calibration items are interchangeable."""
    if a is b:
        return True
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor):
        return a.shape == b.shape and a.dtype == b.dtype and bool(torch.equal(a, b))
    if isinstance(a, (tuple, list)) and isinstance(b, (tuple, list)):
        return len(a) == len(b) and all(_same_value(x, y) for x, y in zip(a, b))
    if isinstance(a, torch.Tensor) or isinstance(b, torch.Tensor):
        return False
    try:
        return bool(a == b)
    except Exception:  # noqa: BLE001
        return False


class _BlockReplay:
    """Inputs of each repeated block for the calibration items, so that a block can be run on its own.

    The positional and keyword arguments each block is called with are recorded by forward pre-hooks.  The hidden
    state (first positional argument) is kept for the first block only; ``advance`` computes the next block's
    from the current block's output, i.e. through the weights the block holds at that moment.  Objects that
    accumulate state across calls (key / value caches) are not replayed: they are replaced by None.

    Two things keep the cost of the replay near that of the arithmetic:
    * Only the first item runs through the whole model.  If every block received the very same argument objects
      as the first block (masks, position embeddings computed once and handed to every layer, as transformer
      implementations do), the other items' forwards stop at the first block: its inputs are all that is needed.
    * Items whose hidden states have one shape and whose other arguments are equal are stacked along the batch
      axis into micro-batches of up to ``batch_tokens`` tokens, so a block runs a few large calls instead of one
      small call per item.  A stacked activation [B, T, C] counts as B samples in the Hessian, exactly like a
      batch in the reference (WC/gptq.py:229), and per-item statistics are taken from its B slices."""

    class _Stop(Exception):
        pass

    def __init__(self, model: nn.Module, blocks: list, items: list, batch_tokens: int = 32768):
        self.blocks = blocks
        per_item: list = []       # per item: (hidden of block 0, [per block: (rest, kwargs, positional?)])
        state = {"stop_after_first": False, "record": None}
        handles = []

        def make(bi):
            def hook(mod, args, kwargs):
                rec = state["record"]
                if bi == 0:
                    rec["hidden"] = (args[0] if args else kwargs["hidden_states"]).detach()
                kw = {k: (None if _is_stateful_cache(v) else v) for k, v in kwargs.items() if k != "hidden_states"}
                if "use_cache" in kw:
                    kw["use_cache"] = False
                rec["calls"][bi] = (tuple(args[1:]) if args else (), kw, bool(args))
                if bi == 0 and state["stop_after_first"]:
                    raise _BlockReplay._Stop
            return hook

        for bi, b in enumerate(blocks):
            handles.append(b.register_forward_pre_hook(make(bi), with_kwargs=True))
        try:
            with torch.no_grad():
                for k, item in enumerate(items):
                    state["record"] = {"hidden": None, "calls": [None] * len(blocks)}
                    try:
                        _run(model, item)
                    except _BlockReplay._Stop:
                        pass
                    rec = state["record"]
                    if state["stop_after_first"]:
                        rec["calls"] = [rec["calls"][0]] * len(blocks)
                    elif k == 0:
                        first = rec["calls"][0]
                        shared = all(c is not None and len(c[0]) == len(first[0]) and
                                     all(x is y for x, y in zip(c[0], first[0])) and c[1].keys() == first[1].keys() and
                                     all(c[1][n] is first[1][n] for n in first[1]) and c[2] == first[2]
                                     for c in rec["calls"])
                        state["stop_after_first"] = shared
                    per_item.append(rec)
        finally:
            for h in handles:
                h.remove()
        # micro-batches of consecutive compatible items
        self.hidden: list = []                    # per micro-batch: input of the current block
        self.calls: list = [[] for _ in blocks]   # per block, per micro-batch
        self.splits: list = []                    # per micro-batch: leading size of each stacked item
        k = 0
        while k < len(per_item):
            group = [per_item[k]]
            h0 = group[0]["hidden"]
            limit = max(1, batch_tokens // max(1, h0.numel() // h0.shape[-1])) if h0.ndim == 3 else 1
            while (k + len(group) < len(per_item) and len(group) < limit and
                   self._stackable(group[0], per_item[k + len(group)])):
                group.append(per_item[k + len(group)])
            self.hidden.append(torch.cat([g["hidden"] for g in group], 0) if len(group) > 1 else h0)
            self.splits.append([int(g["hidden"].shape[0]) for g in group])
            for bi in range(len(blocks)):
                self.calls[bi].append(group[0]["calls"][bi])
            k += len(group)

    @staticmethod
    def _stackable(a: dict, b: dict) -> bool:
        ha, hb = a["hidden"], b["hidden"]
        if ha.ndim != 3 or ha.shape[1:] != hb.shape[1:] or ha.dtype != hb.dtype:
            return False
        for ca, cb in zip(a["calls"], b["calls"]):
            if ca[2] != cb[2] or not _same_value(ca[0], cb[0]) or ca[1].keys() != cb[1].keys():
                return False
            if not all(_same_value(ca[1][n], cb[1][n]) for n in ca[1]):
                return False
            if ca is a["calls"][0] and all(c is ca for c in a["calls"]) and all(c is cb for c in b["calls"]):
                break  # every block shares the first block's arguments: one comparison covers them all
        return True

    def _call(self, bi: int, k: int):
        rest, kw, positional = self.calls[bi][k]
        if positional:
            return self.blocks[bi](self.hidden[k], *rest, **kw)
        return self.blocks[bi](hidden_states=self.hidden[k], **kw)

    def runners(self, bi: int) -> list:
        out = []
        for k in range(len(self.hidden)):
            fn = lambda k=k: self._call(bi, k)  # noqa: E731
            fn.split = self.splits[k]
            out.append(fn)
        return out

    def advance(self, bi: int) -> None:
        """Replace the stored hidden states by block ``bi``'s outputs (the inputs of block ``bi + 1``)."""
        with torch.no_grad():
            for k in range(len(self.hidden)):
                out = self._call(bi, k)
                self.hidden[k] = (out[0] if isinstance(out, (tuple, list)) else out).detach()


class _ReplayWorkers:
    """A fixed set of threads that serve as coroutines for the paused block forwards, one per micro-batch, kept
    for the whole compression call: libraries keep per-thread state (BLAS handles and their workspaces), which
    is expensive to set up again for every block."""

    def __init__(self, count: int, device: torch.device):
        import threading

        self.device = device
        self.stream = torch.cuda.current_stream(device) if device.type == "cuda" else None
        self.go = [threading.Semaphore(0) for _ in range(count)]
        self.back = threading.Semaphore(0)
        self.local = threading.local()
        self.job = None          # the _ResumableBlock being served
        self.closed = False
        self.threads = [threading.Thread(target=self._serve, args=(k,), daemon=True) for k in range(count)]
        for t in self.threads:
            t.start()

    def _serve(self, k: int) -> None:
        self.local.k = k
        while True:
            self.go[k].acquire()
            if self.closed:
                return
            job = self.job
            try:
                if not job.abort:
                    with torch.no_grad():
                        if self.stream is not None:
                            with torch.cuda.device(self.device), torch.cuda.stream(self.stream):
                                out = job.replay._call(job.bi, k)
                        else:
                            out = job.replay._call(job.bi, k)
                    job.outputs[k] = (out[0] if isinstance(out, (tuple, list)) else out).detach()
                    job.position[k] = len(job.leaders)
            except _ResumableBlock._Abort:
                pass
            except BaseException as exc:  # noqa: BLE001 - reported to the caller, which raises it
                job.errors.append(exc)
            finally:
                job.running[k] = False
                self.back.release()

    def close(self) -> None:
        self.closed = True
        for k, t in enumerate(self.threads):
            if t.is_alive():
                self.go[k].release()
        for t in self.threads:
            t.join(timeout=60)


class _ResumableBlock:
    """One forward pass of a block per micro-batch, paused at the first layer of every target group.

    Quantising the layers of a block one group after another (q/k/v, then o, then gate/up, then down) needs, for
    each group, the group's input computed through the already quantised layers before it.  Re-running the block
    from its start for every group repeats the work of the earlier layers (about 2.5 block passes per block
    including the final pass that produces the next block's inputs).  Here every micro-batch's forward runs in a
    thread of its own that is used as a coroutine: a forward pre-hook on the group's first layer accumulates
    the Hessian from the layer's input and hands control back; when all micro-batches are waiting at that
    layer, the caller quantises the group and resumes them, and the forwards continue through the new weights.
    After the last group they run to the end, and their outputs are the next block's inputs: one block pass
    per block in total.  Exactly one thread (or the caller) runs at any time, in a fixed order, so results do
    not depend on thread scheduling.  The paused forwards keep their intermediate tensors alive: a few GB at
    32 K tokens per micro-batch."""

    class _Abort(Exception):
        pass

    def __init__(self, workers: _ReplayWorkers, replay: "_BlockReplay", bi: int, leaders: list, g: GPTQ,
                 want_statistics: bool, timer: Optional["_PhaseTimer"]):
        self.workers, self.replay, self.bi, self.g, self.timer = workers, replay, bi, g, timer
        self.leaders = leaders
        self.K = len(replay.hidden)
        dev = leaders[0].weight.device
        self.device = dev
        self.H = [torch.zeros(m.in_features, m.in_features, dtype=torch.float32, device=dev) for m in leaders]
        self.n = [0] * len(leaders)
        self.stats = [WCTensorStatistic() if want_statistics else None for _ in leaders]
        self.position = [-1] * self.K         # index of the group a micro-batch is paused at
        self.running = [False] * self.K       # its forward has been started and has not ended
        self.outputs: list = [None] * self.K
        self.errors: list = []
        self.abort = False
        workers.job = self
        self.handles = [m.register_forward_pre_hook(self._make_hook(gi)) for gi, m in enumerate(leaders)]

    def _make_hook(self, gi: int):
        def hook(mod, args):
            k = getattr(self.workers.local, "k", None)
            if k is None or self.workers.job is not self:   # a call from outside the replay
                return
            x = args[0]
            batch = x.shape[0] if x.ndim == 3 else 1
            h = self.timer.start("hessians") if self.timer is not None else None
            self.n[gi] = self.g.accumulate_hessian(self.H[gi], x, self.n[gi], batch)
            _PhaseTimer.stop(h)
            if self.stats[gi] is not None:
                split = self.replay.splits[k]
                parts = x.split(split, 0) if len(split) > 1 and sum(split) == x.shape[0] else [x]
                for part in parts:
                    one = self.g.activations_to_wc_statistics([part])
                    self.stats[gi].mean_values.append(one.mean_values[0])
                    self.stats[gi].shape_values.append(one.shape_values[0])
            self.position[k] = gi
            self.workers.back.release()        # control back to the caller ...
            self.workers.go[k].acquire()       # ... until it resumes this micro-batch
            if self.abort:
                raise _ResumableBlock._Abort
        return hook

    def _resume(self, k: int) -> None:
        h = self.timer.start("block_segments") if self.timer is not None else None   # includes the Hessian step
        self.running[k] = True if self.position[k] == -1 else self.running[k]
        self.workers.go[k].release()
        ok = self.workers.back.acquire(timeout=600)
        _PhaseTimer.stop(h)
        if not ok:
            self.close()
            msg = "a block forward did not come back within 10 minutes"
            raise RuntimeError(msg)
        if self.errors:
            err = self.errors[0]
            self.close()
            raise err

    def hessian(self, gi: int):
        """Run every micro-batch up to group ``gi``'s first layer; returns (H, statistics or None, samples seen)."""
        for k in range(self.K):
            self._resume(k)
            if self.position[k] != gi:
                self.close()
                msg = (f"micro-batch {k} stopped at group {self.position[k]} instead of {gi}: the block does not call "
                       "its layers in the order they were found")
                raise RuntimeError(msg)
        from . import _lib

        if self.device.type == "cuda":
            with torch.cuda.device(self.device):
                _lib.check(_lib.lib.nncfb_hessian_status(_lib.stream_handle(self.device)))
        return self.H[gi], self.stats[gi], self.n[gi]

    def finish(self) -> None:
        """Run every micro-batch to the end of the block and store the outputs as the next block's inputs."""
        for k in range(self.K):
            self._resume(k)
            if self.position[k] != len(self.leaders):
                self.close()
                msg = f"micro-batch {k} reached a target layer a second time"
                raise RuntimeError(msg)
        self.close()
        for k in range(self.K):
            self.replay.hidden[k] = self.outputs[k]

    def close(self) -> None:
        """Remove the hooks; forwards that are still paused are resumed with the abort flag and unwind."""
        self.abort = True
        for h in self.handles:
            h.remove()
        self.handles = []
        for k in range(self.K):
            if self.running[k]:
                self.workers.go[k].release()
                self.workers.back.acquire(timeout=60)


def _is_stateful_cache(v: Any) -> bool:
    return v is not None and not isinstance(v, torch.Tensor) and (
        hasattr(v, "get_seq_length") or type(v).__name__.endswith("Cache"))


def _make_decompressor(p: WeightCompressionParameters, item) -> nn.Module:
    cfg = p.compression_config
    w = p.weight
    out_ch, in_ch = w.shape
    gs = cfg.group_size if cfg.group_size != -1 else in_ch
    G = in_ch // gs
    if cfg.mode in (_M.FP8_E4M3, _M.MXFP8_E4M3):
        grouped = (out_ch, G, gs) if cfg.group_size != -1 else (out_ch, in_ch)
        pshape = (out_ch, G, 1) if cfg.group_size != -1 else (out_ch, 1)
        scale = item.scale_e8m0.reshape(pshape) if cfg.mode == _M.MXFP8_E4M3 else item.scale.reshape(pshape)
        return FloatCodebookWeightsDecompressor(cfg.mode, scale, grouped, tuple(w.shape), w.dtype)
    if cfg.num_bits == 8:
        pshape = (out_ch, 1)
        if cfg.mode == _M.INT8_ASYM:
            stored = getattr(item, "zero_point_packed", None)
            if stored is not None:   # written by the kernel in its stored form: no range check, no cast
                return INT8AsymmetricWeightsDecompressor(item.scale.reshape(pshape), stored.reshape(pshape), w.dtype,
                                                         zero_point_is_stored=True)
            return INT8AsymmetricWeightsDecompressor(item.scale.reshape(pshape), item.zero_point.reshape(pshape), w.dtype)
        return INT8SymmetricWeightsDecompressor(item.scale.reshape(pshape), w.dtype)
    grouped = (out_ch, G, gs) if cfg.group_size != -1 else (out_ch, in_ch)
    pshape = (out_ch, G, 1) if cfg.group_size != -1 else (out_ch, 1)
    if cfg.mode == _M.INT4_SYM:
        return INT4SymmetricWeightsDecompressor(item.scale.reshape(pshape), grouped, tuple(w.shape), w.dtype)
    if cfg.mode == _M.INT4_ASYM:
        stored = getattr(item, "zero_point_packed", None)
        if stored is not None:       # nibble-packed by the kernel (two groups per byte, flat group order)
            n_groups = out_ch * G
            return INT4AsymmetricWeightsDecompressor(item.scale.reshape(pshape), stored.reshape(-1)[: (n_groups + 1) // 2]
                                                     .reshape(-1, 1), grouped, tuple(w.shape), w.dtype,
                                                     zero_point_shape=pshape)
        return INT4AsymmetricWeightsDecompressor(item.scale.reshape(pshape), item.zero_point.reshape(pshape), grouped,
                                                 tuple(w.shape), w.dtype)
    scale = item.scale_e8m0.reshape(pshape) if cfg.mode == _M.MXFP4 else item.scale.reshape(pshape)
    return FloatCodebookWeightsDecompressor(cfg.mode, scale, grouped, tuple(w.shape), w.dtype)


def _transform_model(active: list, precomputed: dict, lora: Optional[LoraCorrectionAlgorithm] = None) -> None:
    """torch_backend.py:424-485: compress every weight and install its decompressor.  Weights without
    precomputed parameters go through one batched launch; the others through compress_weight.  With ``lora`` every
    4-bit Linear with statistics also gets its pair of correcting adapters (openvino_backend.py:362-369)."""
    from .weight_lowering import compress_weight

    plain = [p for p in active if p.weight_name not in precomputed]
    results = {}
    if plain:
        plan = CompressionPlan([(p.weight_name, p.weight.data.contiguous(), p.compression_config) for p in plain],
                               packed_zero_points=True)
        plan.run(use_graph=False)
        for p, it in zip(plain, plan.items):
            results[p.weight_name] = it
    for p in active:
        if p.weight_name in precomputed:
            # a CompressedWeight carries the same fields a plan item does (packed, scale, zero_point, scale_e8m0)
            results[p.weight_name] = compress_weight(p.weight.data, p.reduction_axes, p.compression_config,
                                                     precomputed[p.weight_name], pack=True)
    for p in active:
        it = results[p.weight_name]
        dec = _make_decompressor(p, it)
        four = p.compression_config.num_bits == 4
        packed = it.packed.reshape(-1, 1) if four else it.packed.reshape(p.weight.shape)
        mod = p.module
        dense_shape, dense_dtype = tuple(p.weight.shape), p.weight.dtype
        original = p.weight.data
        mod.weight.requires_grad_(False)
        mod.weight.data = packed
        # tied weights: every holder of the Parameter gets the same decompressor over the one packed tensor
        for holder in [mod, *p.shared_modules]:
            parametrize.register_parametrization(holder, "weight", dec, unsafe=True)
            serialization.record(holder, p.compression_config, dense_shape, dense_dtype)
        if lora is not None and lora.is_applicable(p) and not p.is_embedding and p.weight_name in lora._statistics:
            with torch.no_grad():
                fq = mod.weight.detach()           # what the layer now computes with
                lora_a, lora_b = lora.calculate_adapters(original, fq, p)
                adapters = LoraAdapters(lora_a, lora_b, dense_dtype, lora.use_int8_adapters)
            attach_adapters(mod, adapters)
            serialization.record_adapters(mod, adapters)
