"""ScaleEstimation: host mirror of
src/nncf/quantization/algorithms/weight_compression/scale_estimation.py (same static entry point,
arguments and result shapes); the candidate sweep itself is one ``nncfb_scale_estimation`` launch
per weight instead of ~100 whole-tensor operations."""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .activation_stats import process_stats
from .config import CompressedWeight, WCTensorStatistic, WeightCompressionConfig, WeightCompressionParameters


class ScaleEstimation:
    """Per-group scale refinement that minimises the output error of the layer on the calibration
    statistics (scale_estimation.py:38-158)."""

    def __init__(self, subset_size: int = 32, initial_steps: int = 5, scale_steps: int = 10,
                 weight_penalty: float = -1.0):
        self._subset_size = subset_size
        self._initial_steps = initial_steps
        self._scale_steps = scale_steps
        self._weight_penalty = weight_penalty

    def apply(self, all_weight_params: list[WeightCompressionParameters],
              statistics: dict[str, WCTensorStatistic]) -> dict[str, CompressedWeight]:
        """scale_estimation.py:97-158: only 4-bit weights that have statistics are refined."""
        res: dict[str, CompressedWeight] = {}
        for wp in all_weight_params:
            config = wp.compression_config
            if config.num_bits != 4 or wp.weight_name not in statistics:
                res[wp.weight_name] = CompressedWeight()
                continue
            scale, zero_point = self.calculate_quantization_params(
                statistics[wp.weight_name], wp.weight, wp.reduction_axes, config, -1, self._subset_size,
                self._initial_steps, self._scale_steps, self._weight_penalty)
            res[wp.weight_name] = CompressedWeight(None, scale, zero_point, None)
        return res

    @staticmethod
    def calculate_quantization_params(
        statistics: WCTensorStatistic,
        weight: torch.Tensor,
        reduction_axes: tuple,
        config: WeightCompressionConfig,
        act_ch_axis: int = -1,
        subset_size: int = 32,
        initial_steps: int = 5,
        scale_steps: int = 10,
        weight_penalty: float = -1.0,
    ) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
        """scale_estimation.py:160-377.  Returns (scale, zero_point) shaped like the reference:
        [out, G, 1] for grouped, [out, 1] for per-channel configs ([.., 1, out] for weights stored
        [in, out]); the zero point is fp32 like the reference's (it is cast to the scale's dtype)."""
        reduction_axis = reduction_axes[0] if isinstance(reduction_axes, (tuple, list)) else reduction_axes
        s, X = process_stats(statistics, subset_size, act_ch_axis=act_ch_axis)
        if weight.ndim != 2:
            msg = "ScaleEstimation kernel supports 2-D weights; stacked expert weights are processed per expert"
            if weight.ndim == 3:
                return ScaleEstimation._stacked(statistics, weight, reduction_axes, config, act_ch_axis, subset_size,
                                                initial_steps, scale_steps, weight_penalty)
            raise ValueError(msg)
        was_transposed = False
        w = weight
        if reduction_axis % 2 == 0:
            w = w.movedim(-1, -2)
            was_transposed = True
        w = w.contiguous()
        if w.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            w = w.float()
        rows, cols = w.shape
        gs = config.group_size if config.group_size != -1 else cols
        scale, zp = _launch(w, s, X, config, gs, initial_steps, scale_steps, weight_penalty)
        G = cols // gs
        scale = scale.reshape(rows, G, 1)
        zp = zp.reshape(rows, G, 1).to(torch.float32) if zp is not None else None
        if config.group_size == -1:
            scale = scale.squeeze(-2)
            zp = zp.squeeze(-2) if zp is not None else None
        if was_transposed:
            if config.group_size == -1:
                scale = scale.movedim(-1, -2)
                zp = zp.movedim(-1, -2) if zp is not None else None
            else:
                scale = scale.movedim((-1, -2, -3), (-2, -3, -1))
                zp = zp.movedim((-1, -2, -3), (-2, -3, -1)) if zp is not None else None
        return scale, zp

    @staticmethod
    def _stacked(statistics, weight, reduction_axes, config, act_ch_axis, subset_size, initial_steps, scale_steps,
                 weight_penalty):
        """3-D (stacked expert) weights: one launch per expert with that expert's statistics."""
        axis = reduction_axes[0] if isinstance(reduction_axes, (tuple, list)) else reduction_axes
        scales, zps = [], []
        for e in range(weight.shape[0]):
            st = WCTensorStatistic([m[e] for m in statistics.mean_values],
                                   [tuple(s[1:]) for s in statistics.shape_values])
            sc, zp = ScaleEstimation.calculate_quantization_params(
                st, weight[e], (axis - 1,), config, act_ch_axis, subset_size, initial_steps, scale_steps,
                weight_penalty)
            scales.append(sc)
            zps.append(zp)
        zp = torch.stack(zps) if zps[0] is not None else None
        return torch.stack(scales), zp


def _launch(w: torch.Tensor, s: torch.Tensor, X: torch.Tensor, config: WeightCompressionConfig, gs: int,
            initial_steps: int, scale_steps: int, weight_penalty: float):
    dev = w.device
    rows, cols = w.shape
    s32 = s.to(device=dev, dtype=torch.float32).contiguous()
    X32 = X.to(device=dev, dtype=torch.float32).contiguous()
    n = X32.shape[-1]
    scale = torch.empty(rows * (cols // gs), dtype=torch.float32, device=dev)
    zp = torch.empty_like(scale, dtype=torch.int32) if config.is_asym_mode else None
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.nncfb_scale_estimation(
            _lib.ptr(w), _lib.DTYPE_IDS[w.dtype], rows, cols, gs, _lib.MODE_IDS[config.mode.value], _lib.ptr(s32),
            _lib.ptr(X32), n, initial_steps, scale_steps, float(weight_penalty), _lib.ptr(scale), _lib.ptr(zp),
            _lib.stream_handle(dev)))
    return scale, zp
