"""Activation statistics shared by AWQ and ScaleEstimation: the host mirror of
src/nncf/quantization/algorithms/weight_compression/activation_stats.py:20-57 (``process_stats``)
and the per-sample reducers that fill a ``WCTensorStatistic``
(src/nncf/common/tensor_statistics/collectors.py:512-516 ``MeanReducer``, :479-485
``ShapeReducer``).  The statistics are tiny ([hidden] per sample), so stacking and
sub-sampling stay plain tensor indexing on the device; the per-sample reduction of the full
activation runs in the ``nncfb_channel_stats`` kernel."""

from __future__ import annotations

from functools import reduce
from operator import mul
from typing import Optional

import torch

from . import _lib
from .config import WCTensorStatistic


def process_stats(stats: WCTensorStatistic, subset_size: int, act_ch_axis: int = -1):
    """Returns (s, X): s [hidden] = max |mean| over the samples, X [hidden, ~subset_size] = the
    per-sample means of a subset chosen by descending token count with a fixed stride."""
    X = torch.stack(list(stats.mean_values))
    axes = list(range(1, X.ndim)) + [0]
    X_full = X.permute(*axes)
    n = X_full.shape[-1]
    if n > subset_size and subset_size > 0:
        lens = [reduce(mul, tuple(shape[:act_ch_axis]) + tuple(shape[act_ch_axis % len(shape) + 1:]), 1)
                for shape in stats.shape_values]
        step = n // subset_size
        idxs = [i for i, _ in sorted(enumerate(lens), key=lambda p: -p[1])][::step]
        X = X_full[..., idxs]
    else:
        X = X_full
    s = X_full.abs().amax(dim=-1)
    return s, X


def channel_stats(x: torch.Tensor, channel_axis: int = -1, want=("mean",)) -> dict:
    """One pass over an activation: per-channel mean (in x.dtype), population variance, abs-max
    and sum of squares.  ``x`` must have its channel axis last (what Linear inputs have)."""
    if channel_axis % x.ndim != x.ndim - 1:
        x = x.movedim(channel_axis, -1)
    x = x.contiguous()
    if x.dtype not in _lib.DTYPE_IDS or x.dtype == torch.int32:
        x = x.float()
    channels = x.shape[-1]
    tokens = x.numel() // channels
    dev = x.device
    out = {}
    mean = torch.empty(channels, dtype=x.dtype, device=dev) if "mean" in want else None
    var = torch.empty(channels, dtype=torch.float32, device=dev) if "var" in want else None
    amax = torch.empty(channels, dtype=torch.float32, device=dev) if "absmax" in want else None
    sumsq = torch.empty(channels, dtype=torch.float64, device=dev) if "sumsq" in want else None
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.nncfb_channel_stats(_lib.ptr(x), _lib.DTYPE_IDS[x.dtype], tokens, channels, _lib.ptr(mean),
                                                _lib.ptr(var), _lib.ptr(amax), _lib.ptr(sumsq),
                                                _lib.stream_handle(dev)))
    for k, v in (("mean", mean), ("var", var), ("absmax", amax), ("sumsq", sumsq)):
        if v is not None:
            out[k] = v
    return out


class MeanReducer:
    """Per-sample mean over every axis but the channel axis, in the activation's dtype
    (collectors.py:512-516 with the axes chosen in WC/torch_backend.py:147-153)."""

    def __init__(self, channel_axis: int = -1):
        self.channel_axis = channel_axis

    def _reduce_out_of_place(self, x: list) -> list:
        return [channel_stats(x[0], self.channel_axis, ("mean",))["mean"]]


class StatisticsCollector:
    """Accumulates (mean, shape) per calibration sample for one activation, up to ``num_samples``
    (NoopAggregator semantics, collectors.py:631-652)."""

    def __init__(self, channel_axis: int = -1, num_samples: Optional[int] = None):
        self.reducer = MeanReducer(channel_axis)
        self.num_samples = num_samples
        self.stat = WCTensorStatistic()

    def register(self, x: torch.Tensor) -> None:
        if self.num_samples is not None and len(self.stat.mean_values) >= self.num_samples:
            return
        self.stat.mean_values.append(self.reducer._reduce_out_of_place([x])[0])
        self.stat.shape_values.append(tuple(x.shape))
