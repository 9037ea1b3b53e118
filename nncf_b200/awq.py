"""AWQ: host mirror of src/nncf/quantization/algorithms/weight_compression/awq.py
(``_data_aware_step``, ``_data_free_step``, the weight / merge-weight rescale of ``apply``).
Group selection (top-k channels, quantile clipping) is a handful of small tensor operations; the
alpha grid search - 100 x (quantise, dequantise, two matmuls, mean) per group in the reference -
is one ``nncfb_awq_search`` call."""

from __future__ import annotations

from types import SimpleNamespace
from typing import Optional

import torch

from . import _lib
from .activation_stats import process_stats
from .config import WCTensorStatistic, WeightCompressionConfig

FP16_MAX_VALUE = 65504.0
FP16_OVERFLOW_MARGIN = 0.25


class AWQ:
    def __init__(self, subset_size: int = 32, percent_to_apply: float = 0.002, alpha_min: float = 0.0,
                 alpha_max: float = 1.0, steps: int = 100, prefer_data_aware_scaling: bool = True):
        self._subset_size = subset_size
        self._percent_to_apply = percent_to_apply
        self._alpha_min = alpha_min
        self._alpha_max = alpha_max
        self._steps = steps
        self._prefer_data_aware_scaling = prefer_data_aware_scaling
        self._scale_per_target_node: dict = {}

    def _data_aware_step(self, wp, weight: torch.Tensor, statistics: WCTensorStatistic, act_ch_axis: int = -1,
                         prev_weight: Optional[torch.Tensor] = None,
                         prev_statistics: Optional[WCTensorStatistic] = None,
                         _prev_s: Optional[float] = None) -> torch.Tensor:
        """awq.py:243-357.  ``wp`` carries ``compression_config`` and ``reduction_axes`` (a 1-tuple).
        Returns the per-input-channel scale [hidden] (fp32); for a stacked weight [E, ., .] with statistics
        [E, hidden] per sample, [E, hidden]: the reference treats the experts independently (top-k channels,
        groups and alpha search per expert), sharing only the maximum of the previous layer's statistics."""
        config: WeightCompressionConfig = wp.compression_config
        alpha_step = (self._alpha_max - self._alpha_min) / self._steps
        if weight.ndim == 3:
            return self._stacked(wp, weight, statistics, act_ch_axis, prev_weight, prev_statistics)
        s, X = process_stats(statistics, self._subset_size, act_ch_axis)
        s = s.to(torch.float32)
        X = X.to(torch.float32).contiguous()
        if weight.ndim != 2:
            msg = "the AWQ kernel supports 2-D weights and stacks of them"
            raise ValueError(msg)
        reduction_axis = wp.reduction_axes[0]
        dev = weight.device
        hidden = s.shape[-1]
        prev_s, prev_w, prev_rdim = 0.0, None, 0.0
        if prev_statistics is not None and prev_weight is not None:
            ps, _ = process_stats(prev_statistics, self._subset_size, act_ch_axis)
            prev_s = float(ps.to(torch.float32).max().item()) if _prev_s is None else _prev_s
            prev_w = prev_weight.float().abs().mean(dim=reduction_axis).contiguous()
            prev_rdim = float(prev_weight.shape[reduction_axis])
        top_k = max(int(hidden * self._percent_to_apply), 1)
        topk_idxs = torch.argsort(-s, stable=True)[:top_k]
        group_size = config.group_size if config.group_size != -1 else hidden
        groups = sorted({int(i) // group_size for i in topk_idxs.tolist()})
        w = weight
        if reduction_axis == 0:
            w = w.movedim(-1, -2)
        w = w.contiguous()
        if w.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            w = w.float()
        rows, cols = w.shape
        # clipped activation magnitudes per selected group (awq.py:302-304)
        gscale = torch.stack([s[g * group_size:(g + 1) * group_size] for g in groups])
        a_min = torch.quantile(gscale, 0.1, dim=1, keepdim=True).to(torch.float32)
        gscale = torch.minimum(torch.maximum(gscale, a_min), torch.tensor(1e2, device=dev)).contiguous()
        alphas, alpha = [], self._alpha_min
        for _ in range(self._steps):
            alphas.append(alpha)
            alpha += alpha_step
        alphas_t = torch.tensor(alphas, dtype=torch.float32, device=dev)
        gidx = torch.tensor(groups, dtype=torch.int32, device=dev)
        scale = torch.ones(hidden, dtype=torch.float32, device=dev)
        ws_bytes = int(_lib.lib.nncfb_awq_workspace_bytes(rows, len(groups), self._steps))
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.nncfb_awq_search(
                _lib.ptr(w), _lib.DTYPE_IDS[w.dtype], rows, cols, _lib.MODE_IDS[config.mode.value], group_size,
                _lib.ptr(gidx), len(groups), _lib.ptr(gscale), _lib.ptr(X), X.shape[-1], _lib.ptr(alphas_t),
                self._steps, _lib.ptr(prev_w), prev_s, prev_rdim, FP16_OVERFLOW_MARGIN * FP16_MAX_VALUE,
                _lib.ptr(scale), _lib.ptr(workspace), ws_bytes, _lib.stream_handle(dev)))
        return scale

    def _stacked(self, wp, weight, statistics, act_ch_axis, prev_weight, prev_statistics) -> torch.Tensor:
        """One 2-D search per expert with that expert's slice of every statistic (awq.py:276-300 iterates
        (expert, group) pairs; prev_s is the maximum over ALL experts, awq.py:264-266)."""
        axis = wp.reduction_axes[0]
        wp2 = SimpleNamespace(compression_config=wp.compression_config, reduction_axes=(axis - 1,))
        prev_s = None
        if prev_statistics is not None and prev_weight is not None:
            ps, _ = process_stats(prev_statistics, self._subset_size, act_ch_axis)
            prev_s = float(ps.to(torch.float32).max().item())
        scales = []
        for e in range(weight.shape[0]):
            st = WCTensorStatistic([m[e] for m in statistics.mean_values], [tuple(sh[1:]) for sh in statistics.shape_values])
            pst = None
            if prev_statistics is not None:
                pst = WCTensorStatistic([m[e] for m in prev_statistics.mean_values],
                                        [tuple(sh[1:]) for sh in prev_statistics.shape_values])
            scales.append(self._data_aware_step(wp2, weight[e], st, act_ch_axis,
                                                prev_weight[e] if prev_weight is not None else None, pst, prev_s))
        return torch.stack(scales)

    def _data_free_step(self, weight: torch.Tensor, axis: int) -> torch.Tensor:
        """1 / max(mean |W| over `axis`, eps).  awq.py:363-366 (a [hidden]-sized reduction)."""
        eps = torch.finfo(torch.float32).eps
        m = weight.float().abs().mean(dim=axis)
        return 1 / torch.clamp(m, min=eps)

    def apply_to_pair(self, wp, target: torch.nn.Parameter, statistics: Optional[WCTensorStatistic],
                      merge: Optional[torch.nn.Parameter] = None,
                      merge_statistics: Optional[WCTensorStatistic] = None) -> torch.Tensor:
        """The body of awq.py:150-214 for one (target, merge) pair of Linear weights [out, in]: compute
        the scale, multiply the target's input channels by it and the merge layer's output channels by
        its inverse, both cast back to the weight dtype.  Returns the activation scale 1/s."""
        weight = target.data
        is_data_free = statistics is None or not self._prefer_data_aware_scaling
        if is_data_free:
            scale = self._data_free_step(weight, axis=0)
        else:
            scale = self._data_aware_step(wp, weight, statistics, -1, merge.data if merge is not None else None,
                                          merge_statistics)
        a_scale = 1.0 / scale
        target.data = (weight.float() * scale.unsqueeze(0)).to(weight.dtype)
        if merge is not None:
            merge.data = (merge.data.float() * a_scale.unsqueeze(1)).to(merge.dtype)
        return a_scale

    def update_statistics(self, statistics: dict, scales: dict) -> dict:
        """awq.py:424-432: stored means follow the rescaled activations."""
        for name, a_scale in scales.items():
            if name in statistics:
                statistics[name].mean_values = [m * a_scale.to(m.dtype).reshape(m.shape) for m in
                                                statistics[name].mean_values]
        return statistics


def make_wp(config: WeightCompressionConfig, reduction_axes=(1,)) -> SimpleNamespace:
    """Minimal stand-in for WeightCompressionParameters when calling ``_data_aware_step`` directly."""
    return SimpleNamespace(compression_config=config, reduction_axes=tuple(reduction_axes))
