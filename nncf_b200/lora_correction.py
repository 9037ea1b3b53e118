"""LoRA correction: low-rank adapters that take back part of the 4-bit quantisation noise of a layer.

Restates ``LoraCorrectionAlgorithm`` of the reference
(src/nncf/quantization/algorithms/weight_compression/lora_correction.py:79-271; parameters
src/nncf/quantization/advanced_parameters.py:360-382).  For a weight W [O, H] and its quantised-dequantised value
fq(W), with the layer's activation statistics X [SS, H] (per-sample channel means, ``process_stats``):

  residual = (W - fq(W))^T                                  [H, O]
  start    : rank-R truncated SVD of residual * s, s = the activation magnitudes normalised per quantisation group
  refine   : alternately solve  | U | V = | residual |   for V, and   | E | U = | residual V^+ |   for U
                                | XU|     | X residual|             | X |     | X residual V^+ |
             (num_iterations times; the first block of rows is the regularisation and is left out without it)
  adapters : lora_A = U^T [R, H],  lora_B = V^T [O, R];   layer(x) + (x lora_A^T) lora_B^T

The reference does this on the CPU with a full SVD and QR-based least squares and inserts the adapters into OpenVINO
graphs only.  Here everything stays on the GPU: the residual comes from the decompression kernel, and because only
R = 8 directions are wanted the dense factorisations are replaced by their small equivalents -

  * the R leading singular triplets of the [H, O] matrix from the eigenvectors of its Gram matrix over the
    smaller dimension (fp64 accumulation), which are the same vectors as the full SVD's up to sign;
  * the least-squares problems through their normal equations: for V an R x R system, for U the system
    (I + X^T X) U = B, solved through the SS x SS matrix (I + X X^T) (Woodbury), all in fp64 -

which give the least-squares solutions themselves, not approximations of them; rounding differs from the
reference's LAPACK drivers in the last digits.  The adapters are stored like the reference's: INT8_ASYM per output
channel through the library's compression path (``use_int8_adapters``) or in the layer's dtype.
"""

from __future__ import annotations

import torch
from torch import nn

from .activation_stats import process_stats
from .config import WCTensorStatistic, WeightCompressionConfig
from .parameters import AdvancedLoraCorrectionParameters, CompressWeightsMode

_M = CompressWeightsMode


def _leading_singular_triplets(a: torch.Tensor, rank: int):
    """(U [m, r], S [r], Vh [r, n]) of the r largest singular values of ``a`` [m, n] (fp32 in, fp32 out)."""
    m, n = a.shape
    a64 = a.double()
    if n <= m:
        gram = a64.T @ a64                                   # [n, n]
        evals, evecs = torch.linalg.eigh(gram)
        v = evecs[:, -rank:].flip(1)                         # descending
        s = evals[-rank:].flip(0).clamp_min(0).sqrt()
        u = (a64 @ v) / s.clamp_min(torch.finfo(torch.float64).tiny)
    else:
        gram = a64 @ a64.T                                   # [m, m]
        evals, evecs = torch.linalg.eigh(gram)
        u = evecs[:, -rank:].flip(1)
        s = evals[-rank:].flip(0).clamp_min(0).sqrt()
        v = (a64.T @ u) / s.clamp_min(torch.finfo(torch.float64).tiny)
    return u.float(), s.float(), v.T.float()


class LoraCorrectionAlgorithm:
    """lora_correction.py:79-271."""

    def __init__(self, statistics: dict[str, WCTensorStatistic], lora_correction_params: AdvancedLoraCorrectionParameters):
        self._statistics = statistics
        self._lora_correction_params = lora_correction_params

    @property
    def use_int8_adapters(self) -> bool:
        return self._lora_correction_params.use_int8_adapters

    @staticmethod
    def is_applicable(wc_params) -> bool:
        return wc_params.compression_config.num_bits == 4

    def calculate_adapters(self, weight: torch.Tensor, fq_weight: torch.Tensor, wc_params):
        """lora_A [R, H], lora_B [O, R] for one layer (lora_correction.py:111-137); ``fq_weight`` is the
        dequantised compressed weight."""
        return self.calculate_low_rank_matrices(weight, fq_weight, wc_params.compression_config, wc_params.reduction_axes,
                                                self._lora_correction_params, self._statistics[wc_params.weight_name])

    @staticmethod
    def calculate_low_rank_matrices(weight: torch.Tensor, fq_weight: torch.Tensor, compression_config: WeightCompressionConfig,
                                    reduction_axes, lora_correction_params: AdvancedLoraCorrectionParameters,
                                    layer_statistics: WCTensorStatistic):
        """lora_correction.py:139-271.  ``weight`` and ``fq_weight`` are [O, H] for reduction axis 1 (Linear) or
        [H, O] for axis 0; returns (lora_A [R, H], lora_B [O, R]) in fp32."""
        p = lora_correction_params
        rank, num_iterations = p.adapter_rank, p.num_iterations
        mode = compression_config.mode
        if mode not in (_M.INT4_SYM, _M.INT4_ASYM, _M.NF4):
            msg = f"{mode.value} mode is invalid for Lora Correction algorithm. Supported modes: INT4_SYM, INT4_ASYM, NF4"
            raise ValueError(msg)
        axes = (reduction_axes,) if isinstance(reduction_axes, int) else tuple(reduction_axes)
        assert len(axes) == 1, "Assumed a single reduction axis"
        residual = (weight.float() - fq_weight.float())
        if axes[0] % residual.ndim == 1:
            residual = residual.T
        residual = residual.contiguous()                       # [H, O]
        hidden = residual.shape[0]

        s, x = process_stats(layer_statistics, p.subset_size)  # [H], [H, SS]
        s = s.float().to(residual.device).clone()
        x = x.float().to(residual.device).T.contiguous()       # [SS, H]
        svd_residual = residual
        if compression_config.group_size > 0:
            # activation magnitudes normalised inside every quantisation group: sum to one, then largest = one
            gs = compression_config.group_size
            sg = s.reshape(hidden // gs, gs)
            sg = sg / sg.sum(dim=1, keepdim=True)
            sg = sg / sg.amax(dim=1, keepdim=True)
            svd_residual = residual * sg.reshape(hidden, 1)

        rank = min(rank, *svd_residual.shape)
        u, sv, vh = _leading_singular_triplets(svd_residual, rank)   # [H, R], [R], [R, O]
        v = sv.reshape(-1, 1) * vh                                    # [R, O]

        x64, res64 = x.double(), residual.double()
        noise = x64 @ res64                                           # [SS, O]
        # (I + X^T X)^-1 B = B - X^T (I + X X^T)^-1 (X B): one SS x SS factorisation serves every iteration
        gram_x = x64 @ x64.T
        if p.apply_regularization:
            small = torch.linalg.cholesky(gram_x + torch.eye(x64.shape[0], dtype=torch.float64, device=x.device))
        else:
            x_pinv = torch.linalg.pinv(x64)                           # [H, SS]
        u64, v64 = u.double(), v.double()
        for _ in range(num_iterations):
            # part 1: U fixed, find V
            xu = x64 @ u64                                            # [SS, R]
            if p.apply_regularization:
                lhs = u64.T @ u64 + xu.T @ xu                         # [R, R]
                rhs = u64.T @ res64 + xu.T @ noise                    # [R, O]
            else:
                lhs = xu.T @ xu
                rhs = xu.T @ noise
            v64 = _solve_small(lhs, rhs)
            # part 2: V fixed, find U
            vi = torch.linalg.pinv(v64)                               # [O, R]
            noise_vi = noise @ vi                                     # [SS, R]
            if p.apply_regularization:
                b = res64 @ vi + x64.T @ noise_vi                     # [H, R]
                u64 = b - x64.T @ torch.cholesky_solve(x64 @ b, small)
            else:
                # least-squares solution of X U = noise V^+ of minimum norm (what a rank-revealing driver returns)
                u64 = x_pinv @ noise_vi
        return u64.T.float().contiguous(), v64.T.float().contiguous()


def _solve_small(lhs: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    """Least-squares solution of an R x R normal system; a singular system (rank-deficient start) falls back to
    the pseudo-inverse, which is what a rank-revealing least-squares driver returns."""
    try:
        chol = torch.linalg.cholesky(lhs)
        return torch.cholesky_solve(rhs, chol)
    except RuntimeError:
        return torch.linalg.pinv(lhs, hermitian=True) @ rhs


class LoraAdapters(nn.Module):
    """The pair of small matrices added to a compressed layer: ``y += (x A^T) B^T``.  Stored either densely in the
    layer's dtype or as INT8_ASYM per output channel with the library's decompressors, as the reference stores
    them (src/nncf/quantization/algorithms/weight_compression/openvino_backend.py:178-218)."""

    def __init__(self, lora_a: torch.Tensor, lora_b: torch.Tensor, dtype: torch.dtype, int8: bool):
        super().__init__()
        self.int8 = bool(int8)
        self.rank = int(lora_a.shape[0])
        self.a = _AdapterWeight(lora_a, dtype, int8)
        self.b = _AdapterWeight(lora_b, dtype, int8)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return nn.functional.linear(nn.functional.linear(x, self.a()), self.b())


class _AdapterWeight(nn.Module):
    def __init__(self, value: torch.Tensor, dtype: torch.dtype, int8: bool):
        super().__init__()
        from .decompressors import INT8AsymmetricWeightsDecompressor
        from .weight_lowering import compress_weight

        self.shape = tuple(value.shape)
        if int8:
            cw = compress_weight(value.to(dtype).contiguous(), 1, WeightCompressionConfig(_M.INT8_ASYM, -1), pack=True)
            rows = self.shape[0]
            self.register_buffer("weight", cw.packed.reshape(self.shape))
            self.decompressor = INT8AsymmetricWeightsDecompressor(cw.scale.reshape(rows, 1), cw.zero_point.reshape(rows, 1),
                                                                  dtype)
        else:
            self.register_buffer("weight", value.to(dtype).contiguous())
            self.decompressor = None

    def forward(self) -> torch.Tensor:
        return self.weight if self.decompressor is None else self.decompressor(self.weight)


def _add_adapters(module: nn.Module, args, output):
    return output + module.lora_correction(args[0]).to(output.dtype)


def attach_adapters(module: nn.Module, adapters: LoraAdapters) -> None:
    """Makes ``module`` (a Linear whose weight is compressed) add the adapters' output to its own."""
    module.add_module("lora_correction", adapters)
    module._lora_correction_hook = module.register_forward_hook(_add_adapters)


def detach_adapters(module: nn.Module) -> None:
    module._lora_correction_hook.remove()
    del module._lora_correction_hook
    del module.lora_correction


def empty_adapters(out_ch: int, in_ch: int, rank: int, dtype: torch.dtype, int8: bool, device) -> LoraAdapters:
    """Adapters of the right shapes for a state dict that is about to be loaded."""
    return LoraAdapters(torch.zeros(rank, in_ch, device=device), torch.zeros(out_ch, rank, device=device), dtype, int8)


__all__ = ["LoraCorrectionAlgorithm", "LoraAdapters", "attach_adapters", "detach_adapters", "empty_adapters",
           "AdvancedLoraCorrectionParameters"]
