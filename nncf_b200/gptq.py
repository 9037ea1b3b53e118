"""GPTQ: host mirror of src/nncf/quantization/algorithms/weight_compression/gptq.py
(``_calculate_hessian`` :200-242 and ``_quantize_weights`` :244-379, same argument meaning and
result shapes).  The Hessian contraction runs on the tcgen05 tensor cores (``nncfb_hessian_accumulate``),
the blocked column sweep in ``nncfb_gptq_quantize`` with its trailing updates on the tensor cores too (bf16x3
operand planes, fp32 accumulate); dead-column fix-up, damping and the Cholesky steps are library calls
(torch.linalg / cuSOLVER) like in the reference."""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib
from .activation_stats import channel_stats, process_stats
from .config import WCTensorStatistic, WeightCompressionConfig
from .parameters import CompressWeightsMode


_TRI_LEAF = 1024  # below this size a triangular block is inverted by one library call
# Below this size a product with a triangular factor is one dense product (its zero quarter included): the tensor-core
# product is fastest on large operands, so skipping zeros pays only above a few thousand rows.
_PRODUCT_LEAF = 2048

# Dense fp32 products of the triangular inverse run on the tcgen05 tensor cores (``nncfb_gemm_f32``: bf16x3 operand
# planes, fp32 accumulation) when the operands are on a CUDA device and the shapes qualify; False, CPU tensors
# (the host-side tests) or other shapes use torch.matmul in fp32.
TENSOR_CORE_PRODUCTS = True
_gemm_workspace: dict = {}


def _gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, accumulate: bool = False, alpha: float = 1.0) -> None:
    """out (+)= alpha * a @ b for fp32 matrix views.  ``a`` and ``out`` are both row-major (unit stride along the
    last axis) or both column-major (what torch.linalg.cholesky returns; that is the row-major product
    out^T = b^T a^T); ``b`` may be either - a column-major [k, n] view is a row-major [n, k] matrix, handed to the
    kernel as a transposed operand."""
    if a.stride(1) != 1 and a.stride(0) == 1 and out.stride(0) == 1 and out.stride(1) != 1:
        _gemm(b.T, a.T, out.T, accumulate, alpha)
        return
    m, k = a.shape
    n = b.shape[1]
    b_row = b.stride(1) == 1
    b_col = b.stride(0) == 1
    if (TENSOR_CORE_PRODUCTS and a.is_cuda and a.dtype == torch.float32 and k % 64 == 0 and min(m, n) >= 256 and
            a.stride(1) == 1 and (b_row or b_col) and out.stride(1) == 1 and out.stride(0) % 4 == 0 and
            out.data_ptr() % 16 == 0):
        need = int(_lib.lib.nncfb_gemm_f32_workspace_bytes(m, n, k))
        ws = _gemm_workspace.get(a.device)
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.uint8, device=a.device)
            _gemm_workspace[a.device] = ws   # one buffer per device, grown on demand, reused by every product
        ldb = b.stride(0) if b_row else b.stride(1)
        with torch.cuda.device(a.device):
            rc = _lib.lib.nncfb_gemm_f32(a.data_ptr(), a.stride(0), b.data_ptr(), ldb, 0 if b_row else 1, out.data_ptr(),
                                         out.stride(0), m, n, k, alpha, 1 if accumulate else 0, ws.data_ptr(),
                                         ws.numel(), _lib.stream_handle(a.device))
        if rc != _lib.E_UNSUPPORTED:
            _lib.check(rc)
            return
    if accumulate:
        out.addmm_(a, b, alpha=alpha)
    else:
        torch.matmul(a, b, out=out)
        if alpha != 1.0:
            out.mul_(alpha)


def _aligned_half(n: int) -> int:
    """Split point of an n x n triangle: about half, on a multiple of 128 when that still splits."""
    h = (n // 2 + 127) // 128 * 128
    return h if 0 < h < n else max(n // 2, 1)


def _mul_right_lower(B: torch.Tensor, A: torch.Tensor, out: torch.Tensor) -> None:
    """out = B @ A for a lower-triangular A, without multiplying A's zero quarter (recursively)."""
    h = A.shape[0]
    if h <= (_PRODUCT_LEAF if TENSOR_CORE_PRODUCTS and A.is_cuda else _TRI_LEAF):
        _gemm(B, A, out)
        return
    k = _aligned_half(h)
    _mul_right_lower(B[:, :k], A[:k, :k], out[:, :k])
    _gemm(B[:, k:], A[k:, :k], out[:, :k], accumulate=True)
    _mul_right_lower(B[:, k:], A[k:, k:], out[:, k:])


def _mul_left_lower(C: torch.Tensor, T: torch.Tensor, out: torch.Tensor) -> None:
    """out = C @ T for a lower-triangular C, without multiplying C's zero quarter (recursively)."""
    h = C.shape[0]
    if h <= (_PRODUCT_LEAF if TENSOR_CORE_PRODUCTS and C.is_cuda else _TRI_LEAF):
        _gemm(C, T, out)
        return
    k = _aligned_half(h)
    _mul_left_lower(C[:k, :k], T[:k], out[:k])
    _mul_left_lower(C[k:, k:], T[k:], out[k:])
    _gemm(C[k:, :k], T[:k], out[k:], accumulate=True)


def _tri_inv_into(L: torch.Tensor, out: torch.Tensor) -> None:
    n = L.shape[0]
    if n <= _TRI_LEAF:
        eye = torch.eye(n, dtype=L.dtype, device=L.device)
        out.copy_(torch.linalg.solve_triangular(L, eye, upper=False))
        return
    h = _aligned_half(n)
    _tri_inv_into(L[:h, :h], out[:h, :h])
    _tri_inv_into(L[h:, h:], out[h:, h:])
    # same memory order as L (torch.linalg.cholesky returns column-major factors), so that every product sees
    # operands of one layout
    column_major = L.stride(0) == 1 and L.stride(1) != 1
    tmp = (torch.empty((h, n - h), dtype=L.dtype, device=L.device).T if column_major
           else torch.empty((n - h, h), dtype=L.dtype, device=L.device))
    _mul_right_lower(L[h:, :h], out[:h, :h], tmp)
    _mul_left_lower(out[h:, h:], tmp, out[h:, :h])
    out[h:, :h].neg_()


def lower_triangular_inverse(L: torch.Tensor) -> torch.Tensor:
    """Inverse of a lower-triangular matrix by recursive halving:
        [[A, 0], [B, C]]^-1 = [[A^-1, 0], [-C^-1 B A^-1, C^-1]]
    with the two products done as dense GEMMs that skip the zero quarter of their triangular factor (down to
    blocks of a few thousand rows).  A triangular solve against the identity does n^3 multiply-adds; this does
    about n^3 / 3, as GEMMs - on a CUDA device fp32-faithful tensor-core products (``nncfb_gemm_f32``; 16 ms
    instead of 27 ms with fp32 CUDA-core GEMMs at n = 14336) - and is as accurate (below 1e-6 relative to an
    fp64 inverse)."""
    out = torch.zeros_like(L)
    _tri_inv_into(L, out)
    return out


class GPTQ:
    def __init__(self, damp_percent: float = 0.1, block_size: int = 128, subset_size: int = 128,
                 scale_estimation: bool = False, tensor_cores: bool = True, inverse_factor: str = "reversed"):
        self._damp_percent = damp_percent
        self._block_size = block_size
        self._subset_size = subset_size
        self._scale_estimation = scale_estimation
        self._tensor_cores = tensor_cores
        if inverse_factor not in ("reversed", "reference"):
            msg = f"inverse_factor must be 'reversed' or 'reference', got {inverse_factor!r}"
            raise ValueError(msg)
        self._inverse_factor = inverse_factor

    # ------------------------------------------------------------------------------------------
    def _calculate_hessian(self, node, inputs: Sequence[torch.Tensor], is_3d_weight: bool = False) -> torch.Tensor:
        """gptq.py:200-242: running H = sum (2/n) X^T X over the calibration inputs.
        ``inputs``: activations [b, T, C] or [T, C] (channel last); returns [1, C, C] fp32 like the reference.
        With ``is_3d_weight`` (stacked experts) every input is [E, T, C], counts as one sample, and the result
        is [E, C, C]: expert e accumulates the e-th slice of every input.  ``node`` is accepted for signature
        compatibility and ignored."""
        C = inputs[0].shape[-1]
        dev = inputs[0].device
        experts = 1
        if is_3d_weight:
            experts = 1
            for d in inputs[0].shape[:-2]:
                experts *= int(d)
        H = torch.zeros((experts, C, C), dtype=torch.float32, device=dev)
        nsamples = 0
        with torch.cuda.device(dev):
            st = _lib.stream_handle(dev)
            for inp in inputs:
                batch = 1 if is_3d_weight or inp.ndim != 3 else inp.shape[0]
                x = inp.reshape(experts, -1, C) if is_3d_weight else inp.reshape(1, -1, C)
                if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
                    x = x.float()
                x = x.contiguous()
                alpha = nsamples / (nsamples + batch)
                nsamples += batch
                beta = 2.0 / nsamples
                for e in range(experts):
                    _lib.check(_lib.lib.nncfb_hessian_accumulate(
                        _lib.ptr(H[e]), C, _lib.ptr(x[e]), _lib.DTYPE_IDS[x.dtype], x.shape[1], alpha, beta,
                        1 if self._tensor_cores else 0, None, 0, st))
            _lib.check(_lib.lib.nncfb_hessian_status(st))
        return H

    def accumulate_hessian(self, H: torch.Tensor, x: torch.Tensor, nsamples: int, batch: int) -> int:
        """One step of the running accumulation for callers that stream activations layer by layer:
        H <- H * n/(n+b) + (2/(n+b)) X^T X.  Returns the new sample count."""
        C = H.shape[-1]
        x = x.reshape(-1, C).contiguous()
        dev = H.device
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.nncfb_hessian_accumulate(
                _lib.ptr(H), C, _lib.ptr(x), _lib.DTYPE_IDS[x.dtype], x.shape[0], nsamples / (nsamples + batch),
                2.0 / (nsamples + batch), 1 if self._tensor_cores else 0, None, 0, _lib.stream_handle(dev)))
        return nsamples + batch

    # ------------------------------------------------------------------------------------------
    def prepare_hessian_inverse(self, hessian: torch.Tensor, weight_tensor: torch.Tensor) -> torch.Tensor:
        """gptq.py:269-295: dead columns, damping, upper Cholesky factor U of the inverse (H^-1 = U^T U).
        Mutates both arguments like the reference.

        The reference takes three steps (gptq.py:293-295): L = chol(H), H^-1 = chol_inverse(L),
        U = chol(H^-1, upper).  U^-1 is an upper-triangular V with H = V V^T, and reversing the order of
        rows and columns turns that into an ordinary lower Cholesky factorisation: with J the reversal
        permutation, J H J = (J V J)(J V J)^T and J V J is lower triangular.  So
            U = J * inverse(chol(J H J)) * J
        - one factorisation and one triangular inverse (``lower_triangular_inverse``) instead of two
        factorisations and a full inverse: under a third of the time at C = 14336 and a smaller rounding error (8.7e-7 against 1.4e-6 relative to an fp64
        evaluation); the two routes differ by 1.7e-6 relative, the size of the reference route's own
        rounding.  ``inverse_factor="reference"`` runs the reference's three calls instead."""
        # Nothing here makes the host wait for the GPU (no boolean-mask indexing, no error check that reads a flag
        # back): the host goes on enqueueing the inverse and the sweeps while the factorisation runs.  The
        # factorisation's status travels with the factor and is read by ``check_factor`` / the caller's one check.
        diag = torch.diagonal(hessian)
        dead = diag == 0
        diag.masked_fill_(dead, 1.0)
        weight_tensor.masked_fill_(dead, 0.0)
        damp = self._damp_percent * torch.mean(torch.diagonal(hessian))
        torch.diagonal(hessian).add_(damp)
        if self._inverse_factor == "reference":
            L, info = torch.linalg.cholesky_ex(hessian)
            Hinv = torch.cholesky_inverse(L)
            U, info2 = torch.linalg.cholesky_ex(Hinv, upper=True)
            U = U.contiguous()
            info = torch.maximum(info, info2)
        else:
            # The factorisation itself stays with the library: a blocked Cholesky whose panel solves and trailing
            # updates run as tensor-core products was measured at 19.7 ms against cuSOLVER's 24.8 ms (C = 14336)
            # but five times less accurate (1.4e-6 against 2.6e-7 relative to an fp64 factor), which is not a trade
            # worth making for GPTQ.
            L, info = torch.linalg.cholesky_ex(torch.flip(hessian, (0, 1)))
            U = torch.flip(lower_triangular_inverse(L), (0, 1)).contiguous()
            del L
        U._dead_columns = dead            # reused when several weights share this factor
        U._cholesky_info = info           # 0, or the order of the leading minor that is not positive definite
        return U

    @staticmethod
    def activations_to_wc_statistics(activations: Sequence[torch.Tensor]) -> WCTensorStatistic:
        """gptq.py:382-396: per input, the mean over every axis but the last (in the input's dtype) and its shape."""
        stat = WCTensorStatistic()
        for act in activations:
            stat.shape_values.append(tuple(act.shape))
            stat.mean_values.append(channel_stats(act, -1, ("mean",))["mean"])
        return stat

    def _quantize_weights(self, wc_params, hessian: torch.Tensor, weight_tensor: torch.Tensor,
                          inputs: Optional[Sequence[torch.Tensor]] = None, hinv: Optional[torch.Tensor] = None,
                          statistics: Optional[WCTensorStatistic] = None, check_status: bool = True):
        """gptq.py:244-379.  ``weight_tensor`` [out, C] fp32 is modified in place (trailing updates) like the
        reference's; returns (dequantised weight [out, C] fp32, scales [out, G, 1], zero points or None).
        ``hinv``: the factor returned by ``prepare_hessian_inverse`` for this Hessian, when several weights
        share one input (q/k/v, gate/up) and the factorisation was already done; dead columns of the weight
        are then zeroed from ``hessian``'s diagonal as usual.  With ``scale_estimation=True`` (4-bit integer
        modes) every group's parameters come from ScaleEstimation on the group's current weight, as in
        gptq.py:319-327; the layer statistics are taken from ``statistics`` (per-sample means and shapes, for
        callers that do not keep the activations) or reduced from ``inputs``.  ``check_status=False`` leaves out the
        (synchronising) read of the tensor-core kernels' status flag, for callers that enqueue several sweeps and
        check once afterwards (``check_tensor_core_status``)."""
        config: WeightCompressionConfig = wc_params.compression_config
        assert hessian.ndim == 2, "Hessian should be 2D"
        if weight_tensor.dtype != torch.float32 or not weight_tensor.is_contiguous():
            msg = "weight_tensor must be a contiguous fp32 tensor (the sweep updates it in place)"
            raise ValueError(msg)
        if hinv is None:
            hinv = self.prepare_hessian_inverse(hessian, weight_tensor)
        elif getattr(hinv, "_dead_columns", None) is not None:
            weight_tensor.masked_fill_(hinv._dead_columns, 0.0)
        rows, cols = weight_tensor.shape
        gs = config.group_size if config.group_size != -1 else cols
        dev = weight_tensor.device
        G = cols // gs
        q = torch.empty_like(weight_tensor)
        scale = torch.empty((rows, G), dtype=torch.float32, device=dev)
        zp = torch.empty((rows, G), dtype=torch.int32, device=dev) if config.is_asym_mode else None
        # room for the operand planes of the tensor-core trailing update when that path is wanted
        ws_bytes = int(_lib.lib.nncfb_gptq_workspace_bytes_tensor_cores(rows, cols) if self._tensor_cores
                       else _lib.lib.nncfb_gptq_workspace_bytes(rows))
        workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        use_se = self._scale_estimation and config.is_integer and config.num_bits == 4
        with torch.cuda.device(dev):
            if use_se:
                if statistics is None:
                    if not inputs:
                        msg = "GPTQ with scale estimation needs the layer's inputs or their statistics"
                        raise ValueError(msg)
                    statistics = self.activations_to_wc_statistics(inputs)
                # the reference calls ScaleEstimation.calculate_quantization_params with its defaults
                # (subset 32, 5 + 10 steps, no weight penalty) on each group's slice of the statistics;
                # slicing commutes with process_stats, so it is done once for the whole layer
                s, X = process_stats(statistics, 32)
                s = s.to(device=dev, dtype=torch.float32).contiguous()
                X = X.to(device=dev, dtype=torch.float32).contiguous()
                _lib.check(_lib.lib.nncfb_gptq_quantize_se(
                    _lib.ptr(weight_tensor), rows, cols, _lib.ptr(hinv), _lib.MODE_IDS[config.mode.value], gs,
                    self._block_size, _lib.ptr(s), _lib.ptr(X), X.shape[-1], 5, 10, -1.0, _lib.ptr(q), _lib.ptr(scale),
                    _lib.ptr(zp), _lib.ptr(workspace), ws_bytes, _lib.stream_handle(dev)))
            else:
                _lib.check(_lib.lib.nncfb_gptq_quantize(
                    _lib.ptr(weight_tensor), rows, cols, _lib.ptr(hinv), _lib.MODE_IDS[config.mode.value], gs,
                    self._block_size, _lib.ptr(q), _lib.ptr(scale), _lib.ptr(zp), _lib.ptr(workspace), ws_bytes,
                    _lib.stream_handle(dev)))
            if check_status:
                self.check_factor(hinv)
                if self._tensor_cores:
                    _lib.check(_lib.lib.nncfb_hessian_status(_lib.stream_handle(dev)))  # bounded waits of the TC kernels
        scales = scale.reshape(rows, G, 1)
        zero_points = zp.reshape(rows, G, 1) if zp is not None else None
        if config.group_size == -1:
            scales = scales.squeeze(-1)
            zero_points = zero_points.squeeze(-1) if zero_points is not None else None
        if config.mode not in (CompressWeightsMode.INT8_ASYM, CompressWeightsMode.INT4_ASYM):
            zero_points = None
        return q, scales, zero_points

    @staticmethod
    def check_factor(hinv: torch.Tensor) -> None:
        """Raises like ``torch.linalg.cholesky`` when the factorisation behind ``hinv`` met a Hessian that is not
        positive definite (reads one integer back: synchronises)."""
        info = getattr(hinv, "_cholesky_info", None)
        if info is not None and int(info.max()) != 0:
            msg = (f"linalg.cholesky: The factorization could not be completed because the input is not "
                   f"positive-definite (the leading minor of order {int(info.max())} is not positive-definite).")
            raise torch.linalg.LinAlgError(msg)

    @staticmethod
    def check_tensor_core_status(device: torch.device) -> None:
        """Raises if a bounded wait of a tensor-core kernel ran out in any call on ``device`` since the last check
        (synchronises the current stream)."""
        with torch.cuda.device(device):
            _lib.check(_lib.lib.nncfb_hessian_status(_lib.stream_handle(device)))

    def quantize_stacked(self, wc_params, hessian: torch.Tensor, weight_tensor: torch.Tensor,
                         inputs: Optional[Sequence[torch.Tensor]] = None):
        """The per-expert loop of GPTQ.apply for a 3-D weight [E, out, C] (gptq.py:147-171): expert e is quantised
        with hessian[e] and the e-th slice of every input; results are stacked on axis 0.  Returns (dequantised
        weight [E, out, C], scales [E, out, G, 1], zero points or None)."""
        qs, scs, zps = [], [], []
        for e in range(weight_tensor.shape[0]):
            inp = [i.reshape(weight_tensor.shape[0], -1, i.shape[-1])[e] for i in inputs] if inputs else None
            w = weight_tensor[e].float().contiguous()
            q, sc, zp = self._quantize_weights(wc_params, hessian[e], w, inp)
            qs.append(q)
            scs.append(sc)
            zps.append(zp)
        zero_point = torch.stack(zps) if None not in zps else None
        return torch.stack(qs), torch.stack(scs), zero_point
