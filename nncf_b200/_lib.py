"""ctypes binding of libnncf_b200.so (the C ABI declared in include/nncf_b200.h).

There is no CPU or PyTorch fallback: if the library is missing or cannot be loaded, importing
this module raises ``LibraryNotBuiltError``; if a call fails, ``NncfbError`` carries the
library's message.  Tensors cross the boundary as raw device pointers plus the current CUDA
stream handle."""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

from .errors import InvalidGroupSizeError, LibraryNotBuiltError

LIB_PATH = Path(__file__).resolve().parent / "libnncf_b200.so"

# status codes / enums (include/nncf_b200.h)
OK, E_BAD_ARG, E_GROUP_SIZE, E_UNSUPPORTED, E_ALIGNMENT, E_CUDA, E_TOO_LARGE, E_TIMEOUT = 0, -1, -2, -3, -4, -5, -6, -7
F32, F16, BF16, I32 = 0, 1, 2, 3
CODES_NONE, CODES_BYTE, CODES_NIBBLE = 0, 1, 2
MODE_IDS = {
    "int8_sym": 0, "int8_asym": 1, "int4_sym": 2, "int4_asym": 3, "nf4": 4, "mxfp4": 5, "fp4": 6, "fp8_e4m3": 7,
    "mxfp8_e4m3": 8,
}
DTYPE_IDS = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int32: I32}


class NncfbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libnncf_b200 error {code}: {message}")
        self.code = code


class QuantizeArgs(C.Structure):
    _fields_ = [
        ("weight", C.c_void_p), ("weight_dtype", C.c_int32), ("mode", C.c_int32),
        ("outer", C.c_int64), ("reduce", C.c_int64), ("inner", C.c_int64), ("group_size", C.c_int64),
        ("pre_scale", C.c_void_p), ("pre_zp", C.c_void_p), ("pre_zp_dtype", C.c_int32), ("codes_format", C.c_int32),
        ("codes_out", C.c_void_p), ("scale_out", C.c_void_p), ("zp_out", C.c_void_p), ("scale_f16_out", C.c_void_p),
        ("scale_e8m0_out", C.c_void_p), ("values_out", C.c_void_p), ("dq_out", C.c_void_p), ("sqerr_out", C.c_void_p),
        ("zp_packed_out", C.c_void_p),
    ]


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        msg = (f"{LIB_PATH} not found. Build it with `python nncf_b200/build.py` (needs nvcc); "
               "nncf_b200 has no CPU fallback.")
        raise LibraryNotBuiltError(msg)
    try:
        lib = C.CDLL(str(LIB_PATH))
    except OSError as e:  # pragma: no cover
        raise LibraryNotBuiltError(f"cannot load {LIB_PATH}: {e}") from e
    vp, i64, i32, u64 = C.c_void_p, C.c_int64, C.c_int32, C.c_uint64
    sigs = {
        "nncfb_abi_version": ([], C.c_int),
        "nncfb_last_error": ([], C.c_char_p),
        "nncfb_quantize": ([C.POINTER(QuantizeArgs), vp], C.c_int),
        "nncfb_quantize_batch": ([C.POINTER(QuantizeArgs), i32, vp], C.c_int),
        "nncfb_scale_estimation": ([vp, i32, i64, i64, i64, i32, vp, vp, i32, i32, i32, C.c_float, vp, vp, vp], C.c_int),
        "nncfb_awq_workspace_bytes": ([i64, i32, i32], C.c_size_t),
        "nncfb_awq_search": ([vp, i32, i64, i64, i32, i64, vp, i32, vp, vp, i32, vp, i32, vp, C.c_float, C.c_float,
                              C.c_float, vp, vp, C.c_size_t, vp], C.c_int),
        "nncfb_channel_stats": ([vp, i32, i64, i64, vp, vp, vp, vp, vp], C.c_int),
        "nncfb_hessian_accumulate": ([vp, i64, vp, i32, i64, C.c_float, C.c_float, i32, vp, C.c_size_t, vp], C.c_int),
        "nncfb_hessian_status": ([vp], C.c_int),
        "nncfb_gptq_workspace_bytes": ([i64], C.c_size_t),
        "nncfb_gptq_workspace_bytes_tensor_cores": ([i64, i64], C.c_size_t),
        "nncfb_gptq_quantize": ([vp, i64, i64, vp, i32, i64, i32, vp, vp, vp, vp, C.c_size_t, vp], C.c_int),
        "nncfb_gptq_quantize_se": ([vp, i64, i64, vp, i32, i64, i32, vp, vp, i32, i32, i32, C.c_float, vp, vp, vp, vp,
                                    C.c_size_t, vp], C.c_int),
        "nncfb_gptq_quantize_noalloc": ([vp, i64, i64, vp, i32, i64, i32, vp, vp, vp, vp], C.c_int),
        "nncfb_gemm_f32_workspace_bytes": ([i64, i64, i64], C.c_size_t),
        "nncfb_gemm_f32": ([vp, i64, vp, i64, i32, vp, i64, i64, i64, i64, C.c_float, i32, vp, C.c_size_t, vp], C.c_int),
        "nncfb_decompress": ([vp, i32, i64, i64, vp, vp, vp, i32, vp], C.c_int),
        "nncfb_pack_nibbles": ([vp, i64, i32, vp, vp], C.c_int),
        "nncfb_unpack_nibbles": ([vp, i64, i32, vp, vp], C.c_int),
        "nncfb_selftest_division": ([i64, u64, vp, vp], C.c_int),
        "nncfb_selftest_bounded_wait": ([vp, i64, vp, i64, vp], C.c_int),
    }
    for name, (argtypes, restype) in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    return lib


lib = _load()
EXPORTED = ["nncfb_abi_version", "nncfb_last_error", "nncfb_quantize", "nncfb_quantize_batch",
            "nncfb_scale_estimation", "nncfb_awq_workspace_bytes", "nncfb_awq_search", "nncfb_channel_stats",
            "nncfb_hessian_accumulate", "nncfb_hessian_status", "nncfb_gptq_workspace_bytes",
            "nncfb_gptq_workspace_bytes_tensor_cores", "nncfb_gptq_quantize",
            "nncfb_gptq_quantize_se", "nncfb_gptq_quantize_noalloc", "nncfb_gemm_f32_workspace_bytes",
            "nncfb_gemm_f32", "nncfb_decompress",
            "nncfb_pack_nibbles", "nncfb_unpack_nibbles",
            "nncfb_selftest_division", "nncfb_selftest_bounded_wait"]


_calls = 0


def launch_count() -> int:
    """How many checked calls into the library this process has made (kernel-launching calls all go
    through ``check``); callers use the difference around a region to count their launches."""
    return _calls


def check(code: int) -> None:
    global _calls
    _calls += 1
    if code == OK:
        return
    message = (lib.nncfb_last_error() or b"").decode("utf-8", "replace")
    if code == E_GROUP_SIZE:
        raise InvalidGroupSizeError(message)
    raise NncfbError(code, message)


def ptr(t: torch.Tensor | None) -> int | None:
    """Device pointer of a contiguous CUDA tensor (None passes NULL)."""
    if t is None:
        return None
    if not t.is_cuda:
        msg = "nncf_b200 kernels run on CUDA tensors only (no CPU fallback)"
        raise ValueError(msg)
    if not t.is_contiguous():
        msg = "tensor must be contiguous"
        raise ValueError(msg)
    return t.data_ptr()


def stream_handle(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
