"""CPU-side checks of the C ABI: the library loads without a GPU and exports every symbol that
include/nncf_b200.h declares; argument validation that needs no device works."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols() -> list[str]:
    text = (ROOT / "include" / "nncf_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nncfb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "nncfb_quantize" in syms and "nncfb_last_error" in syms


@pytest.mark.parametrize("sym", declared_symbols())
def test_library_exports_symbol(sym):
    from nncf_b200 import _lib

    assert hasattr(_lib.lib, sym), f"{sym} is declared in the header but not exported"


def test_binding_covers_every_declared_symbol():
    from nncf_b200 import _lib

    assert sorted(_lib.EXPORTED) == declared_symbols()


def test_abi_version_and_host_side_validation():
    from nncf_b200 import _lib

    assert _lib.lib.nncfb_abi_version() == 2
    args = _lib.QuantizeArgs()
    assert _lib.lib.nncfb_quantize(ctypes.byref(args), None) == _lib.E_BAD_ARG
    assert b"weight is null" in _lib.lib.nncfb_last_error()
    args.weight = 16  # never dereferenced: validation fails first
    args.outer, args.reduce, args.inner, args.group_size = 4, 100, 1, 32
    args.mode = _lib.MODE_IDS["int4_sym"]
    assert _lib.lib.nncfb_quantize(ctypes.byref(args), None) == _lib.E_GROUP_SIZE
    assert b"divisible" in _lib.lib.nncfb_last_error()


def test_cpu_tensor_is_rejected_not_emulated():
    import torch

    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig, compress_weight

    with pytest.raises(ValueError, match="no CPU fallback"):
        compress_weight(torch.zeros(4, 32), 1, WeightCompressionConfig(CompressWeightsMode.INT4_SYM, 32))
