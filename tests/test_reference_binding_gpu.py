"""The drop-in boundary, proven on the reference itself: ``nncf.compress_weights`` (the unmodified reference,
imported from ``oracle/_ref``) is run twice on the same seeded model - once as it is, on CPU tensors, and once
on CUDA tensors with ``nncf_b200.reference_binding`` installed at its ``_can_run_optimized`` seam
(src/nncf/quantization/algorithms/weight_compression/weight_lowering.py:687-702), so that the five lowering
functions run in libnncf_b200 while tracing, orchestration, decompressors and ``pack_weight`` stay the
reference's.  The two state dicts must be equal bit for bit: packed weights, fp16 scales, packed zero points.

Skipped when ``oracle/_ref`` has not been made (``python oracle/make_ref.py``)."""

import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference():
    from oracle import ref_loader

    if not ref_loader.available():
        pytest.skip("oracle/_ref is absent (made by oracle/make_ref.py from a checkout of the reference)")
    return ref_loader.load()


def _stacked_linear(n_layers: int, width: int, dtype=torch.float32) -> torch.nn.Module:
    from models import StackedLinear

    return StackedLinear(n_layers, width).to(dtype).eval()


def _compress(nncf, model, device, **kw):
    model = copy.deepcopy(model).to(device)
    example = model.example_input().to(device=device, dtype=model.layers[0].weight.dtype)
    out = nncf.compress_weights(model, dataset=nncf.Dataset([example]), **kw)
    return {k: v.detach().cpu() for k, v in out.state_dict().items()}


def _assert_same(ref: dict, got: dict):
    assert list(ref) == list(got)
    for k in ref:
        assert ref[k].dtype == got[k].dtype and ref[k].shape == got[k].shape, k
        assert torch.equal(ref[k], got[k]), f"{k}: {int((ref[k] != got[k]).sum())} of {ref[k].numel()} elements differ"


@pytest.mark.parametrize("case", ["config1_int4_sym_g128", "int4_asym_g64_all_layers", "int8_asym", "int8_sym_bf16"])
def test_reference_compress_weights_with_the_library_bound_equals_the_reference_on_cpu(case):
    nncf = _reference()
    from nncf_b200 import reference_binding

    M = nncf.CompressWeightsMode
    if case == "config1_int4_sym_g128":
        # 8 stacked Linear(4096 -> 4096) fp32 layers, N(0, 0.02^2) from seed 0; the last layer gets the
        # INT8_ASYM backup precision because all_layers is not set
        model, kw = _stacked_linear(8, 4096), dict(mode=M.INT4_SYM, group_size=128, ratio=1.0)
    elif case == "int4_asym_g64_all_layers":
        model, kw = _stacked_linear(3, 1024), dict(mode=M.INT4_ASYM, group_size=64, ratio=1.0, all_layers=True)
    elif case == "int8_asym":
        model, kw = _stacked_linear(3, 1024), dict(mode=M.INT8_ASYM)
    else:
        model, kw = _stacked_linear(3, 1024, torch.bfloat16), dict(mode=M.INT8_SYM)
    ref = _compress(nncf, model, "cpu", **kw)
    assert any(v.dtype == torch.uint8 or v.dtype == torch.int8 for v in ref.values())
    reference_binding.install()
    try:
        from nncf_b200 import _lib

        before = _lib.launch_count()
        got = _compress(nncf, model, "cuda", **kw)
        assert _lib.launch_count() > before, "the bound library was never called"
    finally:
        reference_binding.uninstall()
    _assert_same(ref, got)
