"""The allocation-free GPTQ entry point against the regular one, through the C ABI.

Some hosts that embed the library cannot allocate device memory (their runtime's arena owns all of it, or
cudaMalloc's device-wide synchronisation is forbidden in their loop), so they cannot pass the scratch
buffer that `nncfb_gptq_quantize` wants.  `nncfb_gptq_quantize_noalloc` keeps that scratch in a fixed
array inside the library.  Both entry points run the same kernels, so their outputs must be identical;
the second call uses a different, smaller problem so that values the first call left in the shared
scratch would show up if they were ever read.  This file sorts last on purpose: a run that stops at the
first failure has then already executed every other test."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(rows, cols, seed):
    from nncf_b200.gptq import GPTQ

    gen = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(rows, cols, device="cuda", generator=gen) * 0.02
    x = torch.randn(4 * cols, cols, device="cuda", generator=gen)
    H = (2.0 / 4) * (x.T @ x)
    hinv = GPTQ(damp_percent=0.01).prepare_hessian_inverse(H, w)
    return w, hinv


def _run(entry, w, hinv, mode, gs, block):
    from nncf_b200 import _lib

    rows, cols = w.shape
    wt = w.clone()
    q = torch.empty_like(wt)
    scale = torch.empty(rows, cols // gs, device="cuda")
    zp = torch.empty(rows, cols // gs, dtype=torch.int32, device="cuda") if mode.endswith("asym") else None
    st = _lib.stream_handle(wt.device)
    common = (wt.data_ptr(), rows, cols, hinv.data_ptr(), _lib.MODE_IDS[mode], gs, block, q.data_ptr(),
              scale.data_ptr(), None if zp is None else zp.data_ptr())
    if entry == "workspace":
        nbytes = int(_lib.lib.nncfb_gptq_workspace_bytes(rows))
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        _lib.check(_lib.lib.nncfb_gptq_quantize(*common, ws.data_ptr(), nbytes, st))
    else:
        _lib.check(_lib.lib.nncfb_gptq_quantize_noalloc(*common, st))
    torch.cuda.synchronize()
    return q, scale, zp, wt


def test_noalloc_entry_matches_workspace_entry_on_two_calls_in_a_row():
    for rows, cols, mode, gs, block, seed in ((700, 512, "int4_sym", 128, 128, 1), (130, 384, "int4_asym", 64, 128, 2)):
        w, hinv = _problem(rows, cols, seed)
        ref = _run("workspace", w, hinv, mode, gs, block)
        got = _run("noalloc", w, hinv, mode, gs, block)
        for a, b in zip(ref, got):
            if a is None:
                assert b is None
            else:
                assert torch.equal(a, b)
        assert torch.isfinite(got[0]).all()


@pytest.mark.parametrize("rows,cols", [(1024, 1024), (1024, 4096), (2048, 4096)])
def test_noalloc_entry_keeps_the_fp32_trailing_update_for_shapes_the_tensor_core_path_would_take(rows, cols):
    """Rows that are a multiple of 8 with several 128-column blocks qualify for the tensor-core trailing update
    when the workspace is large enough (3.7 MB for 1024 x 1024, exactly 8 MiB for 1024 x 4096, more than the
    built-in array for 2048 x 4096).  The allocation-free entry must not switch to it: it creates a stream
    and events on first use and rounds differently.  Its result has to equal, bit for bit, that of the regular
    entry given the minimum workspace (which always runs the fp32 CUDA-core update)."""
    w, hinv = _problem(rows, cols, 3)
    ref = _run("workspace", w, hinv, "int4_sym", 128, 128)
    got = _run("noalloc", w, hinv, "int4_sym", 128, 128)
    for a, b in zip(ref, got):
        if a is not None:
            assert torch.equal(a, b)


def test_noalloc_entry_rejects_sizes_beyond_its_scratch():
    from nncf_b200 import _lib

    # validation happens before anything is dereferenced or launched
    rc = _lib.lib.nncfb_gptq_quantize_noalloc(16, 16385, 128, 16, _lib.MODE_IDS["int4_sym"], 128, 128, 16, 16, None, None)
    assert rc == _lib.E_TOO_LARGE
    assert b"16384" in _lib.lib.nncfb_last_error()
