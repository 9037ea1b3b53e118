"""GPU parity of the fused quantisation kernels (through the C ABI) against the reference's
golden outputs and, on larger seeded inputs, against the CPU oracle.

Bars: codes, scales, zero points and dequantised values are compared bit for bit (integer and
byte work; fp32 scales come from the same IEEE operations in the same order).  The squared-error
metric is a sum whose order differs, so it uses the reference test's tolerances
(tests/openvino/optimized_functions/test_compression_functions.py:521-559: rtol 1e-4)."""

import numpy as np
import pytest
import torch
from conftest import golden

pytestmark = pytest.mark.gpu

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def _cfg(mode, gs):
    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig

    return WeightCompressionConfig(CompressWeightsMode(mode), gs)


def _dev(w32, dtype):
    return torch.from_numpy(np.ascontiguousarray(w32)).to("cuda").to(TORCH_DTYPE[dtype])


def _eq(got: torch.Tensor, ref: np.ndarray, what: str):
    g = got.detach().cpu().numpy()
    assert g.shape == ref.shape, f"{what}: shape {g.shape} != {ref.shape}"
    np.testing.assert_array_equal(g, ref, err_msg=what)


@pytest.mark.parametrize("key", golden("quant").index("q"))
def test_compress_weight_matches_reference_golden(key):
    from nncf_b200 import weight_lowering as wl

    g = golden("quant")
    _, name, dtype, mode = key.split("/")
    axis, gs = (int(v) for v in g[key + "/meta"])
    w = _dev(g[f"q/{name}/{dtype}/w"], dtype)
    cfg = _cfg(mode, gs)
    cw = wl.compress_weight(w, axis, cfg)
    _eq(cw.scale, g[key + "/scale"], "scale")
    ref_t = g[key + "/tensor"]
    assert str(cw.tensor.dtype).replace("torch.", "") == str(ref_t.dtype)
    _eq(cw.tensor, ref_t, "tensor")
    if cfg.is_asym_mode:
        _eq(cw.zero_point, g[key + "/zp"], "zero_point")
        assert cw.zero_point.dtype == torch.int32
    else:
        assert cw.zero_point is None
    if cfg.is_integer:
        dq = wl.integer_quantize_dequantize_weight(w, cfg, axis)
    else:
        dq = wl.float_quantize_dequantize_weight(w, cfg, axis)
    _eq(dq, g[key + "/dq"], "dq")
    if (key + "/err_max_mean") in g:
        for red in ("max_mean", "frobenius"):
            got = wl.get_integer_quantization_error(w, axis, cfg, red)
            assert got == pytest.approx(float(g[key + f"/err_{red}"]), rel=1e-4, abs=1e-9)


@pytest.mark.parametrize("key", golden("quant").index("pre"))
def test_precomputed_parameters_match_reference_golden(key):
    from nncf_b200 import CompressedWeight
    from nncf_b200 import weight_lowering as wl

    g = golden("quant")
    mode = key.split("/")[1]
    w = _dev(g[key + "/w"], "f32")
    s = torch.from_numpy(g[key + "/scale"]).cuda()
    zp = torch.from_numpy(g[key + "/zp"]).cuda() if (key + "/zp") in g else None
    cw = wl.compress_weight(w, 1, _cfg(mode, 32), CompressedWeight(None, s, zp))
    _eq(cw.tensor, g[key + "/tensor"], "tensor")
    if zp is not None:
        # the ScaleEstimation path hands the zero point over as fp32
        cw2 = wl.compress_weight(w, 1, _cfg(mode, 32), CompressedWeight(None, s, zp.float()))
        _eq(cw2.tensor, g[key + "/tensor"], "tensor (fp32 zero point)")


def test_precomputed_asym_needs_both():
    from nncf_b200 import weight_lowering as wl

    w = torch.randn(4, 64, device="cuda")
    s = torch.ones(4, 2, 1, device="cuda")
    with pytest.raises(ValueError, match="both scale and zero point"):
        wl.do_integer_quantization(w, _cfg("int4_asym", 32), 1, s, None)


def test_invalid_group_size_raises_reference_error():
    from nncf_b200 import InvalidGroupSizeError
    from nncf_b200 import weight_lowering as wl

    with pytest.raises(InvalidGroupSizeError, match="divisible"):
        wl.compress_weight(torch.randn(4, 100, device="cuda"), 1, _cfg("int4_sym", 32))


ORACLE_CASES = [
    # rows, cols, gs, dtype, kind
    (96, 4096, 128, "bf16", "normal"),
    (64, 4096, 128, "f32", "normal"),
    (33, 1024, 32, "bf16", "normal"),
    (40, 1024, 64, "f16", "uniform"),
    (17, 14336, -1, "bf16", "normal"),
    (31, 4096, -1, "f16", "normal"),
    (9, 2048, -1, "f32", "uniform"),
    (5, 20480, -1, "bf16", "normal"),  # row longer than the register cache of the wide kernel
    (12, 1000, 8, "bf16", "normal"),
    (10, 768, 256, "f32", "normal"),
    (7, 520, 520, "bf16", "normal"),    # wide kernel, one group per row, odd vector count
    (6, 999, 333, "f32", "normal"),     # generic kernel
]
MODES = ["int8_sym", "int8_asym", "int4_sym", "int4_asym", "nf4", "mxfp4", "fp4", "fp8_e4m3", "mxfp8_e4m3"]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("rows,cols,gs,dtype,kind", ORACLE_CASES)
def test_compress_weight_matches_oracle(rows, cols, gs, dtype, kind, mode):
    from oracle import wc_oracle as O

    from nncf_b200 import weight_lowering as wl

    gen = torch.Generator().manual_seed(rows * 7919 + cols)
    if kind == "normal":
        w = torch.randn(rows, cols, generator=gen) * 0.02
    else:
        w = torch.rand(rows, cols, generator=gen) * 2 - 1
    w = w.to(TORCH_DTYPE[dtype])
    w_np = w.float().numpy() if dtype != "f16" else w.numpy()
    ref = O.compress_weight(w_np, 1, mode, gs)
    cfg = _cfg(mode, gs)
    cw = wl.compress_weight(w.cuda(), 1, cfg)
    _eq(cw.scale, ref.scale, "scale")
    _eq(cw.tensor, ref.tensor, "tensor")
    if cfg.is_asym_mode:
        _eq(cw.zero_point, ref.zero_point, "zp")
    # storage path: nibble-packed codes straight from the kernel
    packed = wl.compress_weight(w.cuda(), 1, cfg, pack=True)
    if cfg.num_bits == 4 and cfg.is_integer:
        ref_packed = O.pack_int4(ref.tensor) if mode == "int4_sym" else O.pack_uint4(ref.tensor)
        _eq(packed.packed, ref_packed, "packed")
    elif cfg.num_bits == 4:
        codes = O.nibble_code_nf4(ref.tensor) if mode == "nf4" else O.nibble_code_e2m1(ref.tensor)
        _eq(packed.packed, O.pack_uint4(codes), "packed float codes")
    else:
        if cfg.is_integer:
            _eq(packed.packed, ref.tensor, "byte codes")
        else:
            # E4M3 bytes: the quotient rounded to fp16, then to E4M3 (zero keeps the quotient's sign)
            grouped = w_np.astype(np.float32)
            if gs != -1:
                grouped, _ = O.reshape_for_groups(grouped, 1, gs)
            with np.errstate(over="ignore"):
                h = (grouped / ref.scale).astype(np.float32).astype(np.float16).view(np.uint16)
            _eq(packed.packed, O.f16_bits_to_e4m3_bits(h).reshape(tuple(packed.packed.shape)), "e4m3 bytes")
    _eq(packed.scale_f16, ref.scale.astype(np.float16), "fp16 scale")
    if mode in ("mxfp4", "mxfp8_e4m3"):
        _eq(packed.scale_e8m0, O.e8m0_code(ref.scale), "e8m0")


@pytest.mark.parametrize("mode", ["int4_sym", "int4_asym", "int8_asym", "nf4", "mxfp4"])
@pytest.mark.parametrize("shape,axis,gs", [((256, 48), 0, 32), ((128, 30), 0, -1), ((3, 64, 20), 1, 16),
                                           ((4, 8, 128), 2, 64), ((64, 7), 0, 32)])
def test_strided_and_stacked_layouts_match_oracle(shape, axis, gs, mode):
    from oracle import wc_oracle as O

    from nncf_b200 import weight_lowering as wl

    gen = torch.Generator().manual_seed(sum(shape))
    w = (torch.randn(*shape, generator=gen) * 0.05).to(torch.bfloat16)
    ref = O.compress_weight(w.float().numpy(), axis, mode, gs)
    cfg = _cfg(mode, gs)
    cw = wl.compress_weight(w.cuda(), axis, cfg)
    _eq(cw.scale, ref.scale, "scale")
    _eq(cw.tensor, ref.tensor, "tensor")
    if cfg.is_asym_mode:
        _eq(cw.zero_point, ref.zero_point, "zp")
    if cfg.num_bits == 4 and cfg.is_integer:
        packed = wl.compress_weight(w.cuda(), axis, cfg, pack=True)
        ref_packed = O.pack_int4(ref.tensor) if mode == "int4_sym" else O.pack_uint4(ref.tensor)
        _eq(packed.packed, ref_packed, "packed")


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("mode", ["int4_sym", "int4_asym", "int8_sym", "int8_asym", "nf4", "mxfp4"])
@pytest.mark.parametrize("shape,axis,gs", [((1024, 64), 0, -1), ((2, 1536, 40), 1, 512), ((640, 16), 0, 640),
                                           ((3, 520, 72), 1, -1)])
def test_tall_column_groups_stored_form_matches_oracle(shape, axis, gs, mode, dtype):
    """Weights stored [in, out] (or stacked [E, in, out]) with tall groups - per-channel backup precision or a
    group size of 512 and more - take the tiled column kernel: packed codes and every parameter output
    against the oracle, for rows beyond the register cache (more than 32 * 8 rows) and ragged column tiles."""
    from oracle import wc_oracle as O

    from nncf_b200 import weight_lowering as wl

    gen = torch.Generator().manual_seed(sum(shape) + len(mode))
    w = (torch.randn(*shape, generator=gen) * 0.05).to(TORCH_DTYPE[dtype])
    w_np = w.numpy() if dtype == "f16" else w.float().numpy()
    ref = O.compress_weight(w_np, axis, mode, gs)
    cfg = _cfg(mode, gs)
    st = wl.compress_weight(w.cuda(), axis, cfg, pack=True)
    _eq(st.scale, ref.scale, "scale")
    if cfg.is_asym_mode:
        _eq(st.zero_point, ref.zero_point, "zp")
    if cfg.is_integer and cfg.num_bits == 4:
        _eq(st.packed, O.pack_int4(ref.tensor) if mode == "int4_sym" else O.pack_uint4(ref.tensor), "packed")
    elif cfg.is_integer:
        _eq(st.packed, ref.tensor, "byte codes")
    else:
        codes = O.nibble_code_nf4(ref.tensor) if mode == "nf4" else O.nibble_code_e2m1(ref.tensor)
        _eq(st.packed, O.pack_uint4(codes), "packed float codes")
    _eq(st.scale_f16, ref.scale.astype(np.float16), "fp16 scale")
    if mode == "mxfp4":
        _eq(st.scale_e8m0, O.e8m0_code(ref.scale), "e8m0")


def test_division_selftest_has_no_mismatch():
    from nncf_b200 import _lib

    out = torch.zeros(1, dtype=torch.int64, device="cuda")
    for seed in (1, 2, 3):
        _lib.check(_lib.lib.nncfb_selftest_division(1 << 28, seed, out.data_ptr(), _lib.stream_handle(out.device)))
        assert int(out.item()) == 0


def test_pack_unpack_round_trip():
    from nncf_b200 import _lib

    codes = torch.randint(-8, 8, (1 << 20,), dtype=torch.int8, device="cuda")
    packed = torch.empty(codes.numel() // 2, dtype=torch.uint8, device="cuda")
    back = torch.empty_like(codes)
    st = _lib.stream_handle(codes.device)
    _lib.check(_lib.lib.nncfb_pack_nibbles(codes.data_ptr(), codes.numel(), 8, packed.data_ptr(), st))
    _lib.check(_lib.lib.nncfb_unpack_nibbles(packed.data_ptr(), packed.numel(), 8, back.data_ptr(), st))
    assert torch.equal(codes, back)
    ref = ((codes[0::2].to(torch.int16) + 8) | ((codes[1::2].to(torch.int16) + 8) << 4)).to(torch.uint8)
    assert torch.equal(packed, ref)


@pytest.mark.parametrize("mode,gs", [("int4_sym", 128), ("int4_asym", 128), ("int8_asym", -1), ("nf4", 128),
                                     ("mxfp4", 32)])
def test_full_size_properties(mode, gs):
    """Llama-3-8B gate_proj size (14336 x 4096 bf16): size-independent properties.
    (1) |dq - w| <= |scale| / 2 wherever the code is not clipped (integer modes);
    (2) quantising the dequantised weight with the same parameters reproduces the codes."""
    from nncf_b200 import CompressedWeight
    from nncf_b200 import weight_lowering as wl

    torch.manual_seed(1)
    w = (torch.randn(14336, 4096, device="cuda") * 0.02).to(torch.bfloat16)
    cfg = _cfg(mode, gs)
    if cfg.is_integer:
        dq, cw = wl.integer_quantize_dequantize_weight(w, cfg, 1, return_compressed_weight=True)
    else:
        dq, cw = wl.float_quantize_dequantize_weight(w, cfg, 1, return_compressed_weight=True)
    wg = w.float().reshape(dq.shape)
    if cfg.is_integer:
        lo, hi = (0, 2 ** cfg.num_bits - 1) if cfg.is_asym_mode else (-(2 ** (cfg.num_bits - 1)), 2 ** (cfg.num_bits - 1) - 1)
        inside = (cw.tensor > lo) & (cw.tensor < hi)
        # w/s + zp is rounded to fp32 before rint: up to half an ulp of 255 (1.5e-5) on top of 0.5
        bound = cw.scale.abs() * (0.5 + 1e-4) + 1e-12
        assert bool((((dq - wg).abs() <= bound) | ~inside).all())
        again = wl.do_integer_quantization(dq, cfg, None, cw.scale, cw.zero_point)
        assert torch.equal(again.tensor, cw.tensor)
    else:
        again = wl.do_float_quantization(dq, cfg, None, cw.scale)
        assert torch.equal(again.tensor, cw.tensor)
    assert cw.scale.shape == (14336, 4096 // gs if gs != -1 else 1, 1)[: cw.scale.ndim] or gs == -1


@pytest.mark.parametrize("mode,gs", [("int4_sym", 128), ("int4_asym", 128), ("int4_sym", 64), ("int4_asym", 32),
                                     ("int8_asym", -1), ("int8_sym", -1), ("int8_sym", 128), ("int4_sym", -1),
                                     ("nf4", 128), ("nf4", 32), ("mxfp4", 32), ("fp4", 64), ("fp4", 128)])
@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
def test_batched_plan_matches_oracle(mode, gs, dtype):
    """One launch over a list of ragged tensors (the whole-model path) equals the oracle per tensor,
    and a CUDA-graph replay equals the direct launch."""
    from oracle import wc_oracle as O

    from nncf_b200.pipeline import CompressionPlan

    cols = 1024 if gs != -1 else 4096
    shapes = [(7, cols), (1, cols), (33, cols), (130, cols), (2, cols)]
    if gs == -1:
        shapes += [(3, 14336), (5, 4096)]  # a different row length starts a new launch
    gen = torch.Generator().manual_seed(11)
    ws = [(torch.randn(*s, generator=gen) * 0.02).to(TORCH_DTYPE[dtype]) for s in shapes]
    ws[1][0, :128] = 0.0          # an all-zero group: eps guard
    ws[2][3, 5] = 3.0e-9          # tiny values
    cfg = _cfg(mode, gs)
    plan = CompressionPlan([(f"w{i}", w.cuda(), cfg) for i, w in enumerate(ws)])
    plan.run(use_graph=False)
    torch.cuda.synchronize()
    first = [(it.packed.clone(), it.scale.clone(), None if it.zero_point is None else it.zero_point.clone())
             for it in plan.items]
    for w, it in zip(ws, plan.items):
        w_np = w.numpy() if dtype == "f16" else w.float().numpy()
        ref = O.compress_weight(w_np, 1, mode, gs)
        _eq(it.scale, ref.scale.reshape(-1), "scale")
        if cfg.is_asym_mode:
            _eq(it.zero_point, ref.zero_point.reshape(-1), "zp")
        if not cfg.is_integer:
            codes = O.nibble_code_nf4(ref.tensor) if mode == "nf4" else O.nibble_code_e2m1(ref.tensor)
            _eq(it.packed, O.pack_uint4(codes).reshape(-1), "packed float codes")
            if mode == "mxfp4":
                _eq(it.scale_e8m0, O.e8m0_code(ref.scale).reshape(-1), "e8m0")
        elif cfg.num_bits == 4:
            ref_packed = O.pack_int4(ref.tensor) if mode == "int4_sym" else O.pack_uint4(ref.tensor)
            _eq(it.packed, ref_packed.reshape(-1), "packed")
        else:
            _eq(it.packed, ref.tensor.reshape(-1), "codes")
    for it in plan.items:
        it.packed.zero_()
        it.scale.zero_()
    plan.run(use_graph=True)
    torch.cuda.synchronize()
    for it, (p, s, z) in zip(plan.items, first):
        assert torch.equal(it.packed, p) and torch.equal(it.scale, s)
        if z is not None:
            assert torch.equal(it.zero_point, z)


def test_extreme_scales_take_the_ieee_division_path():
    """Groups whose scale lies outside the exponent window of the multiply/FMA division must give
    the same codes as the oracle (they are routed to the plain IEEE division)."""
    from oracle import wc_oracle as O

    from nncf_b200.pipeline import CompressionPlan

    gen = torch.Generator().manual_seed(5)
    w = torch.randn(8, 1024, generator=gen)
    w[0] *= 1e-30
    w[1] *= 1e30
    w[2] *= 1e-20
    w[3] *= 3e15
    for mode in ("int4_sym", "int4_asym", "int8_asym"):
        cfg = _cfg(mode, 128)
        plan = CompressionPlan([("w", w.cuda(), cfg)])
        plan.run(use_graph=False)
        ref = O.compress_weight(w.numpy(), 1, mode, 128)
        _eq(plan.items[0].scale, ref.scale.reshape(-1), "scale")
        if mode == "int8_asym":
            _eq(plan.items[0].packed, ref.tensor.reshape(-1), "codes")
        else:
            ref_packed = O.pack_int4(ref.tensor) if mode == "int4_sym" else O.pack_uint4(ref.tensor)
            _eq(plan.items[0].packed, ref_packed.reshape(-1), "packed")


@pytest.mark.parametrize("mode", ["nf4", "fp4", "mxfp4"])
def test_float_codes_at_and_next_to_every_decision_boundary(mode):
    """Every decision boundary of the code book, the floats just below and above it, and the bucket edges
    of the in-kernel lookup, with a group scale of exactly one, through the batched (storage) path."""
    from oracle import wc_oracle as O

    from nncf_b200.pipeline import CompressionPlan

    if mode == "nf4":
        bounds, top = O.NF4_BOUNDS, 1.0
        edges = (np.arange(0, 33) - 16.5) / np.float32(15.49)
    else:
        bounds, top = O.E2M1_BOUNDS, 6.0
        edges = np.concatenate([(np.arange(0, 26) - 0.5) / 4.0, -(np.arange(0, 26) - 0.5) / 4.0])
    pts = np.concatenate([bounds, np.nextafter(bounds, np.float32(9)), np.nextafter(bounds, np.float32(-9)),
                          edges.astype(np.float32), np.nextafter(edges.astype(np.float32), np.float32(9)),
                          np.float32([0.0, -0.0, top, -top, 1e-30, -1e-30])]).astype(np.float32)
    pts = pts[np.abs(pts) <= top]
    gs = 32 if mode == "mxfp4" else 128
    rows = []
    for i in range(0, len(pts), gs - 1):      # every group carries the value `top` so that its scale is one
        chunk = pts[i:i + gs - 1]
        rows.append(np.concatenate([chunk, np.full(gs - len(chunk), top, np.float32)]))
    w = np.stack(rows)
    ref = O.compress_weight(w, 1, mode, gs)
    assert np.all(ref.scale == 1.0)
    plan = CompressionPlan([("w", torch.from_numpy(w).cuda(), _cfg(mode, gs))])
    plan.run(use_graph=False)
    codes = O.nibble_code_nf4(ref.tensor) if mode == "nf4" else O.nibble_code_e2m1(ref.tensor)
    _eq(plan.items[0].packed, O.pack_uint4(codes).reshape(-1), "packed")


def test_random_shapes_modes_and_dtypes_match_oracle():
    """Seeded fuzz over shapes (ragged rows, group sizes that hit every kernel variant, odd sizes), modes,
    dtypes and value distributions: reference-shaped outputs and the stored (packed) form against the oracle."""
    from oracle import wc_oracle as O

    from nncf_b200 import weight_lowering as wl

    rng = np.random.default_rng(2024)
    group_sizes = [8, 16, 24, 32, 40, 64, 128, 256, 384, 512, 1024, -1]
    for case in range(160):
        mode = MODES[rng.integers(len(MODES))]
        dtype = ["f32", "f16", "bf16"][rng.integers(3)]
        gs = group_sizes[rng.integers(len(group_sizes))]
        rows = int(rng.integers(1, 70))
        groups = int(rng.integers(1, 6)) if gs != -1 else 1
        cols = gs * groups if gs != -1 else int(rng.integers(1, 300)) * 8 + (int(rng.integers(0, 8)) if rng.random() < 0.3 else 0)
        kind = rng.integers(4)
        if kind == 0:
            w = rng.normal(0, 0.02, (rows, cols))
        elif kind == 1:
            w = rng.uniform(-3, 3, (rows, cols))
        elif kind == 2:
            w = rng.normal(0, 1, (rows, cols)) * (rng.random((rows, 1)) < 0.7)   # some all-zero rows
        else:
            w = np.abs(rng.normal(0, 5e-3, (rows, cols))) + 1e-3                 # one-signed
        wt = torch.from_numpy(w.astype(np.float32)).to(TORCH_DTYPE[dtype])
        w_np = wt.numpy() if dtype == "f16" else wt.float().numpy()
        ref = O.compress_weight(w_np, 1, mode, gs)
        cfg = _cfg(mode, gs)
        tag = f"case {case}: {mode} {dtype} {rows}x{cols} g{gs}"
        cw = wl.compress_weight(wt.cuda(), 1, cfg)
        _eq(cw.scale, ref.scale, tag + " scale")
        got_t, ref_t = cw.tensor.cpu().numpy(), ref.tensor
        assert np.array_equal(got_t, ref_t, equal_nan=True), tag + " tensor"
        if cfg.is_asym_mode:
            _eq(cw.zero_point, ref.zero_point, tag + " zp")
        if (rows * cols) % 2 == 0 or cfg.num_bits == 8:
            st = wl.compress_weight(wt.cuda(), 1, cfg, pack=True)
            if cfg.is_integer and cfg.num_bits == 4:
                exp = O.pack_int4(ref.tensor) if mode == "int4_sym" else O.pack_uint4(ref.tensor)
                _eq(st.packed, exp, tag + " packed")
            elif cfg.is_integer:
                _eq(st.packed, ref.tensor, tag + " codes")
            elif cfg.num_bits == 4:
                codes = O.nibble_code_nf4(ref.tensor) if mode == "nf4" else O.nibble_code_e2m1(ref.tensor)
                _eq(st.packed, O.pack_uint4(codes), tag + " packed float codes")


@pytest.mark.parametrize("mode", ["int8_asym", "int8_sym", "int4_sym", "int4_asym", "nf4", "fp8_e4m3"])
@pytest.mark.parametrize("shape,axes", [((24, 16, 3, 3), (1, 2, 3)),     # Conv2d [out, in, kh, kw]: channel axis 0
                                        ((16, 24, 3, 3), (0, 2, 3)),     # ConvTranspose2d [in, out, kh, kw]: channel axis 1
                                        ((8, 12, 5), (1, 2)),            # Conv1d
                                        ((6, 4, 2, 3, 3), (1, 2, 3, 4))])  # Conv3d
def test_convolution_weights_reduce_over_every_axis_but_the_channel(shape, axes, mode):
    """Several reduction axes at once (src/nncf/torch/model_graph_manager.py:374-380: all axes of a convolution
    weight except its output channel; per channel, i.e. the backup precision): codes, scale and zero point in
    the weight's own layout against the oracle with the same tuple of axes; group-wise quantisation over
    several axes is refused like in the reference."""
    from oracle import wc_oracle as O

    from nncf_b200 import weight_lowering as wl
    from nncf_b200.errors import UnsupportedModelError

    gen = torch.Generator().manual_seed(sum(shape) + len(mode))
    w = (torch.randn(*shape, generator=gen) * 0.05).to(torch.bfloat16)
    ref = O.compress_weight(w.float().numpy(), axes, mode, -1)
    cfg = _cfg(mode, -1)
    cw = wl.compress_weight(w.cuda(), axes, cfg)
    _eq(cw.tensor, ref.tensor, "tensor")
    _eq(cw.scale, ref.scale, "scale")
    if cfg.is_asym_mode:
        _eq(cw.zero_point, ref.zero_point, "zp")
    if cfg.is_integer:
        s, z = wl.calculate_integer_quantization_params(w.cuda(), axes, cfg)
        _eq(s, ref.scale, "params scale")
        dq = wl.integer_quantize_dequantize_weight(w.cuda(), cfg, axes)
        _eq(dq, O.do_integer_dequantization(ref), "dequantised")
        if cfg.num_bits == 8:
            st = wl.compress_weight(w.cuda(), axes, cfg, pack=True)
            _eq(st.packed, ref.tensor, "stored bytes")
            _eq(st.scale_f16, ref.scale.astype(np.float16), "fp16 scale")
    with pytest.raises(UnsupportedModelError):
        wl.compress_weight(w.cuda(), axes, _cfg(mode, 4))


@pytest.mark.parametrize("mode", ["int4_asym", "int8_asym"])
@pytest.mark.parametrize("shape,axis,gs", [((96, 4096), 1, 128), ((33, 1024), 1, 32), ((7, 192), 1, 64), ((5, 384), 1, 128),
                                           ((64, 2048), 1, -1), ((9, 1000), 1, 8), ((256, 48), 0, 32), ((3, 64, 20), 1, 16)])
def test_zero_points_leave_the_kernel_in_their_stored_form(shape, axis, gs, mode):
    """`zp_packed_out`: the decompressor's zero-point buffer written by the compression kernel itself - uint8 per
    group, or two 4-bit groups per byte in flat group order with the even group in the low nibble (pack_uint4 of
    the reference's zero-point tensor, layers.py:1390) - on the batched row kernel (even and odd numbers of
    groups, groups of 32 / 64 / 128), the per-channel kernel and the general kernels (atomic OR into zeroed words)."""
    from oracle import wc_oracle as O

    from nncf_b200 import weight_lowering as wl

    gen = torch.Generator().manual_seed(sum(shape) + len(mode))
    w = (torch.randn(*shape, generator=gen) * 0.05).to(torch.bfloat16)
    ref = O.compress_weight(w.float().numpy(), axis, mode, gs)
    zp = ref.zero_point.reshape(-1).astype(np.uint8)
    if mode == "int4_asym":
        padded = np.concatenate([zp, np.zeros(len(zp) % 2, dtype=np.uint8)])
        want = O.pack_uint4(padded).reshape(-1)
    else:
        want = zp
    st = wl.compress_weight(w.cuda(), axis, _cfg(mode, gs), pack=True)
    got = st.zero_point_packed.cpu().numpy().reshape(-1)
    assert got.dtype == np.uint8
    np.testing.assert_array_equal(got[: len(want)], want)
    _eq(st.zero_point, ref.zero_point, "int32 zero point still written")


def test_plan_with_packed_zero_points_matches_oracle_and_installs_decompressors():
    """CompressionPlan(packed_zero_points=True) on the batched kernels (INT4_ASYM g128 incl. an odd number of
    groups per tensor, INT8_ASYM per channel), and the model-level call, which installs the kernel-written buffers
    without the torch-side pack: state dict equal to the reference's golden (api case int4_asym_g16_all)."""
    from oracle import wc_oracle as O

    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig
    from nncf_b200.pipeline import CompressionPlan

    gen = torch.Generator(device="cuda").manual_seed(4)
    items = []
    for k, (shape, mode, gs) in enumerate([((512, 4096), "int4_asym", 128), ((3, 384), "int4_asym", 128),
                                           ((1024, 1024), "int8_asym", -1), ((640, 4096), "int4_asym", 32)]):
        w = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
        w.normal_(0.0, 0.02, generator=gen)
        items.append((f"t{k}", w, WeightCompressionConfig(CompressWeightsMode(mode), gs)))
    plan = CompressionPlan(items, packed_zero_points=True)
    plan.run(use_graph=False)
    torch.cuda.synchronize()
    for (name, w, cfg), it in zip(items, plan.items):
        ref = O.stored_form(w.float().cpu().numpy(), cfg.mode.value, cfg.group_size)
        zp = ref["zero_point"].astype(np.uint8)
        want = O.pack_uint4(np.concatenate([zp, np.zeros(len(zp) % 2, dtype=np.uint8)])).reshape(-1) if cfg.num_bits == 4 else zp
        got = it.zero_point_packed.cpu().numpy()
        np.testing.assert_array_equal(got[: len(want)], want, err_msg=name)
        np.testing.assert_array_equal(it.packed.cpu().numpy().reshape(-1).view(np.uint8), ref["packed"], err_msg=name)
        assert it.zero_point is None
