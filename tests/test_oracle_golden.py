"""Pins the CPU oracle to the reference: golden fixtures produced by the reference itself
(tests/golden/make_golden.py) and the known-answer vectors of the reference's own tests,
transcribed as numbers (tests/openvino/native/quantization/test_weights_compression.py
:700-785, :1489-1617, :1646-1688, :2210-2337; tests/torch/function_hook/quantization/
test_weights_compression.py:557-572)."""

import numpy as np
import pytest
from conftest import golden

from oracle import wc_oracle as O


def _as_dtype(w32: np.ndarray, dtype: str) -> np.ndarray:
    # bf16 has no numpy type; bf16 fixtures hold bf16-representable fp32 values and the
    # reference widens to fp32 before any arithmetic, so fp32 input is equivalent.
    return w32.astype(np.float16) if dtype == "f16" else w32


def _quant_keys():
    return golden("quant").index("q")


@pytest.mark.parametrize("key", _quant_keys())
def test_compress_weight_matches_reference(key):
    g = golden("quant")
    _, name, dtype, mode = key.split("/")
    w = _as_dtype(g[f"q/{name}/{dtype}/w"], dtype)
    axis, gs = (int(v) for v in g[key + "/meta"])
    cw = O.compress_weight(w, axis, mode, gs)
    np.testing.assert_array_equal(cw.scale, g[key + "/scale"])
    ref_t = g[key + "/tensor"]
    assert cw.tensor.shape == ref_t.shape and cw.tensor.dtype == ref_t.dtype
    np.testing.assert_array_equal(cw.tensor, ref_t)
    if O.is_asym(mode):
        np.testing.assert_array_equal(cw.zero_point, g[key + "/zp"])
        assert cw.zero_point.dtype == np.int32
    if O.is_integer(mode):
        dq, _ = O.integer_quantize_dequantize(w, mode, gs, axis)
    else:
        dq, _ = O.float_quantize_dequantize(w, mode, gs, axis)
    np.testing.assert_array_equal(dq, g[key + "/dq"])
    if (key + "/err_max_mean") in g:
        for red in ("max_mean", "frobenius"):
            ref = float(g[key + f"/err_{red}"])
            got = O.integer_quantization_error(w, axis, mode, gs, red)
            assert got == pytest.approx(ref, rel=1e-4, abs=1e-9)


@pytest.mark.parametrize("key", golden("quant").index("pre"))
def test_precomputed_parameters_match_reference(key):
    g = golden("quant")
    mode = key.split("/")[1]
    w = g[key + "/w"]
    s = g[key + "/scale"]
    zp = g[key + "/zp"] if (key + "/zp") in g else None
    cw = O.compress_weight(w, 1, mode, 32, s, zp)
    np.testing.assert_array_equal(cw.tensor, g[key + "/tensor"])


def test_pack_and_decompress_match_reference():
    g = golden("pack")
    np.testing.assert_array_equal(O.pack_uint4(g["pack/u4_in"]), g["pack/u4_out"])
    np.testing.assert_array_equal(O.pack_int4(g["pack/i4_in"]), g["pack/i4_out"])
    assert g["pack/u4_out"].shape == (g["pack/u4_in"].size // 2, 1)
    np.testing.assert_array_equal(O.unpack_uint4(g["pack/u4_out"]).reshape(g["pack/u4_in"].shape), g["pack/u4_in"])
    np.testing.assert_array_equal(O.unpack_int4(g["pack/i4_out"]).reshape(g["pack/i4_in"].shape), g["pack/i4_in"])
    np.testing.assert_array_equal(
        O.decompress_asymmetric(g["pack/u4_in"], g["pack/scale_f16"], g["pack/zp"]), g["pack/dq_asym_f16"])
    np.testing.assert_array_equal(O.decompress_symmetric(g["pack/i4_in"], g["pack/scale_f16"]), g["pack/dq_sym_f16"])
    np.testing.assert_array_equal(
        O.decompress_asymmetric(g["pack/u8_in"], g["pack/scale8_f16"], g["pack/zp8"]), g["pack/dq8_asym_f16"])
    np.testing.assert_array_equal(O.decompress_symmetric(g["pack/i8_in"], g["pack/scale8_f16"]), g["pack/dq8_sym_f16"])


def test_pack_round_trip_random():
    rng = np.random.default_rng(0)
    u = rng.integers(0, 16, size=(33, 6), dtype=np.uint8)
    np.testing.assert_array_equal(O.unpack_uint4(O.pack_uint4(u)).reshape(u.shape), u)
    i = rng.integers(-8, 8, size=(10, 8), dtype=np.int8)
    np.testing.assert_array_equal(O.unpack_int4(O.pack_int4(i)).reshape(i.shape), i)


@pytest.mark.parametrize("subset", [3, 4, 10, 32])
def test_process_stats_matches_reference(subset):
    g = golden("stats")
    means = list(g["stats/process/means"])
    shapes = [tuple(int(v) for v in s) for s in g["stats/process/shapes"]]
    s, X = O.process_stats(means, shapes, subset)
    np.testing.assert_array_equal(s, g[f"stats/process/{subset}/s"])
    np.testing.assert_array_equal(X, g[f"stats/process/{subset}/X"])


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_reducers_match_reference(dtype):
    g = golden("stats")
    key = f"stats/reduce/{dtype}"
    x = g[key + "/x"]
    ref_mean = g[key + "/mean"].reshape(-1)
    got = O.mean_reducer(x).astype(np.float32)
    # the reference rounds the mean to the activation dtype; fp32 sums differ in order only
    tol = {"f32": 2e-6, "f16": 1e-3, "bf16": 8e-3}[dtype]
    np.testing.assert_allclose(got, ref_mean, rtol=tol, atol=tol * 1e-1)
    mv, xv = O.variance_reducers(x, (0, 1))
    n = x.shape[0] * x.shape[1]
    # torch's fns.var is the unbiased estimator by default only when asked; the reference calls
    # torch.var(..., correction=0)
    assert mv == pytest.approx(float(g[key + "/mean_var"]), rel=2e-2)
    assert xv == pytest.approx(float(g[key + "/max_var"]), rel=2e-2)
    assert O.mean_abs_max_reducer(x, (0, 1)) == pytest.approx(float(g[key + "/mean_abs_max"]), rel=1e-2)
    assert n > 1


@pytest.mark.parametrize("key", golden("scale_estimation").index("se"))
def test_scale_estimation_matches_reference(key):
    from cases import SE_CASES

    g = golden("scale_estimation")
    name = key.split("/")[1]
    _, o, i, gs, n, mode, ist, sst, axis, pen = next(c for c in SE_CASES if c[0] == name)
    means = list(g[key + "/means"])
    s, X = O.process_stats(means, [(1, 16, i)] * n, 32)
    scale, zp = O.scale_estimation(s, X, g[key + "/w"], axis, mode, gs, ist, sst, pen)
    ref = g[key + "/scale"]
    assert scale.shape == ref.shape
    # torch and numpy sum in different orders; a candidate whose score is a near-tie may flip.
    rel = np.abs(scale - ref) / np.abs(ref)
    assert np.mean(rel > 1e-5) <= 0.02, f"{np.mean(rel > 1e-5):.3f} of scales differ"
    if zp is not None:
        np.testing.assert_array_equal(zp, g[key + "/zp"])


@pytest.mark.parametrize("key", golden("awq").index("awq"))
def test_awq_matches_reference(key):
    g = golden("awq")
    gs, steps = (int(v) for v in g[key + "/meta"])
    mode = str(g[key + "/mode"])
    means = list(g[key + "/means"])
    w = g[key + "/w"]
    i = w.shape[1]
    s, X = O.process_stats(means, [(1, 16, i)] * len(means), 32)
    prev_w = prev_s = None
    if (key + "/prev_w") in g:
        prev_w = g[key + "/prev_w"]
        pm = list(g[key + "/prev_means"])
        ps, _ = O.process_stats(pm, [(1, 16, prev_w.shape[1])] * len(pm), 32)
        prev_s = float(ps.max())
    scale = O.awq_data_aware_scale(s, X, w, 1, mode, gs, float(g[key + "/pct"]), 0.0, 1.0, steps, prev_w, prev_s)
    np.testing.assert_allclose(scale, g[key + "/scale"], rtol=1e-5)


def test_awq_data_free_matches_reference():
    g = golden("awq")
    np.testing.assert_allclose(O.awq_data_free_scale(g["awq/data_free/w"], 0), g["awq/data_free/scale"], rtol=1e-6)


@pytest.mark.parametrize("key", golden("gptq").index("gptq"))
def test_gptq_matches_reference(key):
    g = golden("gptq")
    gs, block = (int(v) for v in g[key + "/meta"])
    mode = str(g[key + "/mode"])
    xs = list(g[key + "/x"])
    H = O.gptq_hessian(xs)
    Href = g[key + "/H"]
    np.testing.assert_allclose(H, Href, rtol=2e-5, atol=2e-5 * np.abs(Href).max())
    # sweep from the reference's own Hessian so that only the sweep is compared
    w = g[key + "/w"].copy()
    hinv = O.gptq_hinv(Href.copy(), w, float(g[key + "/damp"]))
    Q, S, Z = O.gptq_quantize(w, hinv, mode, gs, block)
    qref = g[key + "/q"]
    assert S.shape == g[key + "/scale"].shape
    # GPTQ amplifies last-bit differences of the trailing matmuls into flipped codes (the
    # reference's own torch and numpy backends differ by 3.5e-3 relative Frobenius on a
    # 512x1024 problem).  On these small problems one flipped code already costs ~1e-2 in
    # relative Frobenius norm, so the flipped fraction is the meaningful measure.
    flipped = np.mean(np.abs(Q - qref) > 1e-6)
    assert flipped < 0.01, flipped
    np.testing.assert_allclose(S, g[key + "/scale"], rtol=1e-4)
    if Z is not None:
        assert Z.shape == g[key + "/zp"].shape


@pytest.mark.parametrize("mode", ["int4_sym", "int4_asym"])
def test_gptq_512x1024_sweep_equals_reference_torch_backend(mode):
    """The oracle's blocked sweep (WC/gptq.py:297-379 restated) on a 512 x 1024 problem, given the upper factor
    the reference's torch backend computed: the dequantised weights, scales and zero points equal the
    reference's bit for bit, and the oracle's Hessian equals the reference's.  With the oracle's own factor
    (LAPACK through scipy, 5e-6 relative away from torch's) a few codes flip: reported, bounded."""
    from cases import GPTQ_LARGE, gptq_large_inputs

    g = golden("gptq_large")
    c = GPTQ_LARGE
    w, xs = gptq_large_inputs()
    iu = np.triu_indices(c["cols"])
    H = np.zeros((c["cols"], c["cols"]), dtype=np.float32)
    H[iu] = g["gptq_large/H_triu"]
    H = H + np.triu(H, 1).T
    U = np.zeros_like(H)
    U[iu] = g["gptq_large/U_triu"]
    key = f"gptq_large/{mode}"
    scale = g[key + "/scale"]
    sg = np.repeat(scale.reshape(c["rows"], -1), c["group_size"], axis=1)
    zg = np.float32(0)
    if (key + "/zp") in g:
        zg = np.repeat(g[key + "/zp"].reshape(c["rows"], -1), c["group_size"], axis=1).astype(np.float32)
    q_ref = ((g[key + "/codes"].astype(np.float32) - zg) * sg).astype(np.float32)
    assert np.array_equal(O.gptq_hessian(xs), H)
    Q, S, Z = O.gptq_quantize(w.copy(), U.copy(), mode, c["group_size"], c["block"])
    assert np.array_equal(Q, q_ref)
    assert np.array_equal(S.reshape(scale.shape), scale)
    if Z is not None:
        assert np.array_equal(Z.reshape(scale.shape), g[key + "/zp"])
    hinv = O.gptq_hinv(H.copy(), w.copy(), c["damp"])
    Q2, _, _ = O.gptq_quantize(w.copy(), hinv, mode, c["group_size"], c["block"])
    rel = np.linalg.norm(Q2 - q_ref) / np.linalg.norm(q_ref)
    assert rel < 5e-3, rel


def _gptq_se_stats(g, key):
    """(s, X) of a GPTQ(scale_estimation=True) fixture: per-input channel means in the activation dtype
    (WC/gptq.py:382-396), then process_stats with the default subset of 32."""
    import torch

    xs = list(g[key + "/x"])
    means = []
    for x in xs:
        m = O.mean_reducer(x, -1)
        if str(g[key + "/xdtype"]) == "bf16":
            m = torch.from_numpy(m).to(torch.bfloat16).float().numpy()
        means.append(m)
    return O.process_stats(means, [x.shape for x in xs], 32)


@pytest.mark.parametrize("key", golden("gptq_se").index("gptq_se"))
def test_gptq_with_scale_estimation_matches_reference(key):
    g = golden("gptq_se")
    gs, block = (int(v) for v in g[key + "/meta"])
    mode = str(g[key + "/mode"])
    s, X = _gptq_se_stats(g, key)
    w = g[key + "/w"].copy()
    hinv = O.gptq_hinv(g[key + "/H"].copy(), w, float(g[key + "/damp"]))
    Q, S, Z = O.gptq_quantize(w, hinv, mode, gs, block, se_stats=(s.astype(np.float32), X.astype(np.float32)))
    qref, sref = g[key + "/q"], g[key + "/scale"]
    assert S.shape == sref.shape
    flipped = np.mean(np.abs(Q - qref) > 1e-6)
    assert flipped < 0.02, flipped
    # the refined scales differ from the min/max ones (otherwise this fixture would not test anything) ...
    w0 = g[key + "/w"].reshape(w.shape[0], -1, gs)
    plain = np.abs(w0).max(-1) / 8.0 if mode == "int4_sym" else (w0.max(-1) - w0.min(-1)) / 15.0
    assert np.mean(np.abs(np.abs(sref[..., 0]) - plain) > 1e-3 * plain) > 0.3
    # ... and the oracle reproduces them
    assert np.mean(np.abs(S - sref) > 2e-3 * np.abs(sref)) < 0.03
    if Z is not None:
        assert Z.shape == g[key + "/zp"].shape
        assert np.mean(Z != g[key + "/zp"]) < 0.05


# ------------------------------------------------------------------------------------
# Known-answer vectors of the reference's own tests (numbers only)
# ------------------------------------------------------------------------------------
_LIN = np.arange(0, 256, 17, dtype=np.float32)
_TWO_ROWS = np.vstack((_LIN * 1.2, _LIN * 3.4))
_L4A = np.arange(0, 16, dtype=np.float32)
_TWO_ROWS_4A = np.vstack((_L4A * 1.2, _L4A * 3.4))
_L4S = np.arange(-8, 7, dtype=np.float32)
_TWO_ROWS_4S = np.vstack((_L4S * 1.2, _L4S * 3.4))
_TWO_GROUPS_S = np.hstack((_TWO_ROWS_4S, np.vstack((_L4S * 5.6, _L4S * 7.8))))
_TWO_GROUPS_A = np.hstack((_TWO_ROWS_4A, np.vstack((_L4A * 5.6, _L4A * 7.8))))

ERROR_KATS = [
    (_TWO_ROWS, O.INT8_ASYM, -1, 0.0, 1e-8),
    (_TWO_ROWS_4S, O.INT4_SYM, -1, 0.0, 1e-8),
    (_TWO_ROWS_4A, O.INT4_ASYM, -1, 0.0, 1e-8),
    (_TWO_GROUPS_S, O.INT4_SYM, 15, 0.0, 1e-8),
    (_TWO_GROUPS_A, O.INT4_ASYM, 16, 0.0, 1e-8),
    (_TWO_ROWS[:, 1:-1], O.INT8_ASYM, -1, 239, 1),
    (_TWO_ROWS.T, O.INT8_ASYM, -1, 46818, 1),
    (_TWO_ROWS_4A, O.INT4_SYM, -1, 4.12, 1),
    (_TWO_ROWS_4A.T, O.INT4_SYM, -1, 0.63, 1),
    (_TWO_ROWS_4A[:, 1:-1], O.INT4_ASYM, -1, 1.49, 1),
    (_TWO_ROWS_4A.T, O.INT4_ASYM, -1, 162, 1),
]


@pytest.mark.parametrize("w,mode,gs,ref,atol", ERROR_KATS)
def test_quantization_error_kats(w, mode, gs, ref, atol):
    assert O.integer_quantization_error(np.ascontiguousarray(w, dtype=np.float32), 1, mode, gs) == pytest.approx(
        ref, abs=atol)


@pytest.mark.parametrize("data", [list(range(-8, 1)), list(range(0, 9)), list(range(-8, 8))])
def test_int4_sym_range_identity(data):
    w = np.array(data, dtype=np.float32)
    cw = O.do_integer_quantization(w, O.INT4_SYM, -1, -1)
    np.testing.assert_allclose(np.abs(cw.tensor), np.abs(w))


_FP4 = {
    "neg": [-8.0, -8.0, -5.333333492279053, -5.333333492279053, -4.0, -2.6666667461395264, -2.0,
            -1.3333333730697632, -0.0],
    "pos": [-0.0, 1.3333333730697632, 2.0, 2.6666667461395264, 4.0, 5.333333492279053, 5.333333492279053, 8.0, 8.0],
}
_FP4["neg-pos"] = _FP4["neg"] + [1.3333333730697632, 2.0, 2.6666667461395264, 4.0, 5.333333492279053,
                                 5.333333492279053, 8.0]
_MX4 = {
    "neg": [-8.0, -8.0, -6.0, -4.0, -4.0, -3.0, -2.0, -1.0, -0.0],
    "pos": [-0.0, 1.0, 2.0, 3.0, 4.0, 4.0, 6.0, 8.0, 8.0],
}
_MX4["neg-pos"] = _MX4["neg"] + [1.0, 2.0, 3.0, 4.0, 4.0, 6.0, 8.0]
_F8 = {
    "neg": [-8.0, -6.857143402099609, -5.714285850524902, -5.142857551574707, -4.0, -2.857142925262451, -2.0, -1.0,
            0.0],
    "pos": [0.0, 1.0, 2.0, 2.857142925262451, 4.0, 5.142857551574707, 5.714285850524902, 6.857143402099609, 8.0],
}
_F8["neg-pos"] = _F8["neg"] + _F8["pos"][1:-1]
_DATA = {"neg": list(range(-8, 1)), "pos": list(range(0, 9)), "neg-pos": list(range(-8, 8))}


@pytest.mark.parametrize("ident", ["neg", "pos", "neg-pos"])
@pytest.mark.parametrize("mode,refs", [(O.FP4, _FP4), (O.MXFP4, _MX4), (O.FP8_E4M3, _F8), (O.MXFP8_E4M3, None)])
def test_float_range_kats(mode, refs, ident):
    w = np.array(_DATA[ident], dtype=np.float32)
    dq, _ = O.float_quantize_dequantize(w, mode, -1, -1)
    ref = np.array(refs[ident], dtype=np.float32) if refs is not None else w
    np.testing.assert_allclose(dq, ref)


def test_nf4_values_at_and_next_to_a_boundary():
    w = np.array([-0.07263] * 2, np.float16).astype(np.float32)
    s = np.array([0.08564102] * 2, np.float32)
    norm = w / s
    assert norm[0] == np.float32(-0.8480964)
    # one bit above the first boundary (-0.84809643): the second level, as the reference returns
    np.testing.assert_array_equal(O.float_quantized_values(norm, O.NF4), O.NF4_LEVELS[[1, 1]])
    # a value exactly on a boundary goes to the lower level (reference: [-1, 0] for these two)
    on_bound = O.NF4_BOUNDS[[0, 7]].copy()
    np.testing.assert_array_equal(O.float_quantized_values(on_bound, O.NF4), np.float32([-1.0, 0.0]))


@pytest.mark.parametrize("x,ref", [(-7.0, -6.0), (7.0, 6.0), (-5.0, -4.0), (-3.5, -4.0), (1.75, 2.0), (2.5, 2.0),
                                   (-4.0, -4.0), (0.0, 0.0), (-0.0, 0.0), (-0.25, 0.0), (0.25, 0.0), (-0.49, -0.5),
                                   (-0.51, -0.5), (0.75, 1.0), (1.25, 1.0), (3.5, 4.0), (5.0, 4.0)])
def test_e2m1_edge_kats(x, ref):
    assert O.float_quantized_values(np.float32([x]), O.FP4)[0] == ref


_E4M3_KATS = [
    (0.0, 0.0), (-0.0, 0.0), (0.0005, 0.0), (0.001, 0.001953125), (-0.001, -0.001953125), (0.003, 0.00390625),
    (0.006, 0.005859375), (-0.006, -0.005859375), (0.03125, 0.03125), (0.030, 0.029296875), (-0.030, -0.029296875),
    (0.0625, 0.0625), (0.0703125, 0.0703125), (0.078125, 0.078125), (0.109375, 0.109375), (0.125, 0.125),
    (0.25, 0.25), (0.26, 0.25), (0.28, 0.28125), (0.5, 0.5), (-0.5, -0.5), (1.0, 1.0), (-1.0, -1.0), (1.75, 1.75),
    (-1.75, -1.75), (2.0, 2.0), (3.0, 3.0), (4.0, 4.0), (5.0, 5.0), (6.0, 6.0), (7.0, 7.0), (8.0, 8.0), (-8.0, -8.0),
    (16.0, 16.0), (32.0, 32.0), (64.0, 64.0), (128.0, 128.0), (256.0, 256.0), (448.0, 448.0), (400.0, 384.0),
    (460.0, 448.0), (500.0, np.nan), (1e4, np.nan), (np.inf, np.nan), (-np.inf, np.nan), (np.nan, np.nan),
]


@pytest.mark.parametrize("x,ref", _E4M3_KATS)
def test_e4m3_edge_kats(x, ref):
    out = O.fp32_to_e4m3_values(np.float32([x]))[0]
    if np.isnan(ref):
        assert np.isnan(out)
    else:
        assert out == ref


def test_e4m3_all_fp16_inputs_match_reference_table():
    """Every fp16 bit pattern: the restated rounding rule equals a brute-force nearest-even
    search over the decode table."""
    h = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    bits = O.f16_bits_to_e4m3_bits(h)
    vals = h.view(np.float16).astype(np.float64)
    table = O.E4M3_TABLE[:127].astype(np.float64)
    mag = np.abs(vals)
    finite = np.isfinite(vals) & (mag >= 2.0 ** -14)  # fp16 normals only; subnormals -> 0
    idx = np.searchsorted(table, mag[finite])
    lo = np.clip(idx - 1, 0, 126)
    hi = np.clip(idx, 0, 126)
    dl, dh = mag[finite] - table[lo], table[hi] - mag[finite]
    pick = np.where((dh < dl) | ((dh == dl) & (hi % 2 == 0)), hi, lo)
    over = mag[finite] > 464.0
    expect = np.where(over, 0x7F, pick)
    np.testing.assert_array_equal(bits[finite] & 0x7F, expect)
    assert np.all((bits[~finite & ~np.isfinite(vals)] & 0x7F) == 0x7F)
    assert np.all((bits[np.isfinite(vals) & (mag < 2.0 ** -14)] & 0x7F) == 0)


def test_precomputed_asym_requires_both():
    w = ((np.arange(11) - 5) / 10).astype(np.float32)[:, None]
    s = -((np.arange(11) - 5) / 100).astype(np.float32)[:, None]
    z = np.arange(11).astype(np.int32)[:, None]
    for mode in (O.INT8_ASYM, O.INT4_ASYM):
        with pytest.raises(ValueError):
            O.do_integer_quantization(w, mode, -1, -1, s, None)
        with pytest.raises(ValueError):
            O.do_integer_quantization(w, mode, -1, -1, None, z)
        O.do_integer_quantization(w, mode, -1, -1, s, z)
    for mode in (O.INT8_SYM, O.INT4_SYM):
        assert O.do_integer_quantization(w, mode, -1, -1, s).zero_point is None


def test_invalid_group_size_raises():
    with pytest.raises(O.InvalidGroupSize):
        O.reshape_for_groups(np.zeros((4, 100), np.float32), 1, 32)
