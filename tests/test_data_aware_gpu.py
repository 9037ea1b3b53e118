"""GPU parity of the data-aware kernels (ScaleEstimation, AWQ, statistic reducers) against golden
outputs of the reference (tests/golden/make_golden.py) and the CPU oracle.

Tolerances: scales are fp32 results of sums evaluated in a different order than the reference's
BLAS / torch reductions, so they are compared with rtol 1e-5 and a small fraction of candidates
whose scores tie to the last bits may resolve differently (the reference's own torch and numpy
backends disagree on 55 % of the last bits and on such ties).  The end-to-end bar is the one of the
task: relative Frobenius error of the dequantised weight <= 1e-3 against the reference."""

import numpy as np
import pytest
import torch
from cases import AWQ_CASES, SE_CASES
from conftest import golden

pytestmark = pytest.mark.gpu


def _cfg(mode, gs):
    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig

    return WeightCompressionConfig(CompressWeightsMode(mode), gs)


def _stats(means, shape):
    from nncf_b200 import WCTensorStatistic

    return WCTensorStatistic([torch.from_numpy(m).cuda() for m in means], [shape] * len(means))


def _dq(w, mode, gs, axis, scale, zp):
    """Dequantised weight for given parameters, by the oracle."""
    from oracle import wc_oracle as O

    wg, ax = (O.reshape_for_groups(w, axis, gs) if gs != -1 else (w, axis))
    if O.is_integer(mode):
        dq, _ = O.integer_quantize_dequantize(wg, mode, scale=scale.reshape(_keep(wg.shape, ax)),
                                              zero_point=None if zp is None else zp.reshape(_keep(wg.shape, ax)))
    else:
        dq, _ = O.float_quantize_dequantize(wg, mode, scale=scale.reshape(_keep(wg.shape, ax)))
    return dq


def _keep(shape, axis):
    s = list(shape)
    s[axis] = 1
    return tuple(s)


@pytest.mark.parametrize("case", SE_CASES, ids=[c[0] for c in SE_CASES])
def test_scale_estimation_matches_reference_golden(case):
    from nncf_b200.scale_estimation import ScaleEstimation

    name, o, i, gs, n, mode, ist, sst, axis, pen = case
    g = golden("scale_estimation")
    key = f"se/{name}"
    w = g[key + "/w"]
    scale, zp = ScaleEstimation.calculate_quantization_params(
        _stats(list(g[key + "/means"]), (1, 16, i)), torch.from_numpy(w).cuda(), (axis,), _cfg(mode, gs), -1, 32, ist,
        sst, pen)
    ref = g[key + "/scale"]
    got = scale.cpu().numpy()
    assert got.shape == ref.shape
    rel = np.abs(got - ref) / np.abs(ref)
    assert np.mean(rel > 1e-5) <= 0.03, f"{np.mean(rel > 1e-5):.3f} of the scales differ"
    if zp is not None:
        refz = g[key + "/zp"]
        assert zp.dtype == torch.float32 and tuple(zp.shape) == refz.shape
        np.testing.assert_array_equal(zp.cpu().numpy(), refz)
    # end-to-end bar: dequantised weight within 1e-3 relative Frobenius of the reference's
    zpn = None if zp is None else zp.cpu().numpy()
    refzp = g[key + "/zp"] if zp is not None else None
    a = _dq(w, mode, gs, axis, got, zpn)
    b = _dq(w, mode, gs, axis, ref, refzp)
    assert np.linalg.norm(a - b) / np.linalg.norm(b) <= 1e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_scale_estimation_llama_sized_matches_oracle(dtype):
    """q_proj-like slice (256 x 4096, g128, 64 samples) in 16-bit weights against the CPU oracle."""
    from oracle import wc_oracle as O

    from nncf_b200.scale_estimation import ScaleEstimation

    gen = torch.Generator().manual_seed(7)
    w = (torch.randn(256, 4096, generator=gen) * 0.02).to(dtype)
    means = [(torch.randn(4096, generator=gen) * (1 + 19 * (torch.rand(4096, generator=gen) < 0.01))).float()
             for _ in range(64)]
    st = _stats([m.numpy() for m in means], (1, 512, 4096))
    for mode in ("int4_asym", "int4_sym"):
        scale, zp = ScaleEstimation.calculate_quantization_params(st, w.cuda(), (1,), _cfg(mode, 128), -1, 64, 5, 5)
        s, X = O.process_stats([m.numpy() for m in means], [(1, 512, 4096)] * 64, 64)
        ref_s, ref_z = O.scale_estimation(s, X, w.float().numpy(), 1, mode, 128, 5, 5)
        got = scale.cpu().numpy()
        rel = np.abs(got - ref_s) / np.abs(ref_s)
        assert np.mean(rel > 1e-5) <= 0.01
        a = _dq(w.float().numpy(), mode, 128, 1, got, None if zp is None else zp.cpu().numpy())
        b = _dq(w.float().numpy(), mode, 128, 1, ref_s, ref_z)
        assert np.linalg.norm(a - b) / np.linalg.norm(b) <= 1e-3


@pytest.mark.parametrize("rows,cols,gs,n", [(13, 256, 128, 64), (5, 512, 256, 40), (70, 256, 64, 70), (9, 256, 128, 150),
                                            (33, 128, 32, 1), (66, 1024, 512, 20)])
@pytest.mark.parametrize("mode", ["int4_asym", "int4_sym"])
def test_scale_estimation_row_and_sample_tilings_match_oracle(rows, cols, gs, n, mode):
    """Row counts that are not multiples of the four rows a warp handles together, group sizes on both sides of
    the 128 that the 4-row tiling takes, and sample counts that need one, two and four 64-sample accumulator
    chunks (each combination is a different instantiation of the kernel)."""
    from oracle import wc_oracle as O

    from nncf_b200.scale_estimation import ScaleEstimation

    gen = torch.Generator().manual_seed(rows + cols + n)
    w = (torch.randn(rows, cols, generator=gen) * 0.02).to(torch.bfloat16)
    means = [(torch.randn(cols, generator=gen) * (1 + 9 * (torch.rand(cols, generator=gen) < 0.03))).float() for _ in range(n)]
    st = _stats([m.numpy() for m in means], (1, 64, cols))
    scale, zp = ScaleEstimation.calculate_quantization_params(st, w.cuda(), (1,), _cfg(mode, gs), -1, 256, 5, 5)
    s, X = O.process_stats([m.numpy() for m in means], [(1, 64, cols)] * n, 256)
    ref_s, ref_z = O.scale_estimation(s, X, w.float().numpy(), 1, mode, gs, 5, 5)
    got = scale.cpu().numpy()
    assert got.shape == ref_s.shape
    rel = np.abs(got - ref_s) / np.abs(ref_s)
    assert np.mean(rel > 1e-5) <= 0.02, float(np.mean(rel > 1e-5))
    if ref_z is not None:
        np.testing.assert_array_equal(zp.cpu().numpy(), ref_z)


@pytest.mark.parametrize("n,gs", [(70, 128), (150, 64), (20, 256)])
def test_awq_sample_and_group_tilings_match_oracle(n, gs):
    """AWQ alpha search with sample counts / group sizes that take the 2-row and 1-row variants of the kernel."""
    from oracle import wc_oracle as O

    from nncf_b200.awq import AWQ, make_wp

    gen = torch.Generator().manual_seed(n + gs)
    out, hid = 37, 512
    w = (torch.randn(out, hid, generator=gen) * 0.05)
    means = [(torch.randn(hid, generator=gen) * (1 + 15 * (torch.arange(hid) % 97 == 3))).float() for _ in range(n)]
    st = _stats([m.numpy() for m in means], (1, 16, hid))
    algo = AWQ(subset_size=256, percent_to_apply=0.01, steps=25)
    got = algo._data_aware_step(make_wp(_cfg("int4_asym", gs)), w.cuda(), st, -1).cpu().numpy()
    s, X = O.process_stats([m.numpy() for m in means], [(1, 16, hid)] * n, 256)
    ref = O.awq_data_aware_scale(s, X, w.numpy(), 1, "int4_asym", gs, 0.01, 0.0, 1.0, 25)
    np.testing.assert_array_equal(got == 1.0, ref == 1.0)
    np.testing.assert_allclose(got, ref, rtol=2e-5)
    assert (ref != 1.0).any()


@pytest.mark.parametrize("case", AWQ_CASES, ids=[c[0] for c in AWQ_CASES])
def test_awq_matches_reference_golden(case):
    from nncf_b200.awq import AWQ, make_wp

    name, o, i, gs, n, mode, pct, steps, with_prev = case
    g = golden("awq")
    key = f"awq/{name}"
    algo = AWQ(subset_size=32, percent_to_apply=pct, steps=steps)
    prev_w = prev_stats = None
    if with_prev:
        pw = g[key + "/prev_w"]
        prev_w = torch.from_numpy(pw).cuda()
        prev_stats = _stats(list(g[key + "/prev_means"]), (1, 16, pw.shape[1]))
    scale = algo._data_aware_step(make_wp(_cfg(mode, gs)), torch.from_numpy(g[key + "/w"]).cuda(),
                                  _stats(list(g[key + "/means"]), (1, 16, i)), -1, prev_w, prev_stats)
    ref = g[key + "/scale"]
    got = scale.cpu().numpy()
    assert got.shape == ref.shape
    # the untouched channels are exactly one; searched groups agree unless two alphas tie
    np.testing.assert_array_equal(got == 1.0, ref == 1.0)
    np.testing.assert_allclose(got, ref, rtol=2e-5)


def test_awq_stacked_experts_equal_per_expert_searches():
    """A 3-D weight [E, out, in] with statistics [E, hidden] per sample: the reference searches every
    (expert, group) pair on its own (awq.py:276-300), so the stacked call must equal E separate 2-D calls, with
    the previous layer's activation maximum taken over all experts (awq.py:264-266)."""
    from nncf_b200.awq import AWQ, make_wp
    from nncf_b200.config import WCTensorStatistic

    gen = torch.Generator().manual_seed(17)
    E, out, hid, n = 3, 48, 256, 12
    w = (torch.randn(E, out, hid, generator=gen) * 0.05).cuda()
    means = [torch.randn(E, hid, generator=gen).cuda() * (1 + 5 * (torch.arange(hid) % 37 == 0)).cuda() for _ in range(n)]
    stats = WCTensorStatistic(means, [(E, 16, hid)] * n)
    prev_w = (torch.randn(E, hid, 64, generator=gen) * 0.05).cuda()   # [E, out_prev = hid, in_prev]
    prev_means = [torch.randn(E, 64, generator=gen).cuda() * (e + 1) for e in range(n)]
    prev_stats = WCTensorStatistic(prev_means, [(E, 16, 64)] * n)
    algo = AWQ(subset_size=32, percent_to_apply=0.02, steps=20)
    cfg = _cfg("int4_asym", 64)
    got = algo._data_aware_step(make_wp(cfg, (2,)), w, stats, -1, prev_w, prev_stats)
    assert tuple(got.shape) == (E, hid)
    prev_s = float(torch.stack(prev_means).abs().amax().item())
    for e in range(E):
        st = WCTensorStatistic([m[e] for m in means], [(16, hid)] * n)
        pst = WCTensorStatistic([m[e] for m in prev_means], [(16, 64)] * n)
        one = algo._data_aware_step(make_wp(cfg, (1,)), w[e], st, -1, prev_w[e], pst, prev_s)
        assert torch.equal(one, got[e])
        assert (one != 1).any()


def test_awq_data_free_matches_reference_golden():
    from nncf_b200.awq import AWQ

    g = golden("awq")
    got = AWQ()._data_free_step(torch.from_numpy(g["awq/data_free/w"]).cuda(), axis=0)
    np.testing.assert_allclose(got.cpu().numpy(), g["awq/data_free/scale"], rtol=1e-6)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_channel_stats_match_reference_golden(dtype):
    from nncf_b200.activation_stats import MeanReducer, channel_stats

    g = golden("stats")
    key = f"stats/reduce/{dtype}"
    td = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dtype]
    x = torch.from_numpy(g[key + "/x"]).cuda().to(td)
    mean = MeanReducer()._reduce_out_of_place([x])[0]
    assert mean.dtype == td and mean.shape == (48,)
    ref = g[key + "/mean"].reshape(-1)
    # one rounding to the activation dtype after an fp32-or-better sum: at most 1 ulp of that dtype apart
    tol = {"f32": 1e-6, "f16": 1e-3, "bf16": 8e-3}[dtype]
    np.testing.assert_allclose(mean.float().cpu().numpy(), ref, rtol=tol, atol=tol * 0.1)
    st = channel_stats(x, -1, ("var", "absmax", "sumsq"))
    assert float(st["var"].mean()) == pytest.approx(float(g[key + "/mean_var"]), rel=5e-3)
    assert float(st["var"].max()) == pytest.approx(float(g[key + "/max_var"]), rel=5e-3)
    # the reference averages the per-channel maxima in the activation's dtype
    assert float(st["absmax"].mean()) == pytest.approx(float(g[key + "/mean_abs_max"]), rel=max(tol, 1e-6))
    assert float(st["sumsq"].sum()) == pytest.approx(float(g[key + "/sumsq"]), rel=1e-9)


@pytest.mark.parametrize("subset", [3, 4, 10, 32])
def test_process_stats_matches_reference_golden(subset):
    from nncf_b200 import WCTensorStatistic
    from nncf_b200.activation_stats import process_stats

    g = golden("stats")
    means = [torch.from_numpy(m).cuda() for m in g["stats/process/means"]]
    shapes = [tuple(int(v) for v in s) for s in g["stats/process/shapes"]]
    s, X = process_stats(WCTensorStatistic(means, shapes), subset)
    np.testing.assert_array_equal(s.cpu().numpy(), g[f"stats/process/{subset}/s"])
    np.testing.assert_array_equal(X.cpu().numpy(), g[f"stats/process/{subset}/X"])
