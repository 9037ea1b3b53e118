"""LoRA correction against tests/golden/lora.npz: the reference's ``calculate_low_rank_matrices``
(src/nncf/quantization/algorithms/weight_compression/lora_correction.py:139-271) on seeded weights, the reference's
own compressed weights and seeded activation statistics.  The adapters themselves are unique only up to an
invertible R x R factor between them, so their product (the correction the layer adds) is compared, and the
activation-weighted noise they leave."""

import numpy as np
import pytest
import torch
from cases import LORA_CASES
from conftest import golden


def _inputs(g, key, hidden):
    from nncf_b200.config import WCTensorStatistic

    w = torch.from_numpy(g[key + "/w"])
    fq = torch.from_numpy(g[key + "/fq"])
    means = [torch.from_numpy(m) for m in g[key + "/means"]]
    shapes = [(1, int(t), hidden) for t in g[key + "/tokens"]]
    return w, fq, WCTensorStatistic(means, shapes)


@pytest.mark.parametrize("case", LORA_CASES, ids=[c[0] for c in LORA_CASES])
def test_adapters_match_reference_golden(case):
    import nncf_b200 as nb
    from nncf_b200.activation_stats import process_stats
    from nncf_b200.lora_correction import LoraCorrectionAlgorithm

    name, o, h, gs, n, mode, rank, iters, reg = case
    g = golden("lora")
    key = f"lora/{name}"
    w, fq, stats = _inputs(g, key, h)
    prm = nb.AdvancedLoraCorrectionParameters(adapter_rank=rank, num_iterations=iters, apply_regularization=reg)
    cfg = nb.WeightCompressionConfig(nb.CompressWeightsMode(mode), gs)
    a, b = LoraCorrectionAlgorithm.calculate_low_rank_matrices(w, fq, cfg, (1,), prm, stats)
    assert tuple(a.shape) == (rank, h) and tuple(b.shape) == (o, rank)
    want = torch.from_numpy(g[key + "/lora_B"]) @ torch.from_numpy(g[key + "/lora_A"])
    have = b @ a
    assert float((have - want).norm() / want.norm()) < 1e-4
    _, x = process_stats(stats, prm.subset_size)
    x = x.T.double()
    res = (w - fq).T.double()
    after = float((x @ res - x @ a.T.double() @ b.T.double()).abs().mean())
    assert after == pytest.approx(float(g[key + "/noise_after"]), rel=1e-3)
    assert after < 0.7 * float(g[key + "/noise_before"])


@pytest.mark.gpu
@pytest.mark.parametrize("case", LORA_CASES[:3], ids=[c[0] for c in LORA_CASES[:3]])
def test_adapters_on_the_gpu_from_the_library_dequantisation(case):
    """The same cases on the GPU, with the dequantised weight taken from the library's own compression (bit-exact
    with the reference's) instead of the stored one."""
    import nncf_b200 as nb
    from nncf_b200 import weight_lowering as wl
    from nncf_b200.lora_correction import LoraCorrectionAlgorithm

    name, o, h, gs, n, mode, rank, iters, reg = case
    g = golden("lora")
    key = f"lora/{name}"
    w, fq, stats = _inputs(g, key, h)
    cfg = nb.WeightCompressionConfig(nb.CompressWeightsMode(mode), gs)
    cw = wl.compress_weight(w.cuda(), 1, cfg)
    axis = 1 if gs != -1 else -1
    mine = (wl.do_float_dequantization(cw, axis) if mode == "nf4" else wl.do_integer_dequantization(cw, axis)).reshape(o, h)
    assert torch.equal(mine.cpu(), fq)
    stats.mean_values = [m.cuda() for m in stats.mean_values]
    prm = nb.AdvancedLoraCorrectionParameters(adapter_rank=rank, num_iterations=iters, apply_regularization=reg)
    a, b = LoraCorrectionAlgorithm.calculate_low_rank_matrices(w.cuda(), mine, cfg, (1,), prm, stats)
    want = torch.from_numpy(g[key + "/lora_B"]) @ torch.from_numpy(g[key + "/lora_A"])
    assert float(((b @ a).cpu() - want).norm() / want.norm()) < 1e-4


@pytest.mark.parametrize("case", LORA_CASES, ids=[c[0] for c in LORA_CASES])
def test_oracle_adapters_match_reference_golden(case):
    """The numpy restatement with the reference's dense routines (full SVD, least squares on the stacked systems)
    against the same goldens, and the package's small-system formulation against the restatement on a wider
    layer than the fixtures hold."""
    from oracle import wc_oracle as O

    name, o, h, gs, n, mode, rank, iters, reg = case
    g = golden("lora")
    key = f"lora/{name}"
    shapes = [(1, int(t), h) for t in g[key + "/tokens"]]
    a, b = O.lora_correction_adapters(g[key + "/w"], g[key + "/fq"], list(g[key + "/means"]), shapes, gs, rank, iters, reg)
    want = g[key + "/lora_B"].astype(np.float64) @ g[key + "/lora_A"].astype(np.float64)
    have = b.astype(np.float64) @ a.astype(np.float64)
    assert np.linalg.norm(have - want) / np.linalg.norm(want) < 1e-4


def test_small_system_formulation_equals_the_dense_one_on_a_wider_layer():
    import nncf_b200 as nb
    from nncf_b200.config import WCTensorStatistic
    from nncf_b200.lora_correction import LoraCorrectionAlgorithm
    from oracle import wc_oracle as O

    rng = np.random.default_rng(5)
    o, h, gs, n = 192, 512, 64, 48
    w = rng.normal(0, 0.05, size=(o, h)).astype(np.float32)
    dq, _ = O.integer_quantize_dequantize(w, "int4_asym", gs, 1)
    fq = np.asarray(dq, dtype=np.float32).reshape(o, h)
    means = [(rng.normal(0, 1.0, size=(h,)) * (1 + 9 * (rng.random(h) < 0.05))).astype(np.float32) for _ in range(n)]
    shapes = [(1, int(rng.integers(4, 40)), h) for _ in range(n)]
    a0, b0 = O.lora_correction_adapters(w, fq, means, shapes, gs)
    stats = WCTensorStatistic([torch.from_numpy(m) for m in means], shapes)
    a1, b1 = LoraCorrectionAlgorithm.calculate_low_rank_matrices(
        torch.from_numpy(w), torch.from_numpy(fq), nb.WeightCompressionConfig(nb.CompressWeightsMode.INT4_ASYM, gs), (1,),
        nb.AdvancedLoraCorrectionParameters(), stats)
    want = b0.astype(np.float64) @ a0.astype(np.float64)
    have = (b1.double() @ a1.double()).numpy()
    assert np.linalg.norm(have - want) / np.linalg.norm(want) < 1e-4
