"""CPU checks of numeric constants baked into the CUDA kernels (read from the sources, no GPU needed)."""
import re
from pathlib import Path

import numpy as np

from oracle import wc_oracle as O

CSRC = Path(__file__).resolve().parent.parent / "nncf_b200" / "csrc"


def _floats(text, name):
    m = re.search(name + r"\[32\]\s*=\s*\{(.*?)\};", text, re.S)
    body = m.group(1).replace("-kLutNone", "-3.0e38f").replace("kLutNone", "3.0e38f")
    return np.array([np.float32(x.strip().rstrip("f")) for x in body.split(",") if x.strip()], dtype=np.float32)


def test_nf4_bucket_polynomial_keeps_every_quotient_within_one_boundary():
    """The NF4 kernel computes k = rint(7 + q*(c1 + q*(c2 + q*c3))) and index = k + (q > bound[k]).  That is
    exact iff k is index-1 or index for every q in [-1, 1]; check it with margin on a dense grid plus the
    floats next to every boundary, in float64 and in emulated fp32."""
    text = (CSRC / "quantize_fast.cuh").read_text()
    c1, c2, c3 = (np.float32(re.search(rf"kNf4PolyC{i} = (-?[0-9.]+)f", text).group(1)) for i in (1, 2, 3))
    table = _floats(text, "kNf4LutBound")
    bounds = O.NF4_BOUNDS.astype(np.float32)
    assert np.array_equal(table[:15], bounds) and np.all(table[15:31] > 1e38) and table[31] < -1e38

    q = np.linspace(-1.0, 1.0, 2_000_001).astype(np.float32)
    edge = np.concatenate([np.nextafter(bounds, np.float32(-2)), bounds, np.nextafter(bounds, np.float32(2)),
                           np.float32([-1.0, 1.0, 0.0, -0.0])])
    q = np.concatenate([q, edge])
    index = np.searchsorted(bounds, q, side="left")
    q64 = q.astype(np.float64)
    p = 7.0 + q64 * (float(c1) + q64 * (float(c2) + q64 * float(c3)))
    # corridor with margin: index - 1.5 < p < index + 0.5
    margin = np.minimum(p - (index - 1.5), (index + 0.5) - p).min()
    assert margin > 0.03, margin
    # the evaluation the kernel does (fp32 FMAs; emulated here by rounding each step from float64)
    h = (q64 * float(c3) + float(c2)).astype(np.float32).astype(np.float64)
    h = (h * q64 + float(c1)).astype(np.float32).astype(np.float64)
    t = (h * q64 + 12582919.0).astype(np.float32)
    k = (t.view(np.uint32).astype(np.int64) - 0x4B400000).astype(np.int64)
    assert np.all((k == index) | (k == index - 1))
    got = k + (q > table[k % 32])
    assert np.array_equal(got, index)
    # the comparison as the kernel does it: c = saturate(fma(q, 2^40, -bound * 2^40)), 1e30 / -1e30 in the lanes
    # that stand for "-inf" / "no boundary"; the float64 sum of the two exact terms, rounded once to fp32, is what
    # the fused multiply-add returns
    scale = float(re.search(r"kNf4CmpScale = ([0-9.]+)f", text).group(1))
    assert scale == 2.0 ** 40
    lane = np.where(table > 1e38, -1e30, np.where(table < -1e38, 1e30, -table.astype(np.float64) * scale))
    assert np.array_equal(lane.astype(np.float32).astype(np.float64), lane) or np.allclose(lane, lane.astype(np.float32))
    c = np.clip((q64 * scale + lane[k % 32]).astype(np.float32), 0.0, 1.0)
    assert set(np.unique(c)) <= {0.0, 1.0}
    assert np.array_equal(k + c.astype(np.int64), index)
