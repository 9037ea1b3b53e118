"""The multi-threaded torch CPU baseline equals the numpy oracle bit for bit."""

import numpy as np
import pytest
import torch

from oracle import wc_oracle as O
from oracle import wc_oracle_torch as T


@pytest.mark.parametrize("mode", ["int8_sym", "int8_asym", "int4_sym", "int4_asym"])
@pytest.mark.parametrize("gs", [128, 32, -1])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_torch_port_matches_numpy_oracle(mode, gs, dtype):
    torch.manual_seed(3)
    w = (torch.randn(64, 512) * 0.02).to(dtype)
    codes, scale, zp = T.compress_weight_int(w, mode, gs)
    ref = O.compress_weight(w.float().numpy(), 1, mode, gs)
    np.testing.assert_array_equal(codes.numpy(), ref.tensor)
    np.testing.assert_array_equal(scale.numpy(), ref.scale)
    if zp is not None:
        np.testing.assert_array_equal(zp.numpy(), ref.zero_point)
    packed = T.pack_weight(codes, mode).numpy()
    if mode == "int4_sym":
        np.testing.assert_array_equal(packed, O.pack_int4(ref.tensor))
    elif mode == "int4_asym":
        np.testing.assert_array_equal(packed, O.pack_uint4(ref.tensor))
