"""Case tables shared by the fixture generator (make_golden.py) and the tests."""

import numpy as np

QUANT_CASES = [
    # name, shape, reduction axis, group size, kind
    ("g128", (8, 256), 1, 128, "normal"),
    ("g32", (6, 96), 1, 32, "normal"),
    ("g64", (4, 192), 1, 64, "uniform"),
    ("g16", (4, 48), 1, 16, "normal"),
    ("g8", (3, 40), 1, 8, "uniform"),
    ("g12_odd", (3, 36), 1, 12, "normal"),
    ("row", (5, 64), 1, -1, "normal"),
    ("row_odd", (7, 130), 1, -1, "uniform"),
    ("row_long", (2, 2056), 1, -1, "normal"),
    ("special_g32", (5, 64), 1, 32, "special"),
    ("special_row", (5, 32), 1, -1, "special"),
    ("pos_g32", (3, 64), 1, 32, "positive"),
    ("neg_g32", (3, 64), 1, 32, "negative"),
    ("arange_row", (4, 4), 1, -1, "arange"),
    ("t_g32", (64, 24), 0, 32, "normal"),      # [in, out] layout, groups strided by out
    ("t_row", (48, 10), 0, -1, "uniform"),
    ("e3d_g32", (2, 4, 64), 2, 32, "normal"),   # stacked experts, reduce last
    ("e3d_t_g16", (2, 32, 6), 1, 16, "normal"),  # stacked experts [E, in, out]
]
MODES = ["int8_sym", "int8_asym", "int4_sym", "int4_asym", "nf4", "mxfp4", "fp4", "fp8_e4m3", "mxfp8_e4m3"]
DTYPES = ["f32", "f16", "bf16"]

SE_CASES = [
    # name, out, in, gs, n_samples, mode, initial, scale_steps, axis, penalty
    ("int4_sym_g32", 16, 128, 32, 8, "int4_sym", 5, 5, 1, -1.0),
    ("int4_asym_g32", 16, 128, 32, 8, "int4_asym", 5, 5, 1, -1.0),
    ("int4_asym_g64_10", 12, 128, 64, 6, "int4_asym", 5, 10, 1, -1.0),
    ("int4_sym_row", 8, 64, -1, 5, "int4_sym", 5, 5, 1, -1.0),
    ("int4_asym_row", 8, 64, -1, 5, "int4_asym", 3, 4, 1, -1.0),
    ("nf4_g32", 10, 96, 32, 7, "nf4", 5, 5, 1, -1.0),
    ("int4_sym_g128", 24, 256, 128, 16, "int4_sym", 5, 5, 1, -1.0),
    ("int4_asym_g128", 24, 256, 128, 16, "int4_asym", 5, 5, 1, -1.0),
    ("int4_asym_t_g32", 16, 64, 32, 6, "int4_asym", 5, 5, 0, -1.0),  # weight [in, out]
    ("int4_sym_pen", 8, 64, 32, 6, "int4_sym", 5, 5, 1, 0.5),
    ("int4_asym_0steps", 8, 64, 32, 6, "int4_asym", 0, 0, 1, -1.0),
]

AWQ_CASES = [
    # name, out, in, gs, n, mode, percent, steps, with_prev
    ("int4_sym_g32", 16, 128, 32, 8, "int4_sym", 0.02, 100, False),
    ("int4_asym_g32", 16, 128, 32, 8, "int4_asym", 0.02, 100, False),
    ("int4_asym_g64_prev", 12, 128, 64, 6, "int4_asym", 0.02, 50, True),
    ("nf4_g32", 8, 64, 32, 5, "nf4", 0.05, 20, False),
    ("int4_sym_row", 8, 64, -1, 5, "int4_sym", 0.05, 30, False),
]

GPTQ_CASES = [
    # name, out, C, gs, block, mode, damp, n_inputs, tokens, x dtype
    ("int4_sym_g16", 20, 32, 16, 128, "int4_sym", 0.1, 10, 128, "f32"),
    ("int4_asym_g16", 20, 32, 16, 128, "int4_asym", 0.1, 10, 128, "f32"),
    ("int4_sym_g32_b32", 24, 128, 32, 32, "int4_sym", 0.01, 6, 96, "f32"),
    ("int4_sym_g64_b32", 16, 128, 64, 32, "int4_sym", 0.01, 6, 96, "f32"),
    ("int4_asym_g32_b64", 24, 128, 32, 64, "int4_asym", 0.01, 6, 96, "bf16"),
    ("nf4_g32_b64", 16, 128, 32, 64, "nf4", 0.05, 4, 96, "f32"),
    ("int4_sym_row", 12, 64, -1, 32, "int4_sym", 0.1, 4, 64, "f32"),
    ("int4_sym_g128", 32, 256, 128, 128, "int4_sym", 0.01, 4, 160, "bf16"),
]

# GPTQ(scale_estimation=True): same fields as GPTQ_CASES
GPTQ_SE_CASES = [
    ("se_int4_sym_g32_b64", 24, 128, 32, 64, "int4_sym", 0.01, 6, 96, "f32"),
    ("se_int4_asym_g32_b32", 16, 128, 32, 32, "int4_asym", 0.01, 6, 96, "f32"),
    ("se_int4_asym_g64_b128", 24, 256, 64, 128, "int4_asym", 0.05, 5, 64, "f32"),
    ("se_int4_sym_g128", 32, 256, 128, 128, "int4_sym", 0.01, 4, 160, "bf16"),
]


# inputs of the large GPTQ fixtures are regenerated in the tests from this frozen generator (np.random.RandomState
# streams never change between numpy versions), so only the reference's outputs are stored
GPTQ_LARGE = dict(rows=512, cols=1024, group_size=128, block=128, damp=0.01, n_inputs=8, tokens=128, seed=20240)


def gptq_large_inputs():
    """(w fp32 [rows, cols], list of bf16-representable fp32 activations [1, tokens, cols])."""
    import torch

    c = GPTQ_LARGE
    rs = np.random.RandomState(c["seed"])
    w = (rs.randn(c["rows"], c["cols"]) * 0.02).astype(np.float32)
    mix = np.eye(c["cols"], dtype=np.float32) + 0.5 * (rs.randn(c["cols"], c["cols"]).astype(np.float32) / np.sqrt(c["cols"]))
    xs = []
    for _ in range(c["n_inputs"]):
        x = rs.randn(1, c["tokens"], c["cols"]).astype(np.float32) @ mix
        xs.append(torch.from_numpy(x).to(torch.bfloat16).float().numpy())
    return w, xs


LORA_CASES = [
    # name, out, in, gs, n samples, mode, rank, iterations, regularization
    ("int4_sym_g32_r8", 96, 128, 32, 24, "int4_sym", 8, 3, True),
    ("int4_asym_g32_r4", 64, 128, 32, 16, "int4_asym", 4, 3, True),
    ("nf4_g64_r8", 80, 192, 64, 32, "nf4", 8, 2, True),
    ("int4_sym_g32_noreg", 96, 128, 32, 24, "int4_sym", 8, 3, False),
    ("int4_asym_row_r8", 48, 64, -1, 12, "int4_asym", 8, 3, True),
    ("int4_sym_g32_many_samples", 40, 64, 32, 150, "int4_sym", 8, 2, True),   # more samples than subset_size = 128
]
