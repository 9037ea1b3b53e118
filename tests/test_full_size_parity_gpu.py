"""Parity at the benchmark configurations' own sizes, through ``CompressionPlan`` (the batched launch that
``bench.py`` times, including its predicate-free bodies for full tensors), against the numpy oracle on the
same seeded inputs: every packed byte, fp32 scale, zero point and exponent byte must be equal.

  configuration 1   4096 x 4096 fp32, INT4_SYM group 128, seed 0 (+ SHA-256 digests of the state dict the
                    reference itself produced for the 8-layer model, tests/golden/config1.npz)
  configuration 2   Llama-3-8B shapes in bf16, INT8_ASYM per channel: 14336 x 4096, 4096 x 14336 and the
                    128256 x 4096 embedding
  headline          the same decoder shapes, INT4_SYM / INT4_ASYM group 128
  configuration 5   Mixtral expert shapes in bf16: NF4 group 128 and MXFP4 group 32 on 14336 x 4096 and
                    4096 x 14336
"""

import hashlib

import numpy as np
import pytest
import torch
from conftest import golden

pytestmark = pytest.mark.gpu


def _check_plan(items, rows_per_chunk=8192):
    """items: (name, weight on the GPU, mode, group size).  One plan, one launch, every output compared."""
    from oracle import wc_oracle as O

    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig
    from nncf_b200.pipeline import CompressionPlan

    plan = CompressionPlan([(n, w, WeightCompressionConfig(CompressWeightsMode(m), g)) for n, w, m, g in items])
    plan.run(use_graph=False)
    torch.cuda.synchronize()
    for (name, w, mode, gs), it in zip(items, plan.items):
        ref = O.stored_form(w.float().cpu().numpy(), mode, gs, rows_per_chunk)
        got = {"packed": it.packed, "scale": it.scale, "zero_point": it.zero_point, "scale_e8m0": it.scale_e8m0}
        for key, want in ref.items():
            have = got[key].cpu().numpy().reshape(-1)
            if have.dtype == np.int8 and want.dtype == np.uint8:
                have = have.view(np.uint8)
            assert have.shape == want.shape, f"{name} {mode} {key}: shape {have.shape} != {want.shape}"
            bad = int(np.count_nonzero(have.view(want.dtype) != want)) if have.dtype != want.dtype else \
                int(np.count_nonzero(have != want))
            assert bad == 0, f"{name} {mode} g{gs} {key}: {bad} of {want.size} values differ from the oracle"
        assert set(k for k, v in got.items() if v is not None) == set(ref), f"{name}: outputs {set(ref)} expected"


def _normal(shape, seed, dtype):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.empty(shape, dtype=dtype, device="cuda")
    w.normal_(0.0, 0.02, generator=gen)
    return w


def test_configuration_1_int4_sym_fp32_layers_match_oracle_and_reference_digests():
    from models import StackedLinear

    import nncf_b200 as nb

    model = StackedLinear(8, 4096).eval()
    _check_plan([(f"layers.{i}", lin.weight.detach().cuda().contiguous(), "int4_sym", 128)
                 for i, lin in enumerate(model.layers)][:3])
    # the whole model through the model-level call, against digests of the reference's own state dict
    cm = nb.compress_weights(model.cuda(), mode=nb.CompressWeightsMode.INT4_SYM, group_size=128, ratio=1.0)
    sd = cm.state_dict()
    g = golden("config1")
    for key, digest, meta in zip(g["config1/keys"], g["config1/sha256"], g["config1/meta"]):
        key = str(key)
        if key.startswith("__nncf_hooks"):
            # reference key: __nncf_hooks.post_hooks.layers:<i>:weight__0.0.<buffer>
            layer = key.split("post_hooks.")[1].split(":weight__")[0].replace(":", ".")
            mine = f"{layer}.parametrizations.weight.0.{key.rsplit('.', 1)[1]}"
        else:
            mine = key.replace(".weight", ".parametrizations.weight.original")
        a = np.ascontiguousarray(sd[mine].cpu().numpy())
        assert f"{a.dtype}{list(a.shape)}" == str(meta), f"{key}: {a.dtype}{list(a.shape)} != {meta}"
        assert hashlib.sha256(a.tobytes()).hexdigest() == str(digest), f"{key}: bytes differ from the reference's"


def test_configuration_2_int8_asym_per_channel_llama_shapes_match_oracle():
    _check_plan([
        ("gate_proj", _normal((14336, 4096), 11, torch.bfloat16), "int8_asym", -1),
        ("down_proj", _normal((4096, 14336), 12, torch.bfloat16), "int8_asym", -1),
        ("k_proj", _normal((1024, 4096), 13, torch.bfloat16), "int8_asym", -1),
    ])


def test_configuration_2_embedding_128256_rows_matches_oracle():
    _check_plan([("embed_tokens", _normal((128256, 4096), 1, torch.bfloat16), "int8_asym", -1)], rows_per_chunk=16032)


@pytest.mark.parametrize("mode", ["int4_sym", "int4_asym"])
def test_headline_int4_group_128_llama_shapes_match_oracle(mode):
    _check_plan([
        ("q_proj", _normal((4096, 4096), 21, torch.bfloat16), mode, 128),
        ("k_proj", _normal((1024, 4096), 22, torch.bfloat16), mode, 128),
        ("gate_proj", _normal((14336, 4096), 23, torch.bfloat16), mode, 128),
        ("down_proj", _normal((4096, 14336), 24, torch.bfloat16), mode, 128),
    ])


@pytest.mark.parametrize("mode,gs", [("nf4", 128), ("mxfp4", 32)])
def test_configuration_5_expert_shapes_match_oracle(mode, gs):
    _check_plan([
        ("experts.0.w1", _normal((14336, 4096), 4, torch.bfloat16), mode, gs),
        ("experts.0.w2", _normal((4096, 14336), 5, torch.bfloat16), mode, gs),
    ])
