"""``nncf_b200.compress_weights`` on a toy Llama-like torch model against the state dict that the
reference's ``nncf.compress_weights`` produced for the same seeded model (tests/golden/api.npz).

Data-free cases must match bit for bit (packed weights, fp16 scales, packed zero points, which layers got
which precision).  Data-aware cases take their statistics from a forward pass on the GPU whose fp32
matmuls differ from the reference's CPU pass in the last bits, so scales are compared with a tolerance and
the model outputs against the reference's outputs."""

import numpy as np
import pytest
import torch
from conftest import golden
from models import API_CASES, LAYERWISE, TinyGatedLM, calibration_ids, layerwise_ids

pytestmark = pytest.mark.gpu

LAYERS = ["embed", "blocks.0.q", "blocks.0.gate", "blocks.0.up", "blocks.0.down", "blocks.1.q", "blocks.1.gate",
          "blocks.1.up", "blocks.1.down", "head"]


def _compress(kwargs, use_ds):
    import nncf_b200 as nb

    torch.backends.cuda.matmul.allow_tf32 = False
    model = TinyGatedLM().cuda()
    ids = [i.cuda() for i in calibration_ids()]
    kw = dict(kwargs)
    kw["mode"] = nb.CompressWeightsMode(kw["mode"])
    if "sensitivity_metric" in kw:
        kw["sensitivity_metric"] = nb.SensitivityMetric(kw["sensitivity_metric"])
    if kw.get("awq"):
        kw["advanced_parameters"] = nb.AdvancedCompressionParameters(awq_params=nb.AdvancedAWQParameters(percent_to_apply=0.05))
    # the reference needs a dataset item for tracing in every case; here it only fixes the layer order
    return nb.compress_weights(model, dataset=nb.Dataset(ids) if use_ds else None, **kw), ids


def _ref(g, key, layer, what):
    k = f"{key}/__nncf_hooks.post_hooks.{layer.replace('.', ':')}:weight__0.0.{what}"
    return g[k] if k in g else None


@pytest.mark.parametrize("case", API_CASES, ids=[c[0] for c in API_CASES])
def test_compress_weights_matches_reference_state_dict(case):
    name, kwargs, use_ds = case
    g = golden("api")
    key = f"api/{name}"
    model, ids = _compress(kwargs, use_ds)
    sd = model.state_dict()
    exact = not (kwargs.get("awq") or kwargs.get("scale_estimation") or "sensitivity_metric" in kwargs)
    mism, total = 0, 0
    for layer in LAYERS:
        ref_w = g[f"{key}/{layer}.weight"]
        got_w = sd[f"{layer}.parametrizations.weight.original"].cpu().numpy()
        assert got_w.shape == ref_w.shape and got_w.dtype == ref_w.dtype, f"{layer}: precision assignment differs"
        ref_s = _ref(g, key, layer, "_scale")
        got_s = sd[f"{layer}.parametrizations.weight.0._scale"].cpu().numpy()
        assert got_s.shape == ref_s.shape and got_s.dtype == np.float16
        ref_z = _ref(g, key, layer, "_zero_point")
        got_z = sd.get(f"{layer}.parametrizations.weight.0._zero_point")
        assert (ref_z is None) == (got_z is None)
        if exact:
            np.testing.assert_array_equal(got_w, ref_w, err_msg=layer)
            np.testing.assert_array_equal(got_s, ref_s, err_msg=layer)
            if ref_z is not None:
                np.testing.assert_array_equal(got_z.cpu().numpy(), ref_z, err_msg=layer)
        else:
            np.testing.assert_allclose(got_s.astype(np.float32), ref_s.astype(np.float32), rtol=2e-2, atol=1e-4)
            mism += int(np.sum(got_w != ref_w))
            total += got_w.size
    if not exact:
        assert mism / total < 0.05, f"{mism}/{total} packed bytes differ"
    with torch.no_grad():
        out = model(ids[0]).float().cpu().numpy()
    ref_out = g[key + "/logits"]
    tol = 1e-5 if exact else 3e-2
    assert np.linalg.norm(out - ref_out) / np.linalg.norm(ref_out) < tol


def test_nf4_and_mxfp4_models_run_and_stay_close_to_the_original():
    """Modes the reference's torch backend rejects: the compressed model must run and approximate the original."""
    import nncf_b200 as nb

    ids = [i.cuda() for i in calibration_ids()]
    with torch.no_grad():
        base = TinyGatedLM().cuda()(ids[0])
    for mode, gs in (("nf4", 16), ("mxfp4", 32), ("fp4", 16)):
        model = nb.compress_weights(TinyGatedLM().cuda(), mode=nb.CompressWeightsMode(mode), group_size=gs)
        with torch.no_grad():
            out = model(ids[0])
        rel = float((out - base).norm() / base.norm())
        assert rel < 0.25, (mode, rel)
        assert model.blocks[0].q.parametrizations.weight.original.dtype == torch.uint8
        # the default backup of the embedding / last layer: MXFP8 for MXFP4, FP8 for FP4, INT8_ASYM otherwise
        expect = {"nf4": "int8_asym", "mxfp4": "mxfp8_e4m3", "fp4": "fp8_e4m3"}[mode]
        assert model.head.parametrizations.weight[0].mode.value == expect


def test_invalid_options_raise_like_the_reference():
    import nncf_b200 as nb

    m = TinyGatedLM().cuda()
    with pytest.raises(nb.ParameterNotSupportedError):
        nb.compress_weights(m, mode=nb.CompressWeightsMode.INT8_ASYM, group_size=64)
    with pytest.raises(nb.ParameterNotSupportedError):
        nb.compress_weights(m, mode=nb.CompressWeightsMode.INT8_SYM, awq=True)
    with pytest.raises(nb.ValidationError):
        nb.compress_weights(m, mode=nb.CompressWeightsMode.INT4_SYM, ratio=1.5)
    with pytest.raises(nb.ValidationError):
        nb.compress_weights(m, mode=nb.CompressWeightsMode.MXFP4, group_size=64)
    with pytest.raises(nb.InvalidGroupSizeError):
        nb.compress_weights(m, mode=nb.CompressWeightsMode.INT4_SYM, group_size=24)
    with pytest.raises(nb.ParameterNotSupportedError):
        nb.compress_weights(m, mode=nb.CompressWeightsMode.INT4_SYM, lora_correction=True)


def test_gptq_model_level_reduces_output_error():
    """GPTQ through the model API: output error on the calibration data must not exceed plain rounding's."""
    import nncf_b200 as nb

    ids = [i.cuda() for i in calibration_ids(n=8, seq=32)]
    with torch.no_grad():
        base = torch.cat([TinyGatedLM().cuda()(i) for i in ids])
    errs = {}
    for use_gptq in (False, True):
        model = nb.compress_weights(TinyGatedLM().cuda(), mode=nb.CompressWeightsMode.INT4_SYM, group_size=16,
                                    dataset=nb.Dataset(ids), gptq=use_gptq or None,
                                    advanced_parameters=nb.AdvancedCompressionParameters(
                                        gptq_params=nb.AdvancedGPTQParameters(damp_percent=0.1, subset_size=8)))
        with torch.no_grad():
            out = torch.cat([model(i) for i in ids])
        errs[use_gptq] = float((out - base).norm() / base.norm())
    assert errs[True] < errs[False] * 1.05, errs


def test_gptq_with_scale_estimation_model_level():
    """gptq=True together with scale_estimation=True hands the flag to GPTQ (every group's parameters come from
    ScaleEstimation inside the sweep): it runs through the model API, changes the stored scales and keeps the
    output error at the level of plain GPTQ."""
    import nncf_b200 as nb

    ids = [i.cuda() for i in calibration_ids(n=8, seq=32)]
    with torch.no_grad():
        base = torch.cat([TinyGatedLM().cuda()(i) for i in ids])
    errs, scales = {}, {}
    for se in (False, True):
        model = nb.compress_weights(TinyGatedLM().cuda(), mode=nb.CompressWeightsMode.INT4_ASYM, group_size=16,
                                    dataset=nb.Dataset(ids), gptq=True, scale_estimation=se or None,
                                    advanced_parameters=nb.AdvancedCompressionParameters(
                                        gptq_params=nb.AdvancedGPTQParameters(damp_percent=0.1, subset_size=8)))
        with torch.no_grad():
            out = torch.cat([model(i) for i in ids])
        errs[se] = float((out - base).norm() / base.norm())
        scales[se] = torch.cat([v.flatten().float() for k, v in model.state_dict().items() if k.endswith("_scale")])
    assert (scales[True] != scales[False]).float().mean().item() > 0.3
    assert errs[True] < errs[False] * 1.5, errs


@pytest.mark.parametrize("kwargs", [dict(mode="int4_asym", group_size=16), dict(mode="int4_sym", group_size=16, all_layers=True),
                                    dict(mode="int8_sym"), dict(mode="int8_asym"), dict(mode="nf4", group_size=16),
                                    dict(mode="mxfp4", group_size=32)])
def test_config_state_dict_round_trip_and_strip(kwargs):
    """get_config + state_dict rebuild the compressed model on a fresh instance (same logits bit for bit, same
    state); strip leaves plain dense weights that compute the same outputs."""
    import json

    import nncf_b200 as nb

    ids = calibration_ids(n=2, seq=12)[0].cuda()
    kw = dict(kwargs)
    kw["mode"] = nb.CompressWeightsMode(kw["mode"])
    model = nb.compress_weights(TinyGatedLM().cuda(), **kw)
    with torch.no_grad():
        want = model(ids)
    config = json.loads(json.dumps(nb.get_config(model)))      # the config survives JSON
    state = {k: v.cpu() for k, v in model.state_dict().items()}
    assert config["weights"], "nothing was recorded"
    fresh = nb.load_from_config(TinyGatedLM(seed=5).cuda(), config, state)
    with torch.no_grad():
        assert torch.equal(fresh(ids), want)
    assert fresh.state_dict().keys() == model.state_dict().keys()
    sizes = nb.serialization.compressed_nbytes(fresh)
    assert 0 < sizes["compressed_bytes"] < sizes["dense_bytes"]
    nb.strip(fresh)
    assert not any("parametrizations" in k for k in fresh.state_dict())
    assert all(p.dtype == torch.float32 for p in fresh.parameters())
    with torch.no_grad():
        torch.testing.assert_close(fresh(ids), want, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        nb.load_from_config(TinyGatedLM().cuda(), {"format": "other", "weights": {}})


def test_gptq_block_replay_equals_full_prefix_runs_on_hf_llama(monkeypatch):
    """Model-level GPTQ on a Hugging Face Llama: replaying each decoder layer on cached inputs (through the
    already-quantised layers before it) - with one resumable forward per block, or re-running the block for
    every layer - gives the same compressed model as re-running the whole prefix of the model for every layer,
    and the key / value cache the model passes to its layers is not replayed."""
    transformers = pytest.importorskip("transformers")
    import nncf_b200 as nb
    from nncf_b200 import compress_api

    cfg = transformers.LlamaConfig(vocab_size=96, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    gen = torch.Generator().manual_seed(0)
    ids = [torch.randint(0, 96, (1, 24), generator=gen).cuda() for _ in range(6)]
    states = {}
    for replay in ("resumable", True, False):
        monkeypatch.setattr(compress_api, "LAYERWISE_REPLAY", bool(replay))
        monkeypatch.setattr(compress_api, "RESUMABLE_REPLAY", replay == "resumable")
        torch.manual_seed(0)
        model = transformers.LlamaForCausalLM(cfg).cuda().eval()
        blocks = compress_api._decoder_blocks(model, compress_api.get_weight_compression_parameters(model, None, ids[0]))
        assert blocks is not None and len(blocks) == 3
        model = nb.compress_weights(model, mode=nb.CompressWeightsMode.INT4_SYM, group_size=32, dataset=nb.Dataset(ids),
                                    gptq=True, advanced_parameters=nb.AdvancedCompressionParameters(
                                        gptq_params=nb.AdvancedGPTQParameters(damp_percent=0.1, subset_size=6)))
        states[replay] = {k: v.clone() for k, v in model.state_dict().items()}
        with torch.no_grad():
            states[replay]["__logits"] = model(ids[0]).logits
    for other in ("resumable", True):
        assert states[other].keys() == states[False].keys()
        differing = [k for k in states[other] if not torch.equal(states[other][k], states[False][k])]
        # identical computations up to the batch size of the matrix products (six items in one stacked call
        # against one call per item), which may change a few codes
        frac = sum(states[other][k].numel() for k in differing) / sum(v.numel() for v in states[other].values())
        assert frac < 0.05, (other, differing)
        rel = (states[other]["__logits"] - states[False]["__logits"]).norm() / states[False]["__logits"].norm()
        assert rel < 0.05, other
    # the two replay forms see the very same micro-batches: identical results
    assert all(torch.equal(states["resumable"][k], states[True][k]) for k in states[True])


@pytest.mark.parametrize("mode,gs", [("int4_sym", 128), ("int4_asym", 64), ("int8_asym", -1), ("int8_sym", -1),
                                     ("nf4", 128), ("mxfp4", 32), ("fp8_e4m3", 128), ("mxfp8_e4m3", 32)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_decompress_kernel_matches_oracle(mode, gs, dtype):
    """nncfb_decompress against the reference's fp16 decompression arithmetic restated by the oracle."""
    from oracle import wc_oracle as O

    import nncf_b200 as nb
    from nncf_b200 import weight_lowering as wl
    from nncf_b200.compress_api import _make_decompressor
    from nncf_b200.config import WeightCompressionParameters

    gen = torch.Generator().manual_seed(9)
    lin = torch.nn.Linear(512, 96, bias=False)
    lin.weight.data = (torch.randn(96, 512, generator=gen) * 0.05)
    lin = lin.cuda().to(dtype)
    cfg = nb.WeightCompressionConfig(nb.CompressWeightsMode(mode), gs)
    p = WeightCompressionParameters("l", lin, "weight", (1,), cfg)
    cw = wl.compress_weight(lin.weight.data, 1, cfg, pack=True)
    dec = _make_decompressor(p, cw)
    got = dec(cw.packed).float().cpu().numpy()
    w_np = lin.weight.data.float().cpu().numpy()
    ref = O.compress_weight(w_np if dtype != torch.float16 else lin.weight.data.cpu().numpy(), 1, mode, gs)
    if O.is_integer(mode):
        s16 = ref.scale.astype(np.float16)
        dq = O.decompress_asymmetric(ref.tensor, s16, ref.zero_point) if O.is_asym(mode) else O.decompress_symmetric(ref.tensor, s16)
        exp = torch.from_numpy(dq.astype(np.float32)).to(dtype).float().numpy().reshape(96, 512)
    else:
        exp = torch.from_numpy((ref.tensor * ref.scale).astype(np.float32)).to(dtype).float().numpy().reshape(96, 512)
    np.testing.assert_array_equal(got, exp)


def test_hf_llama_model_awq_scale_estimation_end_to_end():
    """A randomly initialised Hugging Face Llama decoder (2 layers, hidden 64): INT4_ASYM g32 with AWQ and
    ScaleEstimation must find the up_proj -> multiply -> down_proj pairs, keep the embedding and lm_head in the
    INT8_ASYM backup, and stay close to the original model's logits."""
    transformers = pytest.importorskip("transformers")
    import nncf_b200 as nb
    from nncf_b200.compress_api import find_mul_merge_pairs

    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=256, max_position_embeddings=64,
                                   tie_word_embeddings=False)
    model = transformers.LlamaForCausalLM(cfg).cuda().eval()
    gen = torch.Generator().manual_seed(2)
    items = [{"input_ids": torch.randint(0, 256, (1, 24), generator=gen).cuda()} for _ in range(8)]
    with torch.no_grad():
        base = model(**items[0]).logits.float()
    targets = {n: m for n, m in model.named_modules() if isinstance(m, torch.nn.Linear)}
    pairs = find_mul_merge_pairs(model, items[0], targets)
    assert {n.split(".")[-1] for n in pairs} == {"down_proj"}
    assert all(m is model.get_submodule(n.replace("down_proj", "up_proj")) for n, m in pairs.items())
    cm = nb.compress_weights(model, mode=nb.CompressWeightsMode.INT4_ASYM, group_size=32, dataset=nb.Dataset(items),
                             awq=True, scale_estimation=True,
                             advanced_parameters=nb.AdvancedCompressionParameters(
                                 awq_params=nb.AdvancedAWQParameters(percent_to_apply=0.05)))
    with torch.no_grad():
        out = cm(**items[0]).logits.float()
    rel = float((out - base).norm() / base.norm())
    assert rel < 0.2, rel
    sd = cm.state_dict()
    assert sd["lm_head.parametrizations.weight.original"].shape == (256, 64)           # INT8 backup, unpacked bytes
    assert sd["model.embed_tokens.parametrizations.weight.original"].shape == (256, 64)
    assert sd["model.layers.0.mlp.down_proj.parametrizations.weight.original"].shape == (64 * 128 // 2, 1)


def test_tied_embedding_and_head_are_compressed_once_and_both_keep_working():
    """``lm_head.weight is embed_tokens.weight`` (the default of many Hugging Face models): the shared Parameter is
    compressed once, in the embedding's precision (INT8_ASYM backup), both modules decompress the one packed
    tensor, the last remaining Linear stays in the primary precision (the reference skips a shared last layer,
    algorithm.py:992-1007, 559-561), and the model's outputs stay close to the dense model's."""
    transformers = pytest.importorskip("transformers")
    import nncf_b200 as nb

    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                   num_key_value_heads=2, vocab_size=256, max_position_embeddings=64,
                                   tie_word_embeddings=True)
    model = transformers.LlamaForCausalLM(cfg).cuda().eval()
    assert model.lm_head.weight is model.model.embed_tokens.weight
    ids = torch.randint(0, 256, (1, 24), generator=torch.Generator().manual_seed(2)).cuda()
    with torch.no_grad():
        base = model(input_ids=ids).logits.float()
    cm = nb.compress_weights(model, mode=nb.CompressWeightsMode.INT4_SYM, group_size=32)
    sd = cm.state_dict()
    emb = sd["model.embed_tokens.parametrizations.weight.original"]
    head = sd["lm_head.parametrizations.weight.original"]
    assert emb.dtype == torch.uint8 and tuple(emb.shape) == (256, 64)            # INT8_ASYM, unpacked bytes
    assert head.data_ptr() == emb.data_ptr()                                       # one packed tensor, two holders
    assert cm.lm_head.parametrizations.weight[0] is cm.model.embed_tokens.parametrizations.weight[0]
    assert tuple(cm.lm_head.weight.shape) == (256, 64) and cm.lm_head.weight.dtype == base.dtype
    # the last decoder layer's down_proj is the last remaining Linear: still 4-bit (nibble-packed)
    assert tuple(sd["model.layers.1.mlp.down_proj.parametrizations.weight.original"].shape) == (64 * 128 // 2, 1)
    with torch.no_grad():
        out = cm(input_ids=ids).logits.float()
    assert float((out - base).norm() / base.norm()) < 0.25


@pytest.mark.parametrize("mode,kw", [("int8_asym", {}), ("int8_sym", {}),
                                     ("int4_asym", dict(group_size=4, all_layers=True)),
                                     ("int4_sym", dict(group_size=10, all_layers=True))])
def test_inner_dimension_that_is_not_a_multiple_of_8_compresses_and_runs(mode, kw):
    """Linear(100 -> 20 -> 100): per-channel groups of 100 elements (or groups of 4 / 10) end inside an 8-element vector
    of the decompression kernel's fast path; the element-per-thread path must give the oracle's fp16 arithmetic."""
    from oracle import wc_oracle as O

    import nncf_b200 as nb

    torch.manual_seed(1)
    model = torch.nn.Sequential(torch.nn.Linear(100, 20, bias=False), torch.nn.Linear(20, 100, bias=False)).cuda().half()
    dense = [m.weight.detach().clone() for m in model]
    cm = nb.compress_weights(model, mode=nb.CompressWeightsMode(mode), **kw)
    x = torch.randn(3, 100, device="cuda", dtype=torch.float16)
    assert torch.isfinite(cm(x)).all()
    for m, w in zip(cm, dense):
        gs = kw.get("group_size", -1)
        ref = O.compress_weight(w.cpu().numpy(), 1, mode, gs)
        s16 = ref.scale.astype(np.float16)
        dq = O.decompress_asymmetric(ref.tensor, s16, ref.zero_point) if O.is_asym(mode) else O.decompress_symmetric(ref.tensor, s16)
        np.testing.assert_array_equal(m.weight.detach().cpu().numpy(), dq.reshape(w.shape))


def _distributed_gptq_model():
    """A two-block Llama and 16 x 64 calibration tokens over a vocabulary of 512: more tokens than hidden channels and
    more distinct embeddings than that, so every Hessian has full rank and the comparison between two summation
    orders is not dominated by the damping of a singular matrix."""
    import transformers

    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    gen = torch.Generator().manual_seed(0)
    ids = [torch.randint(0, 512, (1, 64), generator=gen).cuda() for _ in range(16)]
    torch.manual_seed(0)
    return transformers.LlamaForCausalLM(cfg).cuda().eval(), ids


def _distributed_gptq_worker(rank, world, port, q):
    import os

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import nncf_b200 as nb

        model, ids = _distributed_gptq_model()
        model = nb.compress_weights(model, mode=nb.CompressWeightsMode.INT4_ASYM, group_size=64, dataset=nb.Dataset(ids),
                                    gptq=True, process_group=dist.group.WORLD,
                                    advanced_parameters=nb.AdvancedCompressionParameters(
                                        gptq_params=nb.AdvancedGPTQParameters(damp_percent=0.1, subset_size=16)))
        sd = {k: v.cpu() for k, v in model.state_dict().items()}
        with torch.no_grad():
            sd["__logits"] = model(ids[0]).logits.float().cpu()
        q.put((rank, sd))
    except Exception as exc:  # noqa: BLE001
        q.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_gptq_shared_among_two_ranks_matches_one_rank():
    """Distributed GPTQ on two GPUs (calibration items shared out, Hessians all-reduced, one inverse factor,
    rows swept by different ranks and all-gathered): both ranks end with the same compressed model, and it
    agrees with the single-process result up to the code flips that another summation order of the Hessian
    causes.  Needs two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    pytest.importorskip("transformers")
    import socket

    import torch.multiprocessing as mp

    import nncf_b200 as nb

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_distributed_gptq_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    assert all(isinstance(v, dict) for v in results.values()), results
    a, b = results[0], results[1]
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    model, ids = _distributed_gptq_model()
    model = nb.compress_weights(model, mode=nb.CompressWeightsMode.INT4_ASYM, group_size=64, dataset=nb.Dataset(ids),
                                gptq=True, advanced_parameters=nb.AdvancedCompressionParameters(
                                    gptq_params=nb.AdvancedGPTQParameters(damp_percent=0.1, subset_size=16)))
    one = {k: v.cpu() for k, v in model.state_dict().items()}
    with torch.no_grad():
        one["__logits"] = model(ids[0]).logits.float().cpu()
    assert one.keys() == a.keys()
    packed = [k for k in one if k.endswith("weight.original")]
    differing = sum(int((one[k] != a[k]).sum()) for k in packed) / sum(one[k].numel() for k in packed)
    assert differing < 0.05, differing
    rel = float((one["__logits"] - a["__logits"]).norm() / one["__logits"].norm())
    assert rel < 0.05, rel


def test_reference_key_names_and_safetensors_round_trip(tmp_path):
    """The state dict under the reference's key names has exactly the keys, dtypes and shapes the reference's own
    compressed model has (tests/golden/api.npz), and a safetensors file with the manifest in its metadata
    rebuilds the compressed model in a fresh process-like setting (new dense model, no compression call)."""
    import nncf_b200 as nb

    name, kwargs, use_ds = API_CASES[3]   # int4_asym group 16, all layers
    model, ids = _compress(kwargs, use_ds)
    g = golden("api")
    ref_keys = [str(k) for k in g[f"api/{name}/keys"]]
    sd = nb.reference_state_dict(model)
    assert sorted(sd) == sorted(ref_keys)
    for k in ref_keys:
        want = g[f"api/{name}/{k}"]
        assert tuple(sd[k].shape) == want.shape and str(sd[k].dtype).replace("torch.", "") == str(want.dtype), k
        np.testing.assert_array_equal(sd[k].cpu().numpy(), want)
    path = str(tmp_path / "model.safetensors")
    nb.save_safetensors(model, path)
    fresh = nb.load_safetensors(TinyGatedLM().cuda(), path)
    with torch.no_grad():
        assert torch.equal(fresh(ids[0]), model(ids[0]))
    for (ka, va), (kb, vb) in zip(model.state_dict().items(), fresh.state_dict().items()):
        assert ka == kb and torch.equal(va, vb)


@pytest.mark.parametrize("mode,gs", [("int4_asym", 32), ("int4_sym", 128), ("int8_asym", -1), ("int8_sym", -1)])
def test_gptq_style_layout_decodes_to_the_decompressed_weight(mode, gs):
    """qweight / qzeros / scales / g_idx of a compressed Linear, decoded with the GPTQ formula
    W[o, i] = scales[g_idx[i], o] * (code[i, o] - zero[g_idx[i], o]), equal the decompressor's output (which
    multiplies in fp16; the formula is evaluated in fp32 here, hence the 2^-10 tolerance)."""
    import nncf_b200 as nb

    torch.manual_seed(3)
    lin = torch.nn.Linear(256, 64, bias=False).cuda().half()
    holder = torch.nn.Sequential(lin)
    kw = {} if gs == -1 else dict(group_size=gs, all_layers=True)
    nb.compress_weights(holder, mode=nb.CompressWeightsMode(mode), **kw)
    lay = nb.gptq_layout(holder[0])
    bits, pack = lay["bits"], 32 // lay["bits"]
    assert lay["qweight"].shape == (256 // pack, 64) and lay["qweight"].dtype == torch.int32
    groups = 256 // (gs if gs != -1 else 256)
    assert lay["qzeros"].shape == (groups, 64 // pack) and lay["scales"].shape == (groups, 64)
    shifts = torch.arange(pack, device="cuda", dtype=torch.int64) * bits
    mask = (1 << bits) - 1
    qw = lay["qweight"].to(torch.int64) & 0xFFFFFFFF
    codes = ((qw.unsqueeze(1) >> shifts.view(1, pack, 1)) & mask).reshape(256, 64)             # [in, out]
    qz = lay["qzeros"].to(torch.int64) & 0xFFFFFFFF
    zeros = ((qz.unsqueeze(2) >> shifts.view(1, 1, pack)) & mask).reshape(groups, 64)         # [groups, out]
    gi = lay["g_idx"].long()
    w = lay["scales"].float()[gi] * (codes - zeros[gi]).float()                                 # [in, out]
    torch.testing.assert_close(w.t(), holder[0].weight.float(), rtol=2 ** -10, atol=1e-7)


@pytest.mark.parametrize("mode", LAYERWISE["modes"])
def test_model_level_gptq_follows_the_reference_schedule_and_reference_gptq(mode):
    """Model-level GPTQ against tests/golden/layerwise.npz: the reference's own schedule on the graph it traced
    from this model, its Hessian and its quantiser per layer, every step fed by the model with the earlier
    steps' weights already quantised (embedding and head left in floating point on both sides).  Later layers see
    inputs that passed through earlier quantised layers, so a rounding flip early on would perturb everything
    after it: the integer codes of all eight layers must still agree with the reference's except for a handful,
    and the stored fp16 scale is the reference's fp32 scale rounded once."""
    import nncf_b200 as nb

    torch.backends.cuda.matmul.allow_tf32 = False
    c = LAYERWISE
    gs = c["group_size"]
    g = golden("layerwise")
    key = f"layerwise/{mode}"
    ids = [i.cuda() for i in layerwise_ids()]
    model = TinyGatedLM(**c["model"]).eval().cuda()
    cm = nb.compress_weights(model, mode=nb.CompressWeightsMode(mode), group_size=gs, dataset=nb.Dataset(ids),
                             gptq=True, subset_size=len(ids), all_layers=True, ignored_scope=["embed", "head"],
                             advanced_parameters=nb.AdvancedCompressionParameters(
                                 gptq_params=nb.AdvancedGPTQParameters(damp_percent=c["damp"], subset_size=len(ids))))
    mods = dict(cm.named_modules())
    flips = total = 0
    for step in g[key + "/steps"]:
        for m in str(step).split(","):
            want = torch.from_numpy(g[f"{key}/{m}/weight"]).cuda()
            s_want = torch.from_numpy(g[f"{key}/{m}/scale"]).cuda().reshape(want.shape[0], -1)
            have = mods[m].weight.detach().float()
            buffers = mods[m].parametrizations.weight[0].state_dict()
            s_have = [v for k, v in buffers.items() if k.endswith("scale")][0].float().reshape(want.shape[0], -1)
            assert torch.equal(s_have, s_want.half().float()), m     # same fp32 scale, stored in half precision
            # signed distance from the zero point in quantisation steps: identical integers when no code flipped
            k_want = torch.round(want.reshape(want.shape[0], -1, gs) / s_want[..., None])
            k_have = torch.round(have.reshape(want.shape[0], -1, gs) / s_have[..., None])
            flips += int((k_want != k_have).sum())
            total += want.numel()
            assert float((have - want).norm() / want.norm()) < 1e-3, m
    assert flips <= total * 1e-3, (flips, total)
    with torch.no_grad():
        logits = cm(ids[0]).float().cpu()
    want = torch.from_numpy(g[key + "/logits"])
    assert float((logits - want).norm() / want.norm()) < 2e-3


def _lora_model(int8=True, mode="int4_sym", **extra):
    import nncf_b200 as nb

    ids = [i.cuda() for i in calibration_ids(n=8, seq=32)]
    model = TinyGatedLM().cuda()
    adv = nb.AdvancedCompressionParameters(lora_correction_params=nb.AdvancedLoraCorrectionParameters(
        adapter_rank=4, use_int8_adapters=int8))
    cm = nb.compress_weights(model, mode=nb.CompressWeightsMode(mode), group_size=16, dataset=nb.Dataset(ids),
                             lora_correction=True, advanced_parameters=adv, **extra)
    return cm, ids


@pytest.mark.parametrize("int8", [True, False])
def test_lora_correction_model_level_reduces_output_error(int8):
    """``lora_correction=True`` (the reference has it for OpenVINO graphs only, openvino_backend.py:178-218,362-369):
    every 4-bit Linear gets two adapters whose output is added to the layer's; the error of the model's output on
    the calibration data falls below plain rounding's, the adapters are in the state dict (INT8_ASYM with their
    own scale and zero point, or dense), embedding and INT8 backup layers get none."""
    import nncf_b200 as nb

    with torch.no_grad():
        ids = [i.cuda() for i in calibration_ids(n=8, seq=32)]
        base = torch.cat([TinyGatedLM().cuda()(i) for i in ids])
        plain = nb.compress_weights(TinyGatedLM().cuda(), mode=nb.CompressWeightsMode.INT4_SYM, group_size=16)
        err_plain = float((torch.cat([plain(i) for i in ids]) - base).norm() / base.norm())
        cm, _ = _lora_model(int8)
        err_lora = float((torch.cat([cm(i) for i in ids]) - base).norm() / base.norm())
    assert err_lora < 0.9 * err_plain, (err_lora, err_plain)
    sd = cm.state_dict()
    with_adapters = sorted({k.split(".lora_correction.")[0] for k in sd if ".lora_correction." in k})
    assert with_adapters == sorted(n for n in LAYERS if n not in ("embed", "head"))
    a = sd["blocks.0.q.lora_correction.a.weight"]
    assert tuple(a.shape) == (4, 32) and a.dtype == (torch.uint8 if int8 else torch.float32)
    assert ("blocks.0.q.lora_correction.a.decompressor._scale" in sd) == int8


def test_lora_correction_survives_config_round_trip_and_strip(tmp_path):
    import nncf_b200 as nb

    cm, ids = _lora_model(True, "int4_asym")
    with torch.no_grad():
        want = cm(ids[0])
    cfg = nb.get_config(cm)
    assert cfg["weights"]["blocks.1.down"]["lora_correction"] == {"rank": 4, "int8": True}
    fresh = nb.load_from_config(TinyGatedLM(seed=5).cuda(), cfg, cm.state_dict())
    nb.save_safetensors(cm, str(tmp_path / "lora.safetensors"))
    from_file = nb.load_safetensors(TinyGatedLM(seed=6).cuda(), str(tmp_path / "lora.safetensors"))
    with torch.no_grad():
        assert torch.equal(fresh(ids[0]), want)
        assert torch.equal(from_file(ids[0]), want)
        stripped = nb.strip(fresh)
        assert not any("lora_correction" in k or "parametrizations" in k for k in stripped.state_dict())
        got = stripped(ids[0])
    assert float((got - want).norm() / want.norm()) < 1e-5     # adapters folded into the dense weights


def test_lora_correction_option_checks():
    import nncf_b200 as nb

    ids = [i.cuda() for i in calibration_ids()]
    with pytest.raises(nb.ParameterNotSupportedError):
        nb.compress_weights(TinyGatedLM().cuda(), mode=nb.CompressWeightsMode.INT4_SYM, group_size=16,
                            dataset=nb.Dataset(ids), gptq=True, lora_correction=True)
    with pytest.raises(nb.ParameterNotSupportedError):
        nb.compress_weights(TinyGatedLM().cuda(), mode=nb.CompressWeightsMode.MXFP4, dataset=nb.Dataset(ids),
                            lora_correction=True)
    with pytest.raises(nb.ValidationError):
        nb.compress_weights(TinyGatedLM().cuda(), mode=nb.CompressWeightsMode.INT4_SYM, group_size=16,
                            dataset=nb.Dataset(ids), lora_correction=True,
                            advanced_parameters=nb.AdvancedCompressionParameters(
                                lora_correction_params=nb.AdvancedLoraCorrectionParameters(adapter_rank=0)))


def test_lora_correction_after_awq_and_scale_estimation():
    """The adapters are computed from the statistics as they stand after AWQ rescaled the activations and from
    the weight ScaleEstimation's parameters produced (WC/algorithm.py:1150-1195): the combination runs and the
    adapters still lower the output error of the same compression without them."""
    import nncf_b200 as nb

    ids = [i.cuda() for i in calibration_ids(n=8, seq=32)]
    adv = nb.AdvancedCompressionParameters(awq_params=nb.AdvancedAWQParameters(percent_to_apply=0.05),
                                           lora_correction_params=nb.AdvancedLoraCorrectionParameters(adapter_rank=4))
    errs = {}
    with torch.no_grad():
        base = torch.cat([TinyGatedLM().cuda()(i) for i in ids])
        for lora in (False, True):
            cm = nb.compress_weights(TinyGatedLM().cuda(), mode=nb.CompressWeightsMode.INT4_ASYM, group_size=16,
                                     dataset=nb.Dataset(ids), awq=True, scale_estimation=True,
                                     lora_correction=lora or None, advanced_parameters=adv)
            errs[lora] = float((torch.cat([cm(i) for i in ids]) - base).norm() / base.norm())
    assert errs[True] < errs[False], errs
