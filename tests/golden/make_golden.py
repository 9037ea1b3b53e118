"""Generate golden fixtures by running the reference implementation (nncf 3.2.0, torch CPU).

Usage (in a container that has the reference checkout; the fixtures are committed, so this
only needs re-running when cases are added):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <path-to-nncf>/src

Every fixture stores the seeded inputs next to the reference's outputs, so the tests need
neither the reference nor this script at run time.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from cases import (AWQ_CASES, DTYPES, GPTQ_CASES, LORA_CASES, GPTQ_LARGE, GPTQ_SE_CASES, MODES, QUANT_CASES, SE_CASES,  # noqa: E402
                   gptq_large_inputs)


def _setup(ref_src: str):
    sys.path.insert(0, ref_src)
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    import torch  # noqa: F401

    torch.set_num_threads(4)
    # the reference's torch tests disable TF32; irrelevant on CPU, kept for symmetry


def _np(t):
    import torch

    d = t.data if hasattr(t, "data") and not isinstance(t, np.ndarray) else t
    if isinstance(d, torch.Tensor):
        if d.dtype == torch.bfloat16:
            d = d.float()
        return d.detach().cpu().numpy()
    return np.asarray(d)


def _torch_weight(w32: np.ndarray, dtype: str):
    import torch

    t = torch.from_numpy(w32.copy())
    return t.to({"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[dtype])


def _round_to(w32: np.ndarray, dtype: str) -> np.ndarray:
    """Make fp32 values exactly representable in `dtype`."""
    return _torch_weight(w32, dtype).float().numpy()


def make_weight(rng, shape, kind: str) -> np.ndarray:
    if kind == "normal":
        w = rng.normal(0.0, 0.02, size=shape)
    elif kind == "uniform":
        w = rng.uniform(-1.0, 1.0, size=shape)
    elif kind == "positive":
        w = rng.uniform(0.1, 3.0, size=shape)
    elif kind == "negative":
        w = -rng.uniform(0.1, 3.0, size=shape)
    elif kind == "arange":
        w = np.arange(int(np.prod(shape)), dtype=np.float64).reshape(shape) - 7.0
    elif kind == "special":
        w = rng.normal(0.0, 1.0, size=shape)
        flat = w.reshape(shape[0], -1)
        flat[0, :] = 0.0  # all-zero row: eps guard
        if shape[0] > 1:
            flat[1, :] = 0.37  # constant row
        if shape[0] > 2:
            flat[2, :] = np.linspace(-7.5, 7.5, flat.shape[1])  # many exact .5 ties for scale 1
            flat[2, 0] = -8.0
        if shape[0] > 3:
            flat[3, :] = 1e-9 * rng.normal(size=flat.shape[1])  # below eps
        w = flat.reshape(shape)
    else:
        raise ValueError(kind)
    return w.astype(np.float32)




def gen_quant(out: dict):
    from nncf.parameters import CompressWeightsMode
    from nncf.quantization.algorithms.weight_compression import weight_lowering as wl
    from nncf.quantization.algorithms.weight_compression.config import WeightCompressionConfig
    from nncf.quantization.algorithms.weight_compression.parameters import CompressedWeight
    from nncf.tensor import Tensor

    rng = np.random.default_rng(1234)
    names = []
    for name, shape, axis, gs, kind in QUANT_CASES:
        for dtype in DTYPES:
            if dtype != "f32" and kind in ("arange",):
                continue
            w32 = _round_to(make_weight(rng, shape, kind), dtype)
            for mode in MODES:
                cfg = WeightCompressionConfig(CompressWeightsMode(mode), gs)
                wt = Tensor(_torch_weight(w32, dtype))
                if "fp8" in mode:
                    # the reference's E4M3 conversion only runs on its numpy backend (its torch
                    # backend cannot wrap numpy scalars); the weight is cast to fp32 first anyway
                    wt = Tensor(w32.astype(np.float16) if dtype == "f16" else w32.copy())
                cw = wl.compress_weight(wt, axis, cfg)
                key = f"q/{name}/{dtype}/{mode}"
                names.append(key)
                out[f"q/{name}/{dtype}/w"] = w32  # shared by all modes of this case
                out[key + "/meta"] = np.array([axis, gs], dtype=np.int64)
                out[key + "/tensor"] = _np(cw.tensor)
                out[key + "/scale"] = _np(cw.scale)
                if cw.zero_point is not None:
                    out[key + "/zp"] = _np(cw.zero_point)
                # quantize-dequantize through the reference's own entry points
                if cfg.is_integer:
                    dq = wl.integer_quantize_dequantize_weight(wt, cfg, axis)
                else:
                    dq = wl.float_quantize_dequantize_weight(wt, cfg, axis)
                out[key + "/dq"] = _np(dq)
                if cfg.is_integer and len(shape) == 2:
                    for red in ("max_mean", "frobenius"):
                        out[key + f"/err_{red}"] = np.float64(wl.get_integer_quantization_error(wt, axis, cfg, red))
    out["q/index"] = np.array(names)

    # precomputed scale / zero point (already grouped weight, reduction axes omitted)
    pre = []
    for mode in MODES:
        w32 = make_weight(rng, (6, 4, 32), "normal")
        cfg = WeightCompressionConfig(CompressWeightsMode(mode), 32)
        import torch

        base_w = w32.reshape(6, 128).copy() if "fp8" in mode else _torch_weight(w32.reshape(6, 128), "f32")
        base = wl.compress_weight(Tensor(base_w), 1, cfg)
        if "fp8" in mode:
            base.scale = Tensor(torch.from_numpy(base.scale.data))

        s = base.scale.data * torch.from_numpy(rng.uniform(0.7, 1.3, size=(6, 4, 1)).astype(np.float32))
        if mode in ("mxfp4", "mxfp8_e4m3"):
            s = base.scale.data * 2.0
        zp = None
        if cfg.is_asym_mode:
            zp = torch.clamp(base.zero_point.data + torch.from_numpy(rng.integers(-1, 2, size=(6, 4, 1))).int(), 0,
                             2 ** cfg.num_bits - 1)
        if "fp8" in mode:
            pcw = CompressedWeight(None, Tensor(s.numpy()), None)
            cw = wl.compress_weight(Tensor(w32.reshape(6, 128)), 1, cfg, pcw)
        else:
            pcw = CompressedWeight(None, Tensor(s), Tensor(zp) if zp is not None else None)
            cw = wl.compress_weight(Tensor(torch.from_numpy(w32.reshape(6, 128))), 1, cfg, pcw)
        key = f"pre/{mode}"
        pre.append(key)
        out[key + "/w"] = w32.reshape(6, 128)
        out[key + "/scale"] = _np(s)
        if zp is not None:
            out[key + "/zp"] = _np(zp)
        out[key + "/tensor"] = _np(cw.tensor)
    out["pre/index"] = np.array(pre)


def gen_pack(out: dict):
    import torch

    from nncf.torch.quantization.quantize_functions import decompress_asymmetric
    from nncf.torch.quantization.quantize_functions import decompress_symmetric
    from nncf.torch.quantization.quantize_functions import pack_int4
    from nncf.torch.quantization.quantize_functions import pack_uint4

    rng = np.random.default_rng(99)
    u = rng.integers(0, 16, size=(6, 2, 32), dtype=np.uint8)
    i = rng.integers(-8, 8, size=(6, 2, 32), dtype=np.int8)
    out["pack/u4_in"] = u
    out["pack/u4_out"] = pack_uint4(torch.from_numpy(u)).numpy()
    out["pack/i4_in"] = i
    out["pack/i4_out"] = pack_int4(torch.from_numpy(i)).numpy()
    scale = torch.from_numpy(rng.normal(0, 0.01, size=(6, 2, 1)).astype(np.float32)).half()
    zp = torch.from_numpy(rng.integers(0, 16, size=(6, 2, 1), dtype=np.uint8))
    out["pack/scale_f16"] = scale.numpy()
    out["pack/zp"] = zp.numpy()
    out["pack/dq_asym_f16"] = decompress_asymmetric(torch.from_numpy(u), scale, zp).numpy()
    out["pack/dq_sym_f16"] = decompress_symmetric(torch.from_numpy(i), scale).numpy()
    u8 = rng.integers(0, 256, size=(6, 64), dtype=np.uint8)
    i8 = rng.integers(-128, 128, size=(6, 64), dtype=np.int8)
    s8 = torch.from_numpy(rng.normal(0, 0.01, size=(6, 1)).astype(np.float32)).half()
    z8 = torch.from_numpy(rng.integers(0, 256, size=(6, 1), dtype=np.uint8))
    out["pack/u8_in"], out["pack/i8_in"] = u8, i8
    out["pack/scale8_f16"], out["pack/zp8"] = s8.numpy(), z8.numpy()
    out["pack/dq8_asym_f16"] = decompress_asymmetric(torch.from_numpy(u8), s8, z8).numpy()
    out["pack/dq8_sym_f16"] = decompress_symmetric(torch.from_numpy(i8), s8).numpy()


def _stats(mean_list, shapes):
    from nncf.common.tensor_statistics.statistics import WCTensorStatistic
    from nncf.tensor import Tensor

    import torch

    return WCTensorStatistic([Tensor(torch.from_numpy(m)) for m in mean_list], [tuple(s) for s in shapes])


def gen_stats(out: dict):
    import torch

    from nncf.common.tensor_statistics.collectors import MaxVarianceReducer
    from nncf.common.tensor_statistics.collectors import MeanAbsMaxReducer
    from nncf.common.tensor_statistics.collectors import MeanReducer
    from nncf.common.tensor_statistics.collectors import MeanVarianceReducer
    from nncf.quantization.algorithms.weight_compression.activation_stats import process_stats
    from nncf.tensor import Tensor

    rng = np.random.default_rng(7)
    # process_stats: 10 samples, hidden 12, different token counts
    means = [rng.normal(size=(12,)).astype(np.float32) for _ in range(10)]
    shapes = [(1, int(t), 12) for t in rng.integers(3, 40, size=10)]
    for subset in (3, 4, 10, 32):
        s, X = process_stats(_stats(means, shapes), subset)
        out[f"stats/process/{subset}/s"] = _np(s)
        out[f"stats/process/{subset}/X"] = _np(X)
    out["stats/process/means"] = np.stack(means)
    out["stats/process/shapes"] = np.array(shapes, dtype=np.int64)

    # reducers on an activation [2, 37, 48]
    for dtype in DTYPES:
        x32 = _round_to(rng.normal(0.0, 1.5, size=(2, 37, 48)).astype(np.float32), dtype)
        xt = Tensor(_torch_weight(x32, dtype))
        key = f"stats/reduce/{dtype}"
        out[key + "/x"] = x32
        out[key + "/mean"] = _np(MeanReducer(axes=(0, 1))._reduce_out_of_place([xt])[0])
        out[key + "/mean_var"] = _np(MeanVarianceReducer(axes=(0, 1))._reduce_out_of_place([xt])[0])
        out[key + "/max_var"] = _np(MaxVarianceReducer(axes=(0, 1))._reduce_out_of_place([xt])[0])
        out[key + "/mean_abs_max"] = _np(MeanAbsMaxReducer(axes=(0, 1))._reduce_out_of_place([xt])[0])
        xf = torch.from_numpy(x32)
        out[key + "/sumsq"] = np.float64(float((xf.double() ** 2).sum()))




def gen_scale_estimation(out: dict):
    import torch

    from nncf.parameters import CompressWeightsMode
    from nncf.quantization.algorithms.weight_compression.config import WeightCompressionConfig
    from nncf.quantization.algorithms.weight_compression.scale_estimation import ScaleEstimation
    from nncf.tensor import Tensor

    rng = np.random.default_rng(42)
    names = []
    for name, o, i, gs, n, mode, ist, sst, axis, pen in SE_CASES:
        w = rng.normal(0, 0.05, size=(o, i)).astype(np.float32)
        if axis == 0:
            w = np.ascontiguousarray(w.T)
        means = [np.abs(rng.normal(0, 1.0, size=(i,))).astype(np.float32) * (1 + 9 * (rng.random(i) < 0.05)) for _ in
                 range(n)]
        means = [m.astype(np.float32) * rng.choice([-1.0, 1.0], size=i).astype(np.float32) for m in means]
        shapes = [(1, 16, i)] * n
        cfg = WeightCompressionConfig(CompressWeightsMode(mode), gs)
        scale, zp = ScaleEstimation.calculate_quantization_params(
            _stats(means, shapes), Tensor(torch.from_numpy(w)), (axis,), cfg, -1, 32, ist, sst, pen)
        key = f"se/{name}"
        names.append(key)
        out[key + "/w"] = w
        out[key + "/means"] = np.stack(means)
        out[key + "/scale"] = _np(scale)
        if zp is not None:
            out[key + "/zp"] = _np(zp)
    out["se/index"] = np.array(names)




def gen_awq(out: dict):
    import torch

    from nncf.parameters import CompressWeightsMode
    from nncf.quantization.algorithms.weight_compression.awq import AWQ
    from nncf.quantization.algorithms.weight_compression.config import WeightCompressionConfig
    from nncf.tensor import Tensor

    rng = np.random.default_rng(4242)
    names = []
    for name, o, i, gs, n, mode, pct, steps, with_prev in AWQ_CASES:
        w = rng.normal(0, 0.05, size=(o, i)).astype(np.float32)
        means = []
        outl = rng.random(i) < 0.04
        for _ in range(n):
            m = rng.normal(0, 1.0, size=(i,)) * (1 + 19 * outl)
            means.append(m.astype(np.float32))
        shapes = [(1, 16, i)] * n
        algo = AWQ(subset_size=32, percent_to_apply=pct, steps=steps)
        cfg = WeightCompressionConfig(CompressWeightsMode(mode), gs)
        wp = SimpleNamespace(compression_config=cfg, reduction_axes=(1,))
        prev_w = prev_stats = None
        key = f"awq/{name}"
        if with_prev:
            # merge node: Linear(hid -> i) whose weight is [i, hid]; large enough to trigger the fp16 clamp
            hid = 40
            pw = (rng.normal(0, 30.0, size=(i, hid))).astype(np.float32)
            pmeans = [rng.normal(0, 40.0, size=(hid,)).astype(np.float32) for _ in range(n)]
            prev_w = Tensor(torch.from_numpy(pw))
            prev_stats = _stats(pmeans, [(1, 16, hid)] * n)
            out[key + "/prev_w"] = pw
            out[key + "/prev_means"] = np.stack(pmeans)
        scale = algo._data_aware_step(wp, Tensor(torch.from_numpy(w)), _stats(means, shapes), -1, prev_w, prev_stats)
        names.append(key)
        out[key + "/w"] = w
        out[key + "/means"] = np.stack(means)
        out[key + "/scale"] = _np(scale)
        out[key + "/meta"] = np.array([gs, steps], dtype=np.int64)
        out[key + "/pct"] = np.float64(pct)
        out[key + "/mode"] = np.array(mode)
    out["awq/index"] = np.array(names)
    w = rng.normal(0, 0.05, size=(16, 48)).astype(np.float32)
    out["awq/data_free/w"] = w
    out["awq/data_free/scale"] = _np(AWQ()._data_free_step(Tensor(torch.from_numpy(w)), axis=0))




def gen_gptq_se(out: dict):
    """GPTQ with scale_estimation=True (the reference's _quantize_weights slices the inputs per group)."""
    gen_gptq(out, cases=GPTQ_SE_CASES, prefix="gptq_se", scale_estimation=True)


def gen_gptq(out: dict, cases=None, prefix="gptq", scale_estimation=False):
    import torch

    from nncf.parameters import CompressWeightsMode
    from nncf.quantization.algorithms.weight_compression.config import WeightCompressionConfig
    from nncf.quantization.algorithms.weight_compression.gptq import GPTQ
    from nncf.tensor import Tensor

    MM = object()
    be = SimpleNamespace(matmul_metatypes=[MM], convolution_metatypes=[])
    node = SimpleNamespace(
        metatype=MM,
        node_name="mm",
        layer_attributes=SimpleNamespace(input_attributes={"transpose": False},
                                         constant_attributes={1: {"transpose": True}}),
    )
    rng = np.random.default_rng(0)
    names = []
    for name, o, C, gs, block, mode, damp, n_in, tokens, xdt in (cases if cases is not None else GPTQ_CASES):
        w = rng.normal(0, 0.05, size=(o, C)).astype(np.float32)
        base = rng.normal(0, 1.0, size=(C, C)) / np.sqrt(C)
        xs = []
        for _ in range(n_in):
            x = rng.normal(0, 1.0, size=(1, tokens, C)) @ (np.eye(C) + 0.5 * base)
            xs.append(_round_to(x.astype(np.float32), xdt))
        if name == "int4_sym_g32_b32":
            for x in xs:
                x[..., 5] = 0.0  # dead column
        g = GPTQ(damp_percent=damp, block_size=block, subset_size=n_in, scale_estimation=scale_estimation)
        g._backend_entity = be
        inputs = [Tensor(_torch_weight(x, xdt)) for x in xs]
        H = g._calculate_hessian(node, inputs)
        cfg = WeightCompressionConfig(CompressWeightsMode(mode), gs)
        wp = SimpleNamespace(node_with_weight=node, weight_port_id=1, compression_config=cfg, reduction_axes=(1,))
        Hc = Tensor(H.data[0].clone())
        q, s, z = g._quantize_weights(wp, Hc, Tensor(torch.from_numpy(w.copy())), inputs)
        key = f"{prefix}/{name}"
        names.append(key)
        out[key + "/w"] = w
        out[key + "/x"] = np.stack(xs)
        out[key + "/xdtype"] = np.array(xdt)
        out[key + "/H"] = _np(H.data[0])
        out[key + "/q"] = _np(q)
        out[key + "/scale"] = _np(s)
        if z is not None:
            out[key + "/zp"] = _np(z)
        out[key + "/meta"] = np.array([gs, block], dtype=np.int64)
        out[key + "/damp"] = np.float64(damp)
        out[key + "/mode"] = np.array(mode)
    out[f"{prefix}/index"] = np.array(names)


def gen_gptq_large(out: dict):
    """GPTQ at 512 x 1024, group 128, block 128, damping 0.01 by the reference's TORCH backend (the oracle of
    record), INT4_SYM and INT4_ASYM on the same weight and activations; plus the same problem on the reference's
    numpy backend, whose distance from the torch result is the reference's own self-noise floor."""
    import torch

    from nncf.parameters import CompressWeightsMode
    from nncf.quantization.algorithms.weight_compression.config import WeightCompressionConfig
    from nncf.quantization.algorithms.weight_compression.gptq import GPTQ
    from nncf.tensor import Tensor
    from nncf.tensor import functions as fns

    MM = object()
    be = SimpleNamespace(matmul_metatypes=[MM], convolution_metatypes=[])
    node = SimpleNamespace(metatype=MM, node_name="mm",
                           layer_attributes=SimpleNamespace(input_attributes={"transpose": False},
                                                            constant_attributes={1: {"transpose": True}}))
    c = GPTQ_LARGE
    w, xs = gptq_large_inputs()
    iu = np.triu_indices(c["cols"])

    def run(backend: str, mode: str):
        g = GPTQ(damp_percent=c["damp"], block_size=c["block"], subset_size=c["n_inputs"])
        g._backend_entity = be
        if backend == "torch":
            inputs = [Tensor(torch.from_numpy(x).to(torch.bfloat16)) for x in xs]
            wt = Tensor(torch.from_numpy(w.copy()))
        else:
            inputs = [Tensor(x.copy()) for x in xs]
            wt = Tensor(w.copy())
        H = g._calculate_hessian(node, inputs)
        Hc = Tensor(H.data[0].clone() if backend == "torch" else H.data[0].copy())
        cfg = WeightCompressionConfig(CompressWeightsMode(mode), c["group_size"])
        wp = SimpleNamespace(node_with_weight=node, weight_port_id=1, compression_config=cfg, reduction_axes=(1,))
        q, s, z = g._quantize_weights(wp, Hc, wt, inputs)
        return _np(H.data[0]), _np(q), _np(s), (None if z is None else _np(z))

    names = []
    for mode in ("int4_sym", "int4_asym"):
        H, q, s, z = run("torch", mode)
        _, qn, _, _ = run("numpy", mode)
        key = f"gptq_large/{mode}"
        names.append(key)
        # codes: q = (code - zp) * scale exactly (WC/weight_lowering.py:428-448), so integer codes + parameters
        # reproduce the reference's dequantised weight bit for bit
        sg = np.repeat(s.reshape(c["rows"], -1), c["group_size"], axis=1)
        zg = 0 if z is None else np.repeat(z.reshape(c["rows"], -1), c["group_size"], axis=1).astype(np.float32)
        codes = np.rint(q / sg + zg)
        assert np.array_equal(((codes - zg) * sg).astype(np.float32), q)
        out[key + "/codes"] = codes.astype(np.int8 if z is None else np.uint8)
        out[key + "/scale"] = s
        if z is not None:
            out[key + "/zp"] = z
        out[key + "/numpy_backend_rel_fro"] = np.float64(np.linalg.norm(qn - q) / np.linalg.norm(q))
        out[key + "/numpy_backend_diff_frac"] = np.float64(np.mean(qn != q))
        if "gptq_large/H_triu" not in out:
            out["gptq_large/H_triu"] = H[iu]
            # the factor the reference's sweep used: its three calls (WC/gptq.py:269-295) on this Hessian
            Ht = Tensor(torch.from_numpy(H.copy()))
            damp = c["damp"] * fns.mean(fns.diag(Ht))
            d = fns.arange(c["cols"], backend=Ht.backend, device=Ht.device)
            Ht[d, d] += damp
            U = fns.linalg.cholesky(fns.linalg.cholesky_inverse(fns.linalg.cholesky(Ht)), upper=True)
            out["gptq_large/U_triu"] = _np(U)[iu]
    out["gptq_large/index"] = np.array(names)
    out["gptq_large/params"] = np.array([c[k] for k in ("rows", "cols", "group_size", "block", "n_inputs", "tokens", "seed")],
                                        dtype=np.int64)
    out["gptq_large/damp"] = np.float64(c["damp"])


def gen_layerwise(out: dict):
    """Model-level GPTQ on a toy decoder, layer by layer: the reference's own schedule
    (quantization/algorithms/layerwise/scheduler.py:92, on the graph the reference traces from the torch model)
    decides which target layers share a step; every step's inputs are collected from the model as it stands at
    that point (earlier steps' weights already replaced by their quantised values, the contract of
    layerwise/openvino_iterator.py and WC/gptq.py:157), and the reference's GPTQ computes the Hessian and the
    quantised weight of each layer (WC/gptq.py:201, :230).  Only the collection of a step's inputs is done here,
    with forward hooks on the torch model, because the reference ships that piece for OpenVINO models only."""
    import torch

    import nncf
    from models import LAYERWISE, TinyGatedLM, layerwise_ids
    from nncf.parameters import CompressWeightsMode
    from nncf.quantization.algorithms.layerwise.scheduler import LayerwiseScheduler
    from nncf.quantization.algorithms.weight_compression.config import WeightCompressionConfig
    from nncf.quantization.algorithms.weight_compression.gptq import GPTQ
    from nncf.tensor import Tensor
    from nncf.torch.graph.operator_metatypes import PTLinearMetatype

    c = LAYERWISE
    ids = layerwise_ids()
    names = []
    for mode in c["modes"]:
        torch.manual_seed(0)
        model = TinyGatedLM(**c["model"]).eval()
        wrapped = nncf.torch.wrap_model(model, example_input=ids[0], trace_parameters=True)
        graph = wrapped.get_graph()
        linear = [n for n in graph.get_all_nodes() if n.metatype is PTLinearMetatype]
        weight_of = {}
        for n in linear:
            const = [p for p in graph.get_previous_nodes(n) if p.node_name.endswith(".weight")]
            weight_of[n.node_name] = const[0].node_name
        targets = [n for n in linear if weight_of[n.node_name] != "head.weight"]
        steps = LayerwiseScheduler().schedule(graph, targets, True)
        modules = dict(model.named_modules())
        be = SimpleNamespace(matmul_metatypes=[PTLinearMetatype], convolution_metatypes=[])
        g = GPTQ(damp_percent=c["damp"], block_size=c["block"], subset_size=len(ids))
        g._backend_entity = be
        cfg = WeightCompressionConfig(CompressWeightsMode(mode), c["group_size"])
        key = f"layerwise/{mode}"
        names.append(key)
        step_names = []
        for step in steps:
            mods = [weight_of[n.node_name][: -len(".weight")] for n in step.target_node_map]
            step_names.append(",".join(mods))
            seen = {m: [] for m in mods}
            handles = [modules[m].register_forward_pre_hook(lambda mod, args, m=m: seen[m].append(args[0].detach().clone()))
                       for m in mods]
            with torch.no_grad():
                for item in ids:
                    model(item)
            for h in handles:
                h.remove()
            for node, m in zip(step.target_node_map, mods):
                node_ns = SimpleNamespace(metatype=PTLinearMetatype, node_name=node.node_name,
                                          layer_attributes=SimpleNamespace(input_attributes={"transpose": False},
                                                                           constant_attributes={1: {"transpose": True}}))
                inputs = [Tensor(x) for x in seen[m]]
                H = g._calculate_hessian(node_ns, inputs)
                wp = SimpleNamespace(node_with_weight=node_ns, weight_port_id=1, compression_config=cfg,
                                     reduction_axes=(1,))
                w = modules[m].weight.detach().clone()
                q, s, z = g._quantize_weights(wp, Tensor(H.data[0].clone()), Tensor(w), inputs)
                with torch.no_grad():
                    modules[m].weight.copy_(q.data)
                out[f"{key}/{m}/weight"] = _np(q)
                out[f"{key}/{m}/scale"] = _np(s)
                if z is not None:
                    out[f"{key}/{m}/zp"] = _np(z)
        out[key + "/steps"] = np.array(step_names)
        with torch.no_grad():
            out[key + "/logits"] = _np(model(ids[0]))
    out["layerwise/index"] = np.array(names)


def gen_lora(out: dict):
    """LoRA correction (WC/lora_correction.py:139-271) on seeded weights and activation statistics: the reference's
    compress_weight, its dequantisation and its adapters.  Stored: inputs, the dequantised weight the adapters
    correct, both adapters, and the activation-weighted noise before and after."""
    import torch

    from nncf.parameters import CompressWeightsMode
    from nncf.quantization.advanced_parameters import AdvancedLoraCorrectionParameters
    from nncf.quantization.algorithms.weight_compression.activation_stats import process_stats
    from nncf.quantization.algorithms.weight_compression.config import WeightCompressionConfig
    from nncf.quantization.algorithms.weight_compression.lora_correction import LoraCorrectionAlgorithm
    from nncf.quantization.algorithms.weight_compression.weight_lowering import (compress_weight,
                                                                                   do_float_dequantization,
                                                                                   do_integer_dequantization)
    from nncf.tensor import Tensor

    rng = np.random.default_rng(777)
    names = []
    for name, o, h, gs, n, mode, rank, iters, reg in LORA_CASES:
        w = rng.normal(0, 0.05, size=(o, h)).astype(np.float32)
        outl = rng.random(h) < 0.06
        means = [(rng.normal(0, 1.0, size=(h,)) * (1 + 9 * outl)).astype(np.float32) for _ in range(n)]
        shapes = [(1, int(rng.integers(4, 40)), h) for _ in range(n)]
        cfg = WeightCompressionConfig(CompressWeightsMode(mode), gs)
        cw = compress_weight(Tensor(torch.from_numpy(w.copy())), (1,), cfg)
        axis = 1 if gs != -1 else -1
        fq = do_float_dequantization(cw, axis) if mode == "nf4" else do_integer_dequantization(cw, axis)
        params = AdvancedLoraCorrectionParameters(adapter_rank=rank, num_iterations=iters, apply_regularization=reg)
        a, b, _ = LoraCorrectionAlgorithm.calculate_low_rank_matrices(Tensor(torch.from_numpy(w.copy())), cw, cfg, (1,),
                                                                      params, _stats(means, shapes))
        key = f"lora/{name}"
        names.append(key)
        out[key + "/w"] = w
        out[key + "/fq"] = _np(fq).reshape(o, h)
        out[key + "/means"] = np.stack(means)
        out[key + "/tokens"] = np.array([s[1] for s in shapes], dtype=np.int64)
        out[key + "/lora_A"] = _np(a)
        out[key + "/lora_B"] = _np(b)
        _, X = process_stats(_stats(means, shapes), params.subset_size)
        X = _np(X).T.astype(np.float64)                       # [SS, H]
        res = (w - out[key + "/fq"]).T.astype(np.float64)    # [H, O]
        out[key + "/noise_before"] = np.float64(np.abs(X @ res).mean())
        out[key + "/noise_after"] = np.float64(np.abs(X @ res - X @ _np(a).T.astype(np.float64) @ _np(b).T.astype(np.float64)).mean())
    out["lora/index"] = np.array(names)


def gen_config1(out: dict):
    """SHA-256 digests of every tensor of the state dict the reference's ``nncf.compress_weights`` produces for
    8 stacked Linear(4096 -> 4096) fp32 layers (INT4_SYM, group 128, ratio 1.0, CPU): a few hundred bytes that
    pin 8 x 16.8 M codes, their fp16 scales and the INT8_ASYM backup layer."""
    import hashlib

    import nncf
    from models import StackedLinear

    model = StackedLinear(8, 4096).eval()
    cm = nncf.compress_weights(model, mode=nncf.CompressWeightsMode.INT4_SYM, group_size=128, ratio=1.0,
                               dataset=nncf.Dataset([model.example_input()]))
    names, digests, metas = [], [], []
    for k, v in cm.state_dict().items():
        a = np.ascontiguousarray(_np(v))
        names.append(k)
        digests.append(hashlib.sha256(a.tobytes()).hexdigest())
        metas.append(f"{a.dtype}{list(a.shape)}")
    out["config1/keys"] = np.array(names)
    out["config1/sha256"] = np.array(digests)
    out["config1/meta"] = np.array(metas)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("NNCF_REFERENCE_SRC"), required="NNCF_REFERENCE_SRC" not in os.environ,
                    help="path to the src/ directory of an nncf 3.2.0 checkout (or set NNCF_REFERENCE_SRC)")
    ap.add_argument("groups", nargs="*", help="fixture groups to regenerate (default: all)")
    args = ap.parse_args()
    _setup(args.reference)
    groups = {
        "quant": gen_quant,
        "pack": gen_pack,
        "stats": gen_stats,
        "scale_estimation": gen_scale_estimation,
        "awq": gen_awq,
        "gptq": gen_gptq,
        "gptq_se": gen_gptq_se,
        "gptq_large": gen_gptq_large,
        "config1": gen_config1,
        "layerwise": gen_layerwise,
        "lora": gen_lora,
        "api": gen_api,
    }
    only = [a for a in sys.argv[1:] if a in groups]
    if only:
        groups = {k: v for k, v in groups.items() if k in only}
    for fname, fn in groups.items():
        data: dict = {}
        fn(data)
        path = HERE / f"{fname}.npz"
        np.savez_compressed(path, **{k.replace("/", "|"): v for k, v in data.items()})
        print(f"{path.name}: {len(data)} arrays, {path.stat().st_size / 1024:.0f} KiB")



def gen_api(out: dict):
    """nncf.compress_weights end to end on a toy Llama-like torch model (CPU): packed weights and
    decompressor buffers per layer."""
    import torch

    import nncf
    from models import API_CASES, TinyGatedLM, calibration_ids

    names = []
    for name, kwargs, use_ds in API_CASES:
        model = TinyGatedLM()
        ids = calibration_ids()
        kw = dict(kwargs)
        kw["mode"] = nncf.CompressWeightsMode(kw["mode"])
        if "sensitivity_metric" in kw:
            kw["sensitivity_metric"] = nncf.SensitivityMetric(kw["sensitivity_metric"])
        if kw.get("awq"):
            kw["advanced_parameters"] = nncf.AdvancedCompressionParameters(
                awq_params=nncf.AdvancedAWQParameters(percent_to_apply=0.05))
        ds = nncf.Dataset(ids)
        # the torch backend traces the model with a dataset item even when the algorithm is data-free
        cm = nncf.compress_weights(model, dataset=ds if use_ds else None, **kw) if use_ds else \
            nncf.compress_weights(nncf.torch.wrap_model(model, example_input=ids[0], trace_parameters=True), **kw)
        sd = cm.state_dict()
        key = f"api/{name}"
        names.append(key)
        for k, v in sd.items():
            out[f"{key}/{k}"] = _np(v)
        out[key + "/keys"] = np.array(list(sd.keys()))
        with torch.no_grad():
            out[key + "/logits"] = _np(cm(ids[0]))
    out["api/index"] = np.array(names)

if __name__ == "__main__":
    main()
