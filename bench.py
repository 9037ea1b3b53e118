"""Benchmark of the weight-compression hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

A step is one pass of the hot path over ONE synthetic Llama-3-8B-shaped bf16 weight set
(8.03e9 parameters, 16.06 GB): INT4_SYM group 128 on the 224 decoder matrices and INT8_ASYM per
channel on the embedding and lm_head, which is what ``compress_weights(mode=INT4_SYM,
group_size=128, ratio=1.0)`` does with its default backup rule.  Every weight is N(0, 0.02^2) from
a seed derived from the configuration's seed 1 and the tensor's index.

N = 1: `value` is source-weight GB/s with inputs resident in HBM (CUDA-graph replay of the two
batched launches, CUDA events).  N > 1 (one process per GPU, torchrun): the SAME model is split over
the ranks by source bytes and every packed result is collected on rank 0 over NCCL while the ranks
are still compressing; `value` is the model's source bytes over the time of compress + gather (max
over ranks), i.e. strong scaling; `multi_gpu` gives the halves on their own.

The one JSON line rank 0 prints also carries: `e2e`, the same metric through the host-buffer API
(pinned host weights -> device -> packed results back in host memory, copies inside the timed region;
for N > 1 the model split over the ranks' PCIe links); `roofline` of the dominant kernel; `parity`, a
check of what the timed passes wrote against the CPU oracle; `gptq`, the second half of the metric
(GPTQ seconds per 8B model: calibration through a random-init Llama-3-8B-architecture model);
`cpu_baseline`, the reference's own CPU implementation on 1/32 of the workload (N = 1 only).
`--impl reference` times only that CPU arm.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "source_weight_GBps_compressed_int4_g128"
UNIT = "GB/s"
WORKLOAD = ("llama3-8b-shaped bf16 weight set (226 tensors, 8.03e9 params, 16.06 GB): INT4_SYM g128 on 224 decoder "
            "matrices + INT8_ASYM per-channel backup on embed_tokens and lm_head")


def _peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_sample(threads: int, steps: int, warmup: int):
    """The reference's CPU path with all host threads on 1/32 of the workload: one decoder layer's 7 matrices
    (INT4_SYM g128) and 1/32 of the embedding and lm_head rows (INT8_ASYM per channel), compress + pack per
    weight as its torch backend does.  Runs the unmodified reference package when a copy of it is present
    (oracle/_ref, made by oracle/make_ref.py; kind "reference"), else the restatement of its torch op chain
    kept under oracle/ (kind "port").  Returns (GB/s, seconds per step, source bytes, kind, note)."""
    kind, note, step_fn = "port", "", None
    try:
        from oracle import ref_loader

        ref_loader.load()
        step_fn = ref_loader.compress_and_pack
        kind = "reference"
        note = ("unmodified reference (nncf 3.2.0) from oracle/_ref: weight_lowering.compress_weight + "
                "decompressor.pack_weight per weight, torch CPU backend")
    except Exception as exc:  # noqa: BLE001 - any import problem falls back to the port, and the line says so
        from oracle import wc_oracle_torch as T

        step_fn = T.compress_and_pack
        note = f"port of the reference's torch op chain (oracle/wc_oracle_torch.py); oracle/_ref unusable: {exc}"
    torch.set_num_threads(threads)
    gen = torch.Generator().manual_seed(1)
    shapes = [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (14336, 4096), (14336, 4096), (4096, 14336)]
    ws = [(torch.randn(s, generator=gen) * 0.02).to(torch.bfloat16) for s in shapes]
    emb = [(torch.randn(128256 // 32, 4096, generator=gen) * 0.02).to(torch.bfloat16) for _ in range(2)]
    nbytes = sum(w.numel() * 2 for w in ws + emb)

    def step():
        for w in ws:
            step_fn(w, "int4_sym", 128)
        for w in emb:
            step_fn(w, "int8_asym", -1)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return nbytes / dt / 1e9, dt, nbytes, kind, note


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    threads = host_threads()
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    gbs, dt, nbytes, kind, note = cpu_reference_sample(threads, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(gbs, 4), "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": "each step is 1/32 of the workload (a rate on the same tensor mix)"},
        "cpu_baseline": {"value": round(gbs, 4), "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"1 decoder layer (7 matrices) INT4_SYM g128 + 1/32 of embed/lm_head rows INT8_ASYM, "
                                   f"{nbytes / 1e6:.0f} MB source per step, compress + pack; {note}"},
        "e2e": {"value": round(gbs, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_gptq_workload(args, device):
    """GPTQ kernels one by one on Llama-3-8B shapes (the model-level run is `run_gptq_model`).  Measures the two kernels that make up
    GPTQ on Llama-3-8B shapes - Hessian accumulation (tcgen05) on bf16 activations and the blocked sweep
    (+ Cholesky steps by torch.linalg) - and combines them into a per-model figure for 128 x 2048 calibration
    tokens: per layer 4 distinct Hessians (q/k/v share, o, gate/up share, down) and 7 sweeps."""
    from types import SimpleNamespace

    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig
    from nncf_b200.gptq import GPTQ

    tokens_meas = 8192 if args.profile_case else 32768      # measured per call; scaled to 262144 by token count
    total_tokens = 128 * 2048
    g = GPTQ(damp_percent=0.01, block_size=128, subset_size=128)
    out = {"metric": "gptq_seconds_per_8b_model", "unit": "s", "higher_is_better": False, "n_gpus": 1,
           "data": "synthetic", "dtype": "bf16 products, fp32 accumulate",
           "config": {"workload": "GPTQ INT4_SYM g128, block 128, damp 0.01 on Llama-3-8B shapes; Hessian timed on "
                                  f"{tokens_meas} tokens per call and scaled to 128 x 2048 tokens"}}
    peak_tf = 1657.8
    try:
        peak_tf = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops"])
    except Exception:
        pass
    hess = {}
    for C in (4096, 14336):
        x = (torch.randn(tokens_meas, C, device=device) * 0.5).to(torch.bfloat16)
        H = torch.zeros(C, C, device=device)
        n = 0
        for _ in range(2):
            n = g.accumulate_hessian(H, x, n, 1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 1 if args.profile_case else 5
        e0.record()
        for _ in range(reps):
            n = g.accumulate_hessian(H, x, n, 1)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        flops = 2.0 * tokens_meas * C * C
        # the kernel computes the 128 x 256 tiles that touch the upper triangle and mirrors the rest
        tm, tn = (C + 127) // 128, (C + 255) // 256
        tiles = sum(tn - mi // 2 for mi in range(tm))
        computed = 2.0 * tokens_meas * tiles * 128 * 256
        hess[C] = {"ms": round(ms, 3), "tokens": tokens_meas,
                   "TFLOPs_computed": round(computed / ms / 1e9, 1),
                   "frac_of_measured_bf16_peak_computed": round(computed / ms / 1e9 / peak_tf, 4),
                   "TFLOPs_full_square": round(flops / ms / 1e9, 1),
                   "frac_of_measured_bf16_peak": round(flops / ms / 1e9 / peak_tf, 4),
                   "note": "computed = the upper-triangle tiles the kernel multiplies; full_square = the C x C product "
                           "the reference computes (includes the time of the mirror kernel)"}
        del x, H
    from nncf_b200 import _lib

    _lib.check(_lib.lib.nncfb_hessian_status(None))
    sweeps, hinv_ms = {}, {}
    cfg = SimpleNamespace(compression_config=WeightCompressionConfig(CompressWeightsMode.INT4_SYM, 128),
                          reduction_axes=(1,))

    def wall(fn):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        r = fn()
        torch.cuda.synchronize()
        return r, (time.perf_counter() - t0) * 1e3

    for C in ((4096,) if args.profile_case else (4096, 14336)):
        x = torch.randn(2 * C, C, device=device)
        H0 = (2.0 / 2) * (x.T @ x)
        del x
        for name, o in {4096: {"q_proj": 4096, "k_proj": 1024, "gate_proj": 14336}, 14336: {"down_proj": 4096}}[C].items():
            if args.profile_case and name != "q_proj":
                continue
            w0 = torch.randn(o, C, device=device) * 0.02
            best_h, best_s = 1e30, 1e30
            for _ in range(2):
                H, w = H0.clone(), w0.clone()
                hinv, th = wall(lambda: g.prepare_hessian_inverse(H, w))
                _, ts = wall(lambda: g._quantize_weights(cfg, H, w, hinv=hinv))
                best_h, best_s = min(best_h, th), min(best_s, ts)
            sweeps[name] = round(best_s, 2)
            hinv_ms[C] = round(best_h, 2)
            del w0, H, w, hinv
        del H0
    out["hessian"] = hess
    out["sweep_ms"] = sweeps
    out["hessian_inverse_factor_ms"] = hinv_ms
    if not args.profile_case:
        scale = total_tokens / tokens_meas
        per_layer_h = (3 * hess[4096]["ms"] + hess[14336]["ms"]) * scale
        per_layer_s = 2 * sweeps["q_proj"] + 2 * sweeps["k_proj"] + 2 * sweeps["gate_proj"] + sweeps["down_proj"]
        per_layer_f = 3 * hinv_ms[4096] + hinv_ms[14336]  # q/k/v and gate/up share one factorisation each
        out["value"] = round(32 * (per_layer_h + per_layer_s + per_layer_f) / 1e3, 2)
        out["breakdown_s"] = {"hessians": round(32 * per_layer_h / 1e3, 2), "sweeps": round(32 * per_layer_s / 1e3, 2),
                              "cholesky_steps_torch_linalg": round(32 * per_layer_f / 1e3, 2),
                              "excluded": "calibration forward passes of the model (not part of the hot path)"}
    if 14336 in hess:
        h = hess[14336]
        out["roofline"] = {"bound": "tensor", "kernel": "tc_tn_kernel<4 stages, Hessian> (tcgen05 / TMEM / TMA), C = 14336",
                           "achieved": h["TFLOPs_computed"], "peak": peak_tf, "unit": "TFLOP/s",
                           "frac": h["frac_of_measured_bf16_peak_computed"], "traffic": None,
                           "peak_source": "measured (MEASURED_PEAKS.json bf16_tflops, burst)"}
    print(json.dumps(out), flush=True)


def run_api_workload(args, device):
    """The model-level API (`nncf_b200.compress_weights`) on a random-init Llama of 1.1 B parameters
    (hidden 2048, 16 layers, bf16; Hugging Face `LlamaForCausalLM`), 16 calibration sequences of 512 tokens:
    wall time of the whole call - tracing, statistics, algorithms, kernels, installing the decompressors."""
    import transformers

    import nncf_b200 as nb

    cfg = transformers.LlamaConfig(vocab_size=32000, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                                   num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=2048)
    gen = torch.Generator().manual_seed(0)
    ids = [torch.randint(0, 32000, (1, 512), generator=gen).to(device) for _ in range(16)]
    cases = (("int4_sym_data_free", {}), ("awq_scale_estimation", {"awq": True, "scale_estimation": True}),
             ("gptq", {"gptq": True}), ("gptq_scale_estimation", {"gptq": True, "scale_estimation": True}))
    seconds = {}
    n_params = 0
    for name, kw in cases:
        torch.manual_seed(0)
        with torch.device(device):
            model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
        n_params = sum(p.numel() for p in model.parameters())
        if kw:
            kw = dict(kw, dataset=nb.Dataset(ids))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        model = nb.compress_weights(model, mode=nb.CompressWeightsMode.INT4_SYM, group_size=128, **kw)
        torch.cuda.synchronize()
        seconds[name] = round(time.perf_counter() - t0, 3)
        with torch.no_grad():
            assert bool(torch.isfinite(model(ids[0]).logits).all()), name
        del model
        torch.cuda.empty_cache()
    print(json.dumps({"metric": "compress_weights_api_seconds", "unit": "s", "higher_is_better": False, "n_gpus": 1,
                      "data": "synthetic", "dtype": "bf16 weights",
                      "config": {"workload": f"LlamaForCausalLM, {n_params / 1e9:.2f} B parameters, random init, INT4_SYM "
                                             "g128, 16 x 512 calibration tokens"},
                      "seconds": seconds, "value": seconds["int4_sym_data_free"]}), flush=True)


def run_decompress_workload(args, device):
    """Decompression of stored weights (what every forward pass of a compressed model runs per layer): the seven
    matrices of `--layers` Llama-3-8B decoder layers, INT4_SYM / INT4_ASYM g128 or INT8_ASYM per channel with fp16
    scales as stored, decompressed to bf16 by one `nncfb_decompress` call per matrix.  GB/s of produced weights and
    the fraction of the measured HBM peak in algorithmic bytes (codes + parameters read, bf16 weights written)."""
    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig, _lib
    from nncf_b200.pipeline import CompressionPlan

    mode = CompressWeightsMode(args.decompress_mode)
    gs = -1 if mode == CompressWeightsMode.INT8_ASYM else 128
    cfg = WeightCompressionConfig(mode, gs)
    shapes = [("q_proj", (4096, 4096)), ("k_proj", (1024, 4096)), ("v_proj", (1024, 4096)), ("o_proj", (4096, 4096)),
              ("gate_proj", (14336, 4096)), ("up_proj", (14336, 4096)), ("down_proj", (4096, 14336))]
    gen = torch.Generator(device=device).manual_seed(1)
    items = []
    for layer in range(args.layers):
        for name, shp in shapes:
            w = torch.empty(shp, dtype=torch.bfloat16, device=device)
            w.normal_(0.0, 0.02, generator=gen)
            items.append((f"layers.{layer}.{name}", w, cfg))
    plan = CompressionPlan(items, device, fp16_scales=True, packed_zero_points=True)
    plan.run(use_graph=False)
    torch.cuda.synchronize()
    stored = []
    out_bytes = alg_bytes = 0
    for (name, w, _), it in zip(items, plan.items):
        n = w.numel()
        group = gs if gs != -1 else w.shape[1]
        it.weight = None
        zp = getattr(it, "zero_point_packed", None)
        if zp is None and it.zero_point is not None:
            zp = it.zero_point.to(torch.uint8)
        out = torch.empty(n, dtype=torch.bfloat16, device=device)
        scale = it.scale_f16 if it.scale_f16 is not None else it.scale.to(torch.float16)
        stored.append((it.packed, n, group, scale, zp, out))
        out_bytes += n * 2
        alg_bytes += n * 2 + it.packed.numel() * it.packed.element_size() + scale.numel() * scale.element_size() + \
            (zp.numel() * zp.element_size() if zp is not None else 0)
    del items, plan
    stream = _lib.stream_handle(device)
    mode_id, bf16 = _lib.MODE_IDS[mode.value], _lib.DTYPE_IDS[torch.bfloat16]

    def step():
        nonlocal stream, stored
        for packed, n, group, scale, zp, out in stored:
            _lib.check(_lib.lib.nncfb_decompress(_lib.ptr(packed), mode_id, n, group, _lib.ptr(scale),
                                                 _lib.ptr(zp) if zp is not None else None, _lib.ptr(out), bf16, stream))

    # one pass = one CUDA graph of the per-matrix launches (28 ctypes calls take longer on the host than the
    # kernels on the GPU); replayed like the compression pass of the headline workload
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        stream = _lib.stream_handle(device)
        step()
    torch.cuda.current_stream(device).wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        stream = _lib.stream_handle(device)
        step()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    peak, peak_src = _peaks()
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    # the same per shape: the launches of one kind of matrix (one per layer, different buffers) as a graph of their own
    per_shape = {}
    all_stored = stored
    for k, (name, shp) in enumerate(shapes):
        stored = all_stored[k::len(shapes)]
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2):
            stream = _lib.stream_handle(device)
            step()
        for _ in range(3):
            g2.replay()
        e0.record()
        for _ in range(args.steps):
            g2.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps / len(stored)
        n = shp[0] * shp[1]
        bytes_one = alg_bytes * n / sum(a * b for _, (a, b) in shapes) / args.layers
        per_shape[name] = {"us_per_launch": round(us, 2), "frac_of_hbm_peak": round(bytes_one / (us * 1e-6) / 1e9 / peak, 3)}
    stored = all_stored
    print(json.dumps({
        "metric": f"decompressed_weight_GBps_{mode.value}", "value": round(out_bytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 3),
        "higher_is_better": True, "data": "synthetic", "dtype": "f16",
        "config": {"workload": f"decompression of {args.layers} Llama-3-8B decoder layers ({len(stored)} matrices, "
                               f"{out_bytes / 1e9:.2f} GB of bf16 weights), {mode.value} group {gs}, fp16 scales; "
                               "working set larger than L2"},
        "gpu_launches": len(stored) * args.steps, "per_shape": per_shape,
        "roofline": {"bound": "hbm", "kernel": "decompress_kernel", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes": "codes + scales (+ zero points) read, bf16 weights written"}}), flush=True)


def run_moe_workload(args, device, rank, world, dist):
    """Benchmark configuration 5: NF4 (g128) or MXFP4 (E2M1 values, E8M0 scale per 32) data-free compression of a
    Mixtral-8x7B-shaped expert stack (per layer 8 experts x (w1, w3: 14336 x 4096; w2: 4096 x 14336), bf16
    N(0, 0.02^2), seed 4), experts sharded over the ranks by bytes.  `--layers` sets how many of the 32 layers
    are generated (90 GB for all 32)."""
    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig
    from nncf_b200.pipeline import CompressionPlan, partition_by_bytes

    mode = CompressWeightsMode(args.mode)
    cfg = WeightCompressionConfig(mode, 32 if mode == CompressWeightsMode.MXFP4 else 128)
    names, shapes = [], []
    for layer in range(args.layers):
        for e in range(8):
            for w, shp in (("w1", (14336, 4096)), ("w3", (14336, 4096)), ("w2", (4096, 14336))):
                names.append(f"layers.{layer}.experts.{e}.{w}")
                shapes.append(shp)
    mine = partition_by_bytes([a * b * 2 for a, b in shapes], world)[rank]
    gen = torch.Generator(device=device).manual_seed(4 + rank)
    items = []
    for i in mine:
        w = torch.empty(shapes[i], dtype=torch.bfloat16, device=device)
        w.normal_(0.0, 0.02, generator=gen)
        items.append((names[i], w, cfg))
    plan = CompressionPlan(items, device)
    steps = 1 if args.profile_case else args.steps
    for _ in range(1 if args.profile_case else max(args.warmup, 3)):
        plan.run(use_graph=False)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        plan.run(use_graph=False)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], dtype=torch.float64, device=device)
    tot = torch.tensor([float(plan.source_bytes), float(plan.algorithmic_bytes)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    if rank != 0:
        return
    ms = float(t.item())
    peak, peak_src = _peaks()
    alg_rank = plan.algorithmic_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": f"source_weight_GBps_compressed_{mode.value}", "value": round(float(tot[0]) / (ms * 1e-3) / 1e9, 1),
        "unit": UNIT, "n_gpus": world, "steps": steps, "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "strong", "data": "synthetic", "dtype": "f32",
        "config": {"workload": f"Mixtral-8x7B-shaped expert stack, {args.layers} of 32 layers ({len(names)} tensors, "
                               f"{float(tot[0]) / 1e9:.1f} GB bf16), {mode.value} group {cfg.group_size}, experts sharded by bytes"},
        "roofline": {"bound": "hbm", "kernel": f"quant_rows_batch_kernel<bf16, {mode.value}>", "achieved": round(alg_rank, 1),
                     "peak": peak, "unit": "GB/s", "frac": round(alg_rank / peak, 4), "peak_source": peak_src}}), flush=True)


def run_data_aware_workload(args, device):
    """ScaleEstimation and AWQ at Llama-3-8B layer shapes (config: INT4_ASYM g128, AWQ subset 32 / 100 alpha
    steps, ScaleEstimation subset 64 / 5 + 5 steps, statistics synthetic with 1 % outlier channels x20),
    extrapolated to the 32 layers of the model."""
    from nncf_b200 import CompressWeightsMode, WCTensorStatistic, WeightCompressionConfig
    from nncf_b200.awq import AWQ, make_wp
    from nncf_b200.scale_estimation import ScaleEstimation

    cfg = WeightCompressionConfig(CompressWeightsMode.INT4_ASYM, 128)
    gen = torch.Generator(device=device).manual_seed(2)

    def stats(hidden, n=128):
        outl = 1 + 19 * (torch.rand(hidden, device=device, generator=gen) < 0.01)
        means = [(torch.randn(hidden, device=device, generator=gen) * outl).to(torch.bfloat16) for _ in range(n)]
        return WCTensorStatistic(means, [(1, 512, hidden)] * n)

    def timed(fn, reps=3):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps * 1e3

    shapes = {"q_proj": (4096, 4096), "k_proj": (1024, 4096), "gate_proj": (14336, 4096), "down_proj": (4096, 14336)}
    if args.profile_case:
        shapes = {"k_proj": (1024, 4096)}
    se_ms, st = {}, {4096: stats(4096), 14336: stats(14336)}
    for name, (o, i) in shapes.items():
        w = (torch.randn(o, i, device=device, generator=gen) * 0.02).to(torch.bfloat16)
        se_ms[name] = round(timed(lambda: ScaleEstimation.calculate_quantization_params(st[i], w, (1,), cfg, -1, 64, 5, 5)), 3)
    out = {"metric": "data_aware_seconds_per_8b_model", "unit": "s", "higher_is_better": False, "n_gpus": 1,
           "data": "synthetic", "dtype": "f32",
           "config": {"workload": "INT4_ASYM g128 ScaleEstimation (64 samples, 5+5 steps) on all 7 matrices per layer and "
                                  "AWQ (32 samples, 100 alpha steps) on down_proj, Llama-3-8B shapes, x32 layers"},
           "scale_estimation_ms": se_ms}
    if not args.profile_case:
        wd = (torch.randn(4096, 14336, device=device, generator=gen) * 0.02).to(torch.bfloat16)
        wu = (torch.randn(14336, 4096, device=device, generator=gen) * 0.02).to(torch.bfloat16)
        algo = AWQ()
        out["awq_down_proj_ms"] = round(timed(lambda: algo._data_aware_step(make_wp(cfg), wd, st[14336], -1, wu, st[4096])), 3)
        per_layer = 2 * se_ms["q_proj"] + 2 * se_ms["k_proj"] + 2 * se_ms["gate_proj"] + se_ms["down_proj"] + out["awq_down_proj_ms"]
        out["value"] = round(32 * per_layer / 1e3, 3)
        n_w = 32 * (2 * 4096 * 4096 + 2 * 1024 * 4096 + 3 * 14336 * 4096)
        out["source_GBps"] = round(n_w * 2 / (32 * per_layer * 1e-3) / 1e9, 1)
    print(json.dumps(out), flush=True)


def tensor_seed(index: int) -> int:
    """Seed of weight `index` of the synthetic model (configuration seed 1): the same tensor has the same values
    whichever rank generates it."""
    return 1 * 1000003 + index


def make_weight(shape, index: int, device):
    gen = torch.Generator(device=device).manual_seed(tensor_seed(index))
    w = torch.empty(shape, dtype=torch.bfloat16, device=device)
    w.normal_(0.0, 0.02, generator=gen)
    return w


def model_specs():
    """(name, shape, dtype, config) of the 226 weights: INT4_SYM g128, embed_tokens / lm_head on the INT8_ASYM backup."""
    from nncf_b200 import CompressWeightsMode, WeightCompressionConfig
    from nncf_b200.pipeline import llama3_8b_weight_shapes

    int4 = WeightCompressionConfig(CompressWeightsMode.INT4_SYM, 128)
    int8 = WeightCompressionConfig(CompressWeightsMode.INT8_ASYM, -1)
    return [(name, shape, torch.bfloat16, int8 if name in ("model.embed_tokens", "lm_head") else int4)
            for name, shape in llama3_8b_weight_shapes()]


def parity_gate(specs, results: dict, device) -> dict:
    """Checks what the timed passes left behind against the CPU oracle: the seven matrices of decoder layer 0 in
    full and the first 1/32 of the embedding's and lm_head's rows (rows are independent, so a row range of the
    weight maps to a byte range of every output).  `results`: {name: {field: tensor}} on this rank, for N > 1
    including what other ranks compressed and sent.  Weights are regenerated here from their seeds."""
    from oracle import wc_oracle as O

    checked, mismatched, compared = 0, 0, 0
    for i, (name, shape, _, cfg) in enumerate(specs):
        backup = name in ("model.embed_tokens", "lm_head")
        if not (backup or name.startswith("model.layers.0.")) or name not in results:
            continue
        rows = shape[0] // 32 if backup else shape[0]
        w = make_weight(shape, i, device)[:rows].float().cpu().numpy()
        ref = O.stored_form(w, cfg.mode.value, cfg.group_size)
        gs = shape[1] if cfg.group_size == -1 else cfg.group_size
        per_row = {"packed": shape[1] // 2 if cfg.num_bits == 4 else shape[1], "scale": shape[1] // gs,
                   "zero_point": shape[1] // gs, "scale_e8m0": shape[1] // gs}
        for field, want in ref.items():
            got = results[name][field][: rows * per_row[field]].cpu().numpy().reshape(-1)
            if got.dtype != want.dtype:
                got = got.view(want.dtype)
            mismatched += int((got != want).sum())
            compared += want.size * want.itemsize
        checked += 1
    return {"checked_tensors": checked, "compared_bytes": compared, "mismatched_bytes": mismatched,
            "against": "numpy oracle of the reference's arithmetic (oracle/wc_oracle.py), after the timed passes",
            "what": "decoder layer 0 (7 matrices, full) + first 1/32 of embed_tokens and lm_head rows"}


def run_gptq_model(args, device, rank, world, dist):
    """Benchmark configuration 4 as written: a random-init Llama-3-8B-architecture bf16 model (Hugging Face
    LlamaForCausalLM, N(0, 0.02^2), seed 1), 128 sequences of 2048 token ids uniform in [0, 128256) from seed 3
    run through the model, INT4_SYM group 128, gptq=True, damping 0.01, block 128, fp32 Hessians - through
    nncf_b200.compress_weights.  `--gptq-layers k` keeps only the first k decoder layers of the model (the line
    says so); the default is all 32.  Returns the `gptq` object of the JSON line."""
    import transformers

    import nncf_b200 as nb
    from nncf_b200 import compress_api

    layers = args.gptq_layers
    cfg = transformers.LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=layers,
                                   num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=8192,
                                   rope_theta=500000.0, tie_word_embeddings=False, initializer_range=0.02)
    torch.manual_seed(1)
    t0 = time.perf_counter()
    with torch.device(device):
        model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t0
    gen = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 128256, (args.gptq_samples, args.gptq_tokens), generator=gen)
    items = [{"input_ids": ids[k:k + 1].to(device)} for k in range(args.gptq_samples)]
    adv = nb.AdvancedCompressionParameters(gptq_params=nb.AdvancedGPTQParameters(damp_percent=0.01, block_size=128,
                                                                                subset_size=args.gptq_samples))
    with torch.no_grad():
        model(input_ids=items[0]["input_ids"])   # process warm-up: one forward pass of one calibration item
    compress_api.COLLECT_TIMERS = True
    compress_api.TIMERS.clear()
    group = dist.group.WORLD if world > 1 else None
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nb.compress_weights(model, mode=nb.CompressWeightsMode.INT4_SYM, group_size=128, ratio=1.0, gptq=True,
                        dataset=nb.Dataset(items), subset_size=args.gptq_samples, advanced_parameters=adv,
                        process_group=group)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    seconds = time.perf_counter() - t0
    with torch.no_grad():
        finite = bool(torch.isfinite(model(input_ids=items[0]["input_ids"][:, :128]).logits).all())
    split = {k: round(v, 3) for k, v in compress_api.TIMERS.items()}
    n_params = sum(p.numel() for p in model.parameters())
    del model, items
    torch.cuda.empty_cache()
    peak_tf = 1373.9
    try:
        peak_tf = float(json.loads((ROOT / "MEASURED_PEAKS.json").read_text())["bf16_tflops_sustained"])
    except Exception:
        pass
    out = {"metric": "gptq_seconds_per_8b_model", "value": round(seconds * 32 / layers, 2) if layers != 32 else round(seconds, 2),
           "unit": "s", "higher_is_better": False, "measured_seconds": round(seconds, 2), "decoder_layers_run": layers,
           "config": {"workload": f"LlamaForCausalLM random init, Llama-3-8B architecture with {layers} of 32 decoder "
                                  f"layers, bf16; {args.gptq_samples} x {args.gptq_tokens} calibration token ids (seed 3) "
                                  "through the model; compress_weights(INT4_SYM, group 128, gptq=True, damp 0.01, block "
                                  "128), embed_tokens / lm_head on the INT8_ASYM backup; one forward pass of one calibration item "
                                  "before the timed call (kernel loading, allocator warm-up)",
                      "extrapolated": None if layers == 32 else f"value = measured x 32 / {layers} (per-layer work is identical)"},
           "split_seconds": split, "model_build_seconds": round(t_build, 2), "outputs_finite": finite,
           "weights_in_model": n_params, "n_gpus": world,
           "sharing": None if world == 1 else "calibration items shared among the ranks (Hessians all-reduced), one inverse "
                                              "factor (rank 0's), layers that share a factor swept by different ranks and "
                                              "broadcast; split_seconds are rank 0's"}
    tokens = args.gptq_samples * args.gptq_tokens
    if split.get("hessians"):
        # per decoder layer 3 Hessians over 4096 channels and 1 over 14336; the kernel multiplies the 128 x 256
        # tiles that touch the upper triangle
        def computed(C):
            tm, tn = (C + 127) // 128, (C + 255) // 256
            return 2.0 * tokens * sum(tn - mi // 2 for mi in range(tm)) * 128 * 256
        flops = layers * (3 * computed(4096) + computed(14336)) / world   # this rank's share of the tokens
        tf = flops / split["hessians"] / 1e12
        out["roofline"] = {"bound": "tensor", "kernel": "tc_tn_kernel<4 stages, Hessian> (tcgen05 / TMEM / TMA), inside the model run",
                           "achieved": round(tf, 1), "peak": peak_tf, "unit": "TFLOP/s", "frac": round(tf / peak_tf, 4),
                           "peak_source": "measured (MEASURED_PEAKS.json bf16_tflops_sustained)",
                           "flops": "computed tiles (upper triangle) of 3 x C=4096 + 1 x C=14336 Hessians per layer",
                           "timed": "CUDA events around every accumulation call, summed"}
    return out


def run_data_aware_model(args, device):
    """Benchmark configuration 3 as written: INT4_ASYM group 128 with awq=True and scale_estimation=True on the
    random-init Llama-3-8B-architecture bf16 model; calibration is 128 sequences of 512 token ids uniform in
    [0, 128256) from seed 2 run through the model, with 1 % of the hidden channels of the embedding table scaled
    by 20 to create activation outliers.  Wall time of the whole nncf_b200.compress_weights call."""
    import transformers

    import nncf_b200 as nb

    layers = args.gptq_layers
    cfg = transformers.LlamaConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=layers,
                                   num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=8192,
                                   rope_theta=500000.0, tie_word_embeddings=False, initializer_range=0.02)
    torch.manual_seed(1)
    with torch.device(device):
        model = transformers.LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    gen = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 128256, (128, 512), generator=gen)
    outliers = torch.randperm(4096, generator=gen)[:41].to(device)      # 1 % of the hidden channels
    with torch.no_grad():
        model.model.embed_tokens.weight[:, outliers] *= 20.0
        model(input_ids=ids[:1, :16].to(device))                         # process warm-up (kernel loading)
    items = [{"input_ids": ids[k:k + 1].to(device)} for k in range(128)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    nb.compress_weights(model, mode=nb.CompressWeightsMode.INT4_ASYM, group_size=128, ratio=1.0, awq=True,
                        scale_estimation=True, dataset=nb.Dataset(items), subset_size=128)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    with torch.no_grad():
        finite = bool(torch.isfinite(model(input_ids=items[0]["input_ids"][:, :64]).logits).all())
    print(json.dumps({
        "metric": "awq_scale_estimation_seconds_per_8b_model", "value": round(seconds * 32 / layers, 2), "unit": "s",
        "higher_is_better": False, "n_gpus": 1, "measured_seconds": round(seconds, 2), "decoder_layers_run": layers,
        "data": "synthetic", "dtype": "f32", "outputs_finite": finite,
        "config": {"workload": f"LlamaForCausalLM random init, Llama-3-8B architecture ({layers} of 32 decoder layers), bf16; "
                               "compress_weights(INT4_ASYM, group 128, awq=True, scale_estimation=True), 128 x 512 calibration "
                               "token ids (seed 2) through the model, 41 of 4096 embedding channels x 20; whole call incl. "
                               "statistics collection, AWQ on the down_proj / up_proj pairs, ScaleEstimation on every 4-bit "
                               "matrix, packing and installing the decompressors"}}), flush=True)


def run_compress(args, device, rank, world, local_rank, dist):
    from nncf_b200.pipeline import CompressionPlan, HostStreamingCompressor, bind_host_thread_near, partition_by_bytes
    from nncf_b200.sharding import ShardedCompression

    # one process per GPU: keep this rank's pinned buffers and copy threads on the CPUs next to its GPU
    cpus_at_start = os.sched_getaffinity(0)
    affinity = bind_host_thread_near(device) if not args.no_affinity else "unchanged (--no-affinity)"
    specs = model_specs()
    if args.profile_case:
        specs = specs[1:8]  # one decoder layer: 436 MB of weights, larger than L2
        args.steps, args.no_e2e, args.no_cpu_baseline, args.no_gptq, args.no_parity = 1, True, True, True, True
    sc = ShardedCompression(specs, device, rank, world, dst=0, n_chunks=args.chunks, dst_share=args.dst_share,
                            registered_buffers=args.registered_buffers, peer_stores=args.transport == "peer",
                            peer_copies=args.transport == "peer_copy")
    index_of = {s[0]: i for i, s in enumerate(specs)}
    weights = {i: make_weight(specs[i][1], i if not args.profile_case else i + 1, device) for i in sc.local_indices}
    sc.bind(weights)
    plan = sc.plan
    idx4 = [k for k, it in enumerate(plan.items) if it.config.num_bits == 4]
    idx8 = [k for k, it in enumerate(plan.items) if it.config.num_bits == 8]
    alg4 = sum(plan.items[k].algorithmic_bytes() for k in idx4)
    src_total = sc.source_bytes_total
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    use_graph = world == 1 and not (args.no_graph or args.profile_case)
    if world == 1:
        if use_graph:
            g4 = plan.capture(idx4)
            g8 = plan.capture(idx8) if idx8 else None
            run4 = g4.replay
            run8 = g8.replay if g8 is not None else (lambda: None)
        else:
            run4 = lambda: plan.launch(idx4)  # noqa: E731
            run8 = (lambda: plan.launch(idx8)) if idx8 else (lambda: None)  # noqa: E731

        def step():
            run4()
            run8()
        launches_per_step = 2 if idx8 else 1
    else:
        def step():
            sc.run()
            sc.wait()
        launches_per_step = len(sc._chunk_items)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)] if world == 1 else None
    t_begin.record()
    for s_ in range(args.steps):
        if world == 1:
            ev[s_][0].record()
            run4()
            ev[s_][1].record()
            run8()
            ev[s_][2].record()
        else:
            step()
    t_end.record()
    barrier()
    total_ms = t_begin.elapsed_time(t_end)
    t = torch.tensor([total_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = src_total / (ms_per_step * 1e-3) / 1e9

    # ---- the halves on their own (N > 1): kernels without transfers, transfers without kernels ------------
    multi = None
    if world == 1:
        ms4 = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
        ms8 = sum(e[1].elapsed_time(e[2]) for e in ev) / args.steps
    else:
        def timed(fn, reps):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            barrier()
            return a.elapsed_time(b) / reps

        own_ms = timed(lambda: sc.run(transfer=False), args.steps)
        ms4 = timed(lambda: plan.launch(idx4), args.steps) if idx4 else 0.0
        ms8 = 0.0

        def transfer_only():
            sc.run(compute=False)
            sc.wait()
        xfer_ms = timed(transfer_only, max(3, args.steps // 2))
        tt = torch.tensor([own_ms, xfer_ms], dtype=torch.float64, device=device)
        mx = tt.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        gathered = [torch.zeros_like(tt) for _ in range(world)]
        dist.all_gather(gathered, tt)
        compress_ms, gather_ms = float(mx[0]), float(mx[1])
        multi = {
            "partition": "ONE model split by source bytes (LPT greedy); the collecting rank's share is sized so that its "
                         "own kernels and its NVLink ingest finish together",
            "dst_share_of_source_bytes": round(sc.dst_share, 4),
            "source_GB_per_rank": [round(sum(specs[i][1][0] * specs[i][1][1] * 2 for i in a) / 1e9, 3) for a in sc.assignment],
            "chunks_per_sender": args.chunks,
            "compress_only": {"ms_per_step_max_over_ranks": round(compress_ms, 4),
                              "value": round(src_total / (compress_ms * 1e-3) / 1e9, 1),
                              "ms_per_rank": [round(float(g[0]), 4) for g in gathered]},
            "transport": ("peer copies" if sc.peer_copies else "peer stores") if sc.peer_stores else "NCCL send/recv",
            "gather_only": None if sc.peer_stores else {
                "ms_per_step": round(gather_ms, 4), "bytes_into_rank0": sc.output_bytes_total -
                sum(sc.out_sizes[i] for i in sc.assignment[0]),
                "ingest_GBps": round((sc.output_bytes_total - sum(sc.out_sizes[i] for i in sc.assignment[0])) /
                                     (gather_ms * 1e-3) / 1e9, 1)},
            "bytes_into_rank0": sc.output_bytes_total - sum(sc.out_sizes[i] for i in sc.assignment[0]),
            "gather_exposed_ms": None if sc.peer_stores else round(ms_per_step - compress_ms, 4),
            "bound_ms": round(compress_ms if sc.peer_stores else max(compress_ms, gather_ms), 4),
            "how": ("rank 0's arena is mapped into every rank's process (CUDA IPC); " +
                    ("every finished chunk of another rank is copied into its byte range of it by one cudaMemcpyAsync "
                     "(copy engines over NVLink, nothing on any SM); " if sc.peer_copies else
                     "the other ranks' compression kernels store codes, scales and zero points straight into their "
                     "byte ranges of it over NVLink; ") +
                    "one 4-byte all-reduce before and after a pass orders them against rank 0's reads; requested: " +
                    args.transport) if sc.peer_stores else
                   ("per chunk one nncfb_quantize_batch launch, an event, one NCCL isend of the chunk's contiguous output "
                    "range on a side stream; rank 0 posts irecvs straight into the final arena (no repacking, no "
                    "manifest); requested: " + args.transport),
            "nccl_env": {k: v for k, v in os.environ.items() if k.startswith("NCCL_")},
        }

    if rank == 0 and not args.profile_case:
        # the timed region lasts tens of milliseconds, less than one nvidia-smi sampling period: keep the same
        # kernels running (untimed) for a moment so that the clock record is taken under this load
        t_probe = time.time() + 0.7
        while time.time() < t_probe:
            for _ in range(10):
                plan.launch()
            torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["window"] = "warm-up + timed region + 0.7 s of the same kernels"
    if world > 1:
        step()   # the probe loop overwrote nothing, but leave a complete pass behind for the parity gate
    barrier()

    # ---- parity gate on what the timed passes wrote ------------------------------------------------------
    parity = None
    if rank == 0 and not args.no_parity:
        parity = parity_gate(specs, sc.results(), device)
    barrier()

    # ---- end to end through host buffers: the model split evenly over the ranks' PCIe links --------------
    e2e = None
    n_launch = args.steps * launches_per_step
    if not args.no_e2e:
        import psutil

        sizes = [s[1][0] * s[1][1] * 2 for s in specs]
        mine = partition_by_bytes(sizes, world)[rank]
        out_sizes = sc.out_sizes
        need = sum(sizes[i] + out_sizes[i] for i in mine)
        budget = psutil.virtual_memory().available / (2.5 * max(world, 1)) * (1 if world == 1 else 1)
        subset_note = None
        if need > budget:
            # keep whole decoder layers' tensors until the budget is used
            keep, acc = [], 0
            for i in sorted(mine, key=lambda i: -sizes[i]):
                if acc + sizes[i] + out_sizes[i] <= budget:
                    keep.append(i)
                    acc += sizes[i] + out_sizes[i]
            subset_note = f"{len(keep)} of this rank's {len(mine)} tensors (host memory budget per rank {budget / 1e9:.1f} GB)"
            mine = keep
        # largest tensors first, the order the reference compresses in (WC/algorithm.py:1198-1199): the copies that
        # cannot overlap with anything (first tensor in, last result out) are then the cheap ones
        mine = sorted(mine, key=lambda i: -sizes[i])
        host_w = []
        for i in mine:
            h = torch.empty(specs[i][1], dtype=torch.bfloat16, pin_memory=True)
            h.copy_(weights[i] if i in weights else make_weight(specs[i][1], i, device))
            host_w.append(h)
        torch.cuda.synchronize()
        e2e_specs = [(specs[i][0], specs[i][1], specs[i][2], specs[i][3]) for i in mine]
        del plan, weights
        sc.close()
        sc = None
        torch.cuda.empty_cache()
        if e2e_specs:
            hsc = HostStreamingCompressor(e2e_specs, device)
            hsc.run(host_w)
            hsc.synchronize()
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.e2e_steps):
                hsc.run(host_w)
                hsc.synchronize()
            barrier()
            dt = (time.perf_counter() - t0) / args.e2e_steps
            agg = torch.tensor([dt, float(hsc.h2d_bytes), float(hsc.d2h_bytes)], dtype=torch.float64, device=device)
            if world > 1:
                mx = agg.clone()
                dist.all_reduce(mx, op=dist.ReduceOp.MAX)
                dist.all_reduce(agg, op=dist.ReduceOp.SUM)
                dt = float(mx[0])
            e2e = {"value": round(float(agg[1]) / dt / 1e9, 3), "unit": UNIT, "h2d_bytes_per_step": int(agg[1]),
                   "d2h_bytes_per_step": int(agg[2]), "ms_per_step": round(dt * 1e3, 3), "steps": args.e2e_steps,
                   "api": "nncf_b200.pipeline.HostStreamingCompressor.run (pinned host weights in, packed results "
                          "back in pinned host memory; 3-stream overlap of H2D, kernels, D2H)",
                   "split": "the one model's tensors split evenly by bytes over the ranks, each rank on its own PCIe link; "
                            "bytes are totals over all ranks, time is the slowest rank's" if world > 1 else "single GPU",
                   "host_affinity": affinity}
            n_launch += (1 + args.e2e_steps) * len(e2e_specs)
            if subset_note:
                e2e["subset"] = subset_note
            del hsc, host_w
        else:
            e2e = {"value": None, "unit": UNIT, "skipped": "not enough free host memory to pin even one tensor"}
        torch.cuda.empty_cache()

    if sc is not None:
        plan = weights = None
        sc.close()
        sc = None
        torch.cuda.empty_cache()

    # ---- GPTQ seconds per 8B model (the second half of the metric) ---------------------------------------
    gptq = None
    if not args.no_gptq:
        gptq = run_gptq_model(args, device, rank, world, dist)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = _peaks()
    achieved = alg4 / (ms4 * 1e-3) / 1e9 if ms4 > 0 else 0.0
    roofline = {
        "bound": "hbm", "kernel": "quant_rows_batch_kernel<bf16, INT4_SYM, 8 lanes x 2 vectors per group, 4 groups in flight> "
                                  "(one launch for all of this rank's 4-bit tensors)",
        "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
        "peak_source": peak_src, "launches_per_step": 1, "tensors_per_launch": len(idx4), "avg_launch_us": round(ms4 * 1e3, 2),
        "algorithmic_bytes_per_launch": alg4, "traffic": None,
        "traffic_note": "not measured in this run (needs a profiler); an ncu capture of the same kernel on one decoder "
                        "layer read DRAM bytes = 0.93 of the algorithmic bytes: part of the writes was still in L2",
        "timed_on": "rank 0" if world > 1 else "the single GPU",
    }
    if world == 1:
        roofline["int8_kernel"] = {"kernel": "quant_channel_batch_kernel<bf16, INT8_ASYM, 64 threads/row>", "ms_per_step": round(ms8, 4)}
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD if not args.profile_case else "profile case: one decoder layer (7 matrices, 436 MB)",
                   "total_source_bytes": src_total,
                   "value_is": "compress only (inputs resident in HBM)" if world == 1 else
                               "compress + gather of every packed result on rank 0 (one model over all ranks)",
                   "launch": "cuda-graph replay" if use_graph else "per-call launches",
                   "l2": "inputs (16 GB per step over all ranks) exceed L2 (126 MB); no flush needed",
                   "seed": "per tensor, from configuration seed 1 and the tensor's index", "distribution": "N(0, 0.02^2) bf16"},
        "roofline": roofline, "e2e": e2e, "multi_gpu": multi, "parity": parity, "gptq": gptq,
        "gpu_launches": n_launch, "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        os.sched_setaffinity(0, cpus_at_start)  # the CPU baseline gets every core the process started with
        threads = host_threads()
        gbs, dt, nbytes, kind, note = cpu_reference_sample(threads, 3, 1)
        line["cpu_baseline"] = {
            "value": round(gbs, 4), "unit": UNIT, "cores": threads, "kind": kind,
            "sample": f"1/32 of the workload ({nbytes / 1e6:.0f} MB source: 1 decoder layer INT4_SYM g128 + 1/32 of "
                      f"embed/lm_head rows INT8_ASYM), compress + pack, 3 timed passes after 1 warm-up; {note}",
            "seconds_per_pass": round(dt, 3)}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of the timed passes' outputs")
    ap.add_argument("--no-gptq", action="store_true", help="skip the GPTQ half of the metric")
    ap.add_argument("--gptq-layers", type=int, default=32, help="decoder layers of the GPTQ model (32 = the whole model)")
    ap.add_argument("--gptq-samples", type=int, default=128)
    ap.add_argument("--gptq-tokens", type=int, default=2048)
    ap.add_argument("--no-graph", action="store_true", help="launch kernels one by one instead of replaying a graph")
    ap.add_argument("--chunks", type=int, default=4, help="N > 1: pieces a sender's work is cut into (one send each)")
    ap.add_argument("--dst-share", type=float, default=None,
                    help="N > 1: share of the source bytes the collecting rank compresses itself (default: balanced "
                         "against its NVLink ingest)")
    ap.add_argument("--registered-buffers", action="store_true",
                    help="N > 1: arenas from NCCL's allocator, registered with the communicator (zero-copy transfers)")
    ap.add_argument("--workload", default="compress", choices=["compress", "gptq", "gptq_model", "data_aware", "data_aware_model", "moe", "api", "decompress"],
                    help="compress: the headline line (default); gptq: per-kernel GPTQ timings; gptq_model: only the "
                         "GPTQ model run of the headline line")
    ap.add_argument("--mode", default="nf4", choices=["nf4", "mxfp4", "fp4"], help="mode of the moe workload")
    ap.add_argument("--transport", default="peer_copy", choices=["nccl", "peer", "peer_copy"],
                    help="N > 1: how results reach rank 0 (NCCL send/recv, or the kernels' own stores into rank 0's "
                         "memory over NVLink)")
    ap.add_argument("--decompress-mode", default="int4_sym", choices=["int4_sym", "int4_asym", "int8_asym"],
                    help="mode of the decompress workload")
    ap.add_argument("--layers", type=int, default=4, help="layers of the moe workload (32 = the full 90 GB stack)")
    ap.add_argument("--no-affinity", action="store_true", help="do not bind the process to the CPUs closest to its GPU")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for profilers: one decoder layer, no e2e / cpu arm, 1 warm-up, 1 step")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product path has no CPU fallback)")
    args.warmup = max(args.warmup, 3) if not args.profile_case else 1
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    import torch.distributed as dist

    if world > 1:
        # NCCL point-to-point transfers between two GPUs use few channels by default; the gather is one-to-one
        # traffic into a single rank, so let every pair use all of them (set before the communicator exists;
        # values already in the environment win)
        os.environ.setdefault("NCCL_NCHANNELS_PER_PEER", "32")
        os.environ.setdefault("NCCL_MIN_P2P_NCHANNELS", "32")
        os.environ.setdefault("NCCL_MAX_P2P_NCHANNELS", "64")
    if args.workload == "moe":
        if world > 1:
            dist.init_process_group("nccl", device_id=device)
        if args.profile_case:
            args.layers = 1
        run_moe_workload(args, device, rank, world, dist)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "gptq_model":
        if world > 1:
            dist.init_process_group("nccl", device_id=device)
        out = run_gptq_model(args, device, rank, world, dist)
        if rank == 0:
            print(json.dumps(out), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload in ("gptq", "data_aware", "api", "data_aware_model", "decompress"):
        if rank == 0:
            {"gptq": run_gptq_workload, "data_aware": run_data_aware_workload, "api": run_api_workload,
             "data_aware_model": run_data_aware_model, "decompress": run_decompress_workload}[args.workload](args, device)
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    run_compress(args, device, rank, world, local_rank, dist)


if __name__ == "__main__":
    main()
