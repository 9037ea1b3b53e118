"""Whole-weight-set compression pipeline.

The reference compresses the weights of a model one after another in a Python loop
(src/nncf/quantization/algorithms/weight_compression/torch_backend.py:442-481: compress_weight,
range check, offset, pack per weight).  At B200 speed a whole 8B-parameter model is a few
milliseconds of kernel time, so per-call host work would dominate.  ``CompressionPlan`` resolves
everything once - tensor list, output buffers, kernel arguments - and replays the launches,
optionally from a CUDA graph, so a step is pure kernel time.

Work sharding over ranks (``partition_by_bytes``) is a longest-processing-time greedy split of the
tensors by source bytes; every tensor (and every MoE expert) compresses independently, so ranks
exchange nothing until the optional gather of the packed results.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from . import _lib
from .config import WeightCompressionConfig
from .parameters import CompressWeightsMode


@dataclass
class PlanItem:
    name: str
    weight: torch.Tensor
    config: WeightCompressionConfig
    reduction_axis: int = -1
    # outputs (allocated by the plan)
    packed: Optional[torch.Tensor] = None
    scale: Optional[torch.Tensor] = None
    scale_f16: Optional[torch.Tensor] = None
    zero_point: Optional[torch.Tensor] = None
    zero_point_packed: Optional[torch.Tensor] = None
    scale_e8m0: Optional[torch.Tensor] = None
    args: Optional[_lib.QuantizeArgs] = field(default=None, repr=False)

    @property
    def source_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def output_tensors(self) -> list[torch.Tensor]:
        outs = [self.packed, self.scale_f16 if self.scale_f16 is not None else self.scale]
        if self.zero_point_packed is not None:
            outs.append(self.zero_point_packed)
        elif self.zero_point is not None:
            outs.append(self.zero_point)
        if self.scale_e8m0 is not None:
            outs.append(self.scale_e8m0)
        return [t for t in outs if t is not None]

    def algorithmic_bytes(self) -> int:
        """Bytes that must cross HBM: the source once plus each stored output once
        (codes, one scale per group, zero points / exponent bytes where the mode has them)."""
        n = self.source_bytes + self.packed.numel()
        n += self.scale.numel() * 4
        if self.zero_point is not None:
            n += self.zero_point.numel() * 4
        if self.zero_point_packed is not None:
            n += self.zero_point_packed.numel()
        if self.scale_e8m0 is not None:
            n += self.scale_e8m0.numel()
        return n


ARENA_ALIGN = 256  # every output starts on a 256-byte boundary inside an arena


def _pad(n: int) -> int:
    return (n + ARENA_ALIGN - 1) // ARENA_ALIGN * ARENA_ALIGN


def stored_outputs(name: str, shape: Sequence[int], axis: int, cfg: WeightCompressionConfig,
                   fp16_scales: bool = False, packed_zero_points: bool = False) -> list[tuple[str, torch.dtype, int]]:
    """(field, dtype, element count) of everything the stored form of one weight consists of, in the order the
    plan allocates them.  Depends only on shape and configuration, so a rank can lay out another rank's results
    without asking it."""
    outer, reduce, inner = _split(tuple(shape), axis % len(shape))
    gs = cfg.group_size if cfg.group_size != -1 else reduce
    if reduce % gs != 0:
        from .errors import InvalidGroupSizeError

        msg = f"Channel size {reduce} should be divisible by size of group {gs}."
        raise InvalidGroupSizeError(msg)
    n, n_groups = outer * reduce * inner, outer * (reduce // gs) * inner
    four_bit = cfg.num_bits == 4
    nibble_ok = four_bit and n % 2 == 0 and ((inner > 1 and inner % 2 == 0) or (inner == 1 and gs % 2 == 0))
    if four_bit and not nibble_ok:
        msg = f"{name}: shape {tuple(shape)} cannot be nibble-packed in one pass"
        raise ValueError(msg)
    signed8 = cfg.is_integer and not cfg.is_asym_mode and not four_bit  # FP8 bit patterns are unsigned bytes
    outs = [("packed", torch.int8 if signed8 else torch.uint8, n // 2 if four_bit else n),
            ("scale", torch.float32, n_groups)]
    if fp16_scales:
        outs.append(("scale_f16", torch.float16, n_groups))
    if cfg.is_integer and cfg.is_asym_mode:
        if packed_zero_points:
            # the decompressor's buffer: a byte per group, or two 4-bit groups per byte (whole 32-bit words)
            outs.append(("zero_point_packed", torch.uint8, (n_groups + 7) // 8 * 4 if four_bit else n_groups))
        else:
            outs.append(("zero_point", torch.int32, n_groups))
    if cfg.mode in (CompressWeightsMode.MXFP4, CompressWeightsMode.MXFP8_E4M3):
        outs.append(("scale_e8m0", torch.uint8, n_groups))
    return outs


def stored_bytes(outs: Sequence[tuple[str, torch.dtype, int]]) -> int:
    """Bytes the outputs of one weight take in an arena (each padded to the arena alignment)."""
    return sum(_pad(n * torch.empty(0, dtype=dt).element_size()) for _, dt, n in outs)


def _split(shape: Sequence[int], axis: int) -> tuple[int, int, int]:
    outer = 1
    for d in shape[:axis]:
        outer *= d
    inner = 1
    for d in shape[axis + 1:]:
        inner *= d
    return outer, shape[axis], inner


class CompressionPlan:
    """Pre-resolved compression of a list of weights on one device.

    ``items``: (name, weight, config[, reduction_axis]) tuples; weights are contiguous CUDA tensors.
    Outputs are the stored form: nibble-packed codes for 4-bit modes (INT4_SYM with the +8
    offset), byte codes for 8-bit modes, fp32 scales [groups], int32 zero points for asymmetric modes,
    E8M0 exponent bytes for MX modes."""

    def __init__(self, items: Sequence[tuple], device: Optional[torch.device] = None, fp16_scales: bool = False,
                 arena: Optional[torch.Tensor] = None, use_arena: bool = False, packed_zero_points: bool = False):
        """``use_arena``: put every output into one byte buffer (``self.arena``; ``arena`` supplies it), item after
        item, each output on a 256-byte boundary - the results of any run of consecutive items are then one
        contiguous range (``item_range``) that can be sent or copied with a single operation.
        ``packed_zero_points``: asymmetric modes write their zero points as the decompressor stores them (uint8 per
        group, or two 4-bit groups per byte) instead of int32 (``PlanItem.zero_point_packed``)."""
        self.items: list[PlanItem] = []
        self.device = torch.device(device) if device is not None else None
        self.arena = arena
        self._use_arena = use_arena or arena is not None
        self._arena_offsets: list[int] = []
        for it in items:
            name, weight, config = it[0], it[1], it[2]
            axis = it[3] if len(it) > 3 else -1
            if not weight.is_cuda or not weight.is_contiguous():
                msg = f"{name}: weights must be contiguous CUDA tensors"
                raise ValueError(msg)
            if self.device is None:
                self.device = weight.device
            self.items.append(PlanItem(name, weight, config, axis % weight.ndim))
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._fp16_scales = fp16_scales
        self._arg_arrays: dict = {}
        self._layouts = [stored_outputs(it.name, it.weight.shape, it.reduction_axis, it.config, fp16_scales,
                                        packed_zero_points) for it in self.items]
        if self._use_arena:
            off = 0
            for lay in self._layouts:
                self._arena_offsets.append(off)
                off += stored_bytes(lay)
            self._arena_offsets.append(off)
            if self.arena is None:
                self.arena = torch.empty(off, dtype=torch.uint8, device=self.device)
            elif self.arena.numel() < off or self.arena.dtype != torch.uint8 or not self.arena.is_contiguous():
                msg = f"the arena must be a contiguous uint8 tensor of at least {off} bytes"
                raise ValueError(msg)
        for k, item in enumerate(self.items):
            self._resolve(item, k)

    def item_range(self, first: int, last: int) -> tuple[int, int]:
        """(offset, bytes) inside the arena of the outputs of items ``first`` .. ``last - 1``."""
        return self._arena_offsets[first], self._arena_offsets[last] - self._arena_offsets[first]

    def _resolve(self, item: PlanItem, k: int) -> None:
        w, cfg, dev = item.weight, item.config, self.device
        outer, reduce, inner = _split(tuple(w.shape), item.reduction_axis)
        gs = cfg.group_size if cfg.group_size != -1 else reduce
        four_bit = cfg.num_bits == 4
        off = self._arena_offsets[k] if self._use_arena else 0
        for field_name, dt, numel in self._layouts[k]:
            if self._use_arena:
                nb = numel * torch.empty(0, dtype=dt).element_size()
                t = self.arena[off:off + nb].view(dt)
                off += _pad(nb)
            else:
                t = torch.empty(numel, dtype=dt, device=dev)
            setattr(item, field_name, t)
        a = _lib.QuantizeArgs()
        a.weight, a.weight_dtype, a.mode = w.data_ptr(), _lib.DTYPE_IDS[w.dtype], _lib.MODE_IDS[cfg.mode.value]
        a.outer, a.reduce, a.inner, a.group_size = outer, reduce, inner, gs
        a.codes_format = _lib.CODES_NIBBLE if four_bit else _lib.CODES_BYTE
        a.codes_out, a.scale_out = item.packed.data_ptr(), item.scale.data_ptr()
        if item.scale_f16 is not None:
            a.scale_f16_out = item.scale_f16.data_ptr()
        if item.zero_point is not None:
            a.zp_out = item.zero_point.data_ptr()
        if item.zero_point_packed is not None:
            a.zp_packed_out = item.zero_point_packed.data_ptr()
        if item.scale_e8m0 is not None:
            a.scale_e8m0_out = item.scale_e8m0.data_ptr()
        item.args = a

    # -- execution --------------------------------------------------------------------------------
    def launch(self, subset: Optional[Sequence[int]] = None) -> None:
        """Enqueue the kernels on the current stream (no synchronisation)."""
        stream = _lib.stream_handle(self.device)
        key = None if subset is None else tuple(subset)
        arr = self._arg_arrays.get(key)
        if arr is None:
            items = self.items if subset is None else [self.items[i] for i in subset]
            arr = (_lib.QuantizeArgs * len(items))(*[it.args for it in items])
            self._arg_arrays[key] = arr
        _lib.check(_lib.lib.nncfb_quantize_batch(arr, len(arr), stream))

    def capture(self, subset: Optional[Sequence[int]] = None) -> torch.cuda.CUDAGraph:
        """Capture the launches in a CUDA graph (the launch-bound loop becomes one replay)."""
        with torch.cuda.device(self.device):
            self.launch(subset)  # warm-up outside capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self.launch(subset)
        return graph

    def run(self, use_graph: bool = True) -> None:
        with torch.cuda.device(self.device):
            if use_graph:
                if self._graph is None:
                    self._graph = self.capture()
                self._graph.replay()
            else:
                self.launch()

    # -- accounting -------------------------------------------------------------------------------
    @property
    def source_bytes(self) -> int:
        return sum(i.source_bytes for i in self.items)

    @property
    def algorithmic_bytes(self) -> int:
        return sum(i.algorithmic_bytes() for i in self.items)

    @property
    def output_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for i in self.items for t in i.output_tensors())


def partition_by_bytes(sizes: Sequence[int], world_size: int,
                       capacity: Optional[Sequence[float]] = None) -> list[list[int]]:
    """Longest-processing-time greedy split: indices sorted by size descending, each to the rank whose load,
    relative to its capacity, is currently the lightest.  Deterministic, so every rank computes the same
    assignment.  ``capacity`` (one positive weight per rank, default all equal) skews the split: a rank with
    twice the capacity receives about twice the bytes - used to give the rank that collects the results more
    of the compression work, since it need not send what it compresses itself.
    (The reference has no counterpart: it walks the weights sequentially,
    src/nncf/quantization/algorithms/weight_compression/algorithm.py:1198-1211.)"""
    cap = [1.0] * world_size if capacity is None else [float(c) for c in capacity]
    if len(cap) != world_size or any(c < 0 for c in cap) or not any(c > 0 for c in cap):
        msg = f"capacity must hold {world_size} non-negative weights, not all zero"
        raise ValueError(msg)
    order = sorted(range(len(sizes)), key=lambda i: (-sizes[i], i))
    loads = [0] * world_size
    parts: list[list[int]] = [[] for _ in range(world_size)]
    usable = [k for k in range(world_size) if cap[k] > 0]
    for i in order:
        r = min(usable, key=lambda k: ((loads[k] + sizes[i]) / cap[k], k))
        parts[r].append(i)
        loads[r] += sizes[i]
    for p in parts:
        p.sort()
    return parts


def llama3_8b_weight_shapes(include_embeddings: bool = True) -> list[tuple[str, tuple[int, int]]]:
    """(name, [out, in]) of every weight matrix of a Llama-3-8B decoder in module order:
    32 layers, hidden 4096, MLP 14336, 32 query / 8 KV heads of 128, vocabulary 128256."""
    hidden, mlp, kv, vocab, layers = 4096, 14336, 1024, 128256, 32
    shapes: list[tuple[str, tuple[int, int]]] = []
    if include_embeddings:
        shapes.append(("model.embed_tokens", (vocab, hidden)))
    for i in range(layers):
        p = f"model.layers.{i}."
        shapes += [
            (p + "self_attn.q_proj", (hidden, hidden)), (p + "self_attn.k_proj", (kv, hidden)),
            (p + "self_attn.v_proj", (kv, hidden)), (p + "self_attn.o_proj", (hidden, hidden)),
            (p + "mlp.gate_proj", (mlp, hidden)), (p + "mlp.up_proj", (mlp, hidden)),
            (p + "mlp.down_proj", (hidden, mlp)),
        ]
    if include_embeddings:
        shapes.append(("lm_head", (vocab, hidden)))
    return shapes


def bind_host_thread_near(device) -> str:
    """Restrict this process to the CPUs NVML reports as closest to ``device`` (same NUMA node / PCIe root), so
    that pinned staging buffers allocated afterwards are placed in that node's memory and the copy threads run
    next to it.  With one process per GPU on a multi-socket host this keeps every rank's host<->device traffic
    off the inter-socket link.  Returns a short description of what was done; any failure leaves the affinity
    unchanged (NVML missing, the container's CPU set does not intersect the ideal one, ...)."""
    import os

    try:
        import pynvml

        index = torch.device(device).index
        if index is None:
            index = torch.cuda.current_device()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        pynvml.nvmlInit()
        if visible:
            ids = [v.strip() for v in visible.split(",") if v.strip()]
            handle = (pynvml.nvmlDeviceGetHandleByIndex(int(ids[index])) if ids[index].isdigit()
                      else pynvml.nvmlDeviceGetHandleByUUID(ids[index]))
        else:
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        ideal = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        target = ideal & allowed
        if not target:
            return "unchanged (the ideal CPUs are outside this process's CPU set)"
        if target == allowed:
            return f"unchanged (already on the {len(target)} closest CPUs)"
        os.sched_setaffinity(0, target)
        return f"bound to {len(target)} CPUs closest to the GPU (of {len(allowed)} allowed)"
    except Exception as exc:  # noqa: BLE001 - affinity is an optimisation, never a failure
        return f"unchanged ({type(exc).__name__})"


class HostStreamingCompressor:
    """Compress weights that live in (pinned) host memory and return the stored form to host
    memory, overlapping the host->device copy of tensor i+1, the kernel of tensor i and the
    device->host copy of tensor i-1 on three streams.

    This is the end-to-end form of the per-weight loop of
    src/nncf/quantization/algorithms/weight_compression/torch_backend.py:442-481 for a model
    whose parameters are on the host (the reference's conformance setup loads the model with
    device_map="cpu").  Device staging is a ring of ``depth`` slots sized for the largest tensor,
    so device memory use is independent of the model size."""

    def __init__(self, specs: Sequence[tuple], device: torch.device, depth: int = 3):
        """``specs``: (name, shape, dtype, config) of the weights, in processing order."""
        self.device = torch.device(device)
        self.depth = depth
        self.specs = list(specs)
        with torch.cuda.device(self.device):
            self.s_in, self.s_run, self.s_out = (torch.cuda.Stream() for _ in range(3))
        max_elems = max(int(torch.Size(s[1]).numel()) for s in self.specs)
        max_item = max(torch.empty(0, dtype=s[2]).element_size() for s in self.specs)
        self.slots = [torch.empty(max_elems * max_item, dtype=torch.uint8, device=self.device) for _ in range(depth)]
        self.slot_free = [torch.cuda.Event() for _ in range(depth)]   # kernel done reading slot
        self.plans: list[CompressionPlan] = []
        self.host_out: list[list[torch.Tensor]] = []
        for k, (name, shape, dtype, cfg) in enumerate(self.specs):
            n = int(torch.Size(shape).numel())
            view = self.slots[k % depth][: n * torch.empty(0, dtype=dtype).element_size()].view(dtype).view(*shape)
            plan = CompressionPlan([(name, view, cfg)], self.device)
            self.plans.append(plan)
            self.host_out.append([torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                                  for t in plan.items[0].output_tensors()])
        self.h2d_bytes = sum(int(torch.Size(s[1]).numel()) * torch.empty(0, dtype=s[2]).element_size() for s in self.specs)
        self.d2h_bytes = sum(t.numel() * t.element_size() for outs in self.host_out for t in outs)

    def run(self, host_weights: Sequence[torch.Tensor]) -> list[list[torch.Tensor]]:
        """Enqueue one pass; returns the pinned host outputs (valid after ``synchronize``)."""
        with torch.cuda.device(self.device):
            loaded = [torch.cuda.Event() for _ in self.specs]
            done = [torch.cuda.Event() for _ in self.specs]
            for k, hw in enumerate(host_weights):
                slot = k % self.depth
                item = self.plans[k].items[0]
                with torch.cuda.stream(self.s_in):
                    if k >= self.depth:
                        self.s_in.wait_event(self.slot_free[slot])
                    item.weight.copy_(hw, non_blocking=True)
                    loaded[k].record(self.s_in)
                with torch.cuda.stream(self.s_run):
                    self.s_run.wait_event(loaded[k])
                    self.plans[k].launch()
                    done[k].record(self.s_run)
                    self.slot_free[slot].record(self.s_run)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(done[k])
                    for dst, src in zip(self.host_out[k], item.output_tensors()):
                        dst.copy_(src, non_blocking=True)
        return self.host_out

    def synchronize(self) -> None:
        for s in (self.s_in, self.s_run, self.s_out):
            s.synchronize()
