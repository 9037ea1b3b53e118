"""Multi-GPU sharding of a compression job: one process per GPU, the weights of ONE model split by source
bytes, results collected on one rank while the others are still compressing.

The reference compresses sequentially in one process
(src/nncf/quantization/algorithms/weight_compression/algorithm.py:1198-1211) and has no collective call site
at all, so this layer is new.  Every weight (and every MoE expert) compresses independently: ranks exchange
nothing while compressing.  The only exchange step is the gather of the stored results (packed codes, scales,
zero points) on one rank, done with ``torch.distributed`` point-to-point operations - NCCL over NVLink for
CUDA tensors, gloo for the CPU tests of the protocol.  Received data always lands in the receiver's own
memory; no kernel reads a peer's memory.

``ShardedCompression`` is the streamed form used by the benchmark and by multi-GPU callers:

* every rank derives the same assignment and the same byte layout of every rank's results from the list of
  (name, shape, dtype, configuration) alone, so no manifest travels;
* a rank's work is cut into a few chunks; each chunk is one batched kernel launch whose outputs are one
  contiguous byte range of the rank's arena, sent with a single ``isend`` as soon as an event says the
  launch has finished, on a side stream, while the next chunk is being compressed;
* the collecting rank owns one arena for the whole model, posts its ``irecv``s straight into the final
  positions (nothing is repacked or copied afterwards) and writes the results of its own share into the
  same arena directly from the kernel;
* the collecting rank gets a larger share of the compression work (``dst_share``): what it compresses
  itself never crosses NVLink, and its NVLink ingest, not the kernels, bounds the job.

``gather_results`` is the simple unstreamed form (manifests as Python objects, one flat buffer per rank).
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .pipeline import CompressionPlan, partition_by_bytes, stored_bytes, stored_outputs

_ALIGN = 256  # every tensor starts on a 256-byte boundary inside a rank's flat buffer


def shard_indices(sizes: Sequence[int], rank: int, world_size: int) -> list[int]:
    """Indices of the tensors this rank compresses (identical partition on every rank)."""
    return partition_by_bytes(sizes, world_size)[rank]


def _itemsize(dtype: torch.dtype) -> int:
    return torch.empty(0, dtype=dtype).element_size()


def default_dst_share(world_size: int, source_bytes: float, output_bytes: float, compress_gbps: float = 4500.0,
                      ingest_gbps: float = 650.0) -> float:
    """Share of the source bytes the collecting rank should compress itself so that it finishes its own share
    when the last remote result arrives: with T_c = time to compress everything on one GPU and T_i = time to
    ingest every result over one NVLink port, the collecting rank's share f solves f T_c = (1 - f) T_i, and the
    other ranks (which work concurrently) must not be slower than that either.  Rates are source GB/s of the
    compression kernels and GB/s into one GPU through NCCL send/recv, measured on B200."""
    if world_size <= 1:
        return 1.0
    t_c = source_bytes / compress_gbps
    t_i = output_bytes / ingest_gbps
    f = t_i / (t_c + t_i)
    # the other ranks each compress (1 - f) / (world - 1) of the model: never hand them more than the collector
    return max(f, 1.0 / world_size)


class ShardedCompression:
    """The weights of one model compressed by ``world_size`` ranks and collected on rank ``dst``.

    ``specs``: (name, shape, dtype, config) of every weight of the model, identical on every rank.
    ``local_indices`` names the weights this rank has to supply to ``bind``.  ``run`` enqueues one pass;
    ``results`` (on ``dst``) maps every weight name to its stored tensors, views into one arena."""

    def __init__(self, specs: Sequence[tuple], device, rank: Optional[int] = None, world_size: Optional[int] = None,
                 dst: int = 0, n_chunks: int = 4, dst_share: Optional[float] = None,
                 group: Optional[dist.ProcessGroup] = None, registered_buffers: bool = False,
                 peer_stores: bool = False, peer_copies: bool = False):
        """``registered_buffers``: allocate the arenas from NCCL's own allocator and register them with the
        communicator (NCCL user-buffer registration), which lets NCCL move point-to-point data without its
        staging copies where the transport supports it.  CUDA + NCCL only.

        ``peer_stores``: no transfer step at all - the collecting rank's arena is mapped into every other rank's
        process (CUDA IPC, one node) and their compression kernels write codes, scales and zero points straight
        into their byte ranges of it over NVLink (plain stores to peer memory).  Nothing runs on the collecting
        rank's SMs for the transfer and there is no staging copy; ``wait`` is a one-element all-reduce that orders
        every rank's kernels before the collecting rank's next read.  Falls back to the NCCL transfers when the
        mapping cannot be set up on every rank.

        ``peer_copies``: the same mapping, but the kernels keep writing into the rank's own arena and every finished
        chunk is copied into the collecting rank's arena by one ``cudaMemcpyAsync`` on a side stream (the copy
        engines move it in large NVLink writes; nothing runs on any SM for the transfer)."""
        self.specs = list(specs)
        self.device = torch.device(device)
        self.group = group
        self.world = world_size if world_size is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.dst = dst
        sizes = [int(torch.Size(s[1]).numel()) * _itemsize(s[2]) for s in self.specs]
        self.layouts = [stored_outputs(s[0], s[1], -1, s[3]) for s in self.specs]
        self.out_sizes = [stored_bytes(lay) for lay in self.layouts]
        if dst_share is None:
            # measured ingest of the collecting GPU: ~650 GB/s through NCCL send/recv or from one peer's copy engine,
            # ~820 GB/s when several peers' copy engines write at once (the share that made all ranks finish
            # together at N = 4 was 0.62)
            several_copiers = bool(peer_copies) and self.world > 2
            dst_share = default_dst_share(self.world, float(sum(sizes)), float(sum(self.out_sizes)),
                                          ingest_gbps=820.0 if several_copiers else 650.0)
        self.dst_share = 1.0 if self.world == 1 else float(dst_share)
        capacity = None
        if self.world > 1:
            other = (1.0 - self.dst_share) / (self.world - 1)
            capacity = [self.dst_share if r == dst else other for r in range(self.world)]
        self.assignment = partition_by_bytes(sizes, self.world, capacity)
        # chunks of every rank: runs of that rank's tensors (largest first, so the chunk sizes even out and the
        # first results leave early), cut where the running output size passes the next multiple of total / n
        self.chunks: list[list[list[int]]] = []
        for r in range(self.world):
            mine = sorted(self.assignment[r], key=lambda i: (-sizes[i], i))
            n = max(1, min(n_chunks if r != dst else 1, len(mine))) if mine else 0
            total = sum(self.out_sizes[i] for i in mine)
            cuts, acc, chunk = [], 0, []
            for i in mine:
                chunk.append(i)
                acc += self.out_sizes[i]
                if len(cuts) < n - 1 and acc >= total * (len(cuts) + 1) / n:
                    cuts.append(chunk)
                    chunk = []
            if chunk:
                cuts.append(chunk)
            self.chunks.append(cuts)
        self.local_indices = [i for chunk in self.chunks[self.rank] for i in chunk]
        self.source_bytes_total = sum(sizes)
        self.source_bytes_local = sum(sizes[i] for i in self.local_indices)
        self.output_bytes_total = sum(self.out_sizes)
        # byte ranges inside the collecting rank's arena: rank after rank, chunk after chunk, tensor after tensor
        self._region: dict = {}
        off = 0
        self._tensor_offset: dict = {}
        for r in range(self.world):
            for c, chunk in enumerate(self.chunks[r]):
                start = off
                for i in chunk:
                    self._tensor_offset[i] = off
                    off += self.out_sizes[i]
                self._region[(r, c)] = (start, off - start)
        self._arena_bytes = off
        self.plan: Optional[CompressionPlan] = None
        self.arena: Optional[torch.Tensor] = None
        self.registered_buffers = bool(registered_buffers) and self.world > 1 and self.device.type == "cuda"
        self.peer_copies = bool(peer_copies) and self.world > 1 and self.device.type == "cuda"
        self.peer_stores = (bool(peer_stores) or self.peer_copies) and self.world > 1 and self.device.type == "cuda"
        self._remote_arena: Optional[torch.Tensor] = None
        self._flag: Optional[torch.Tensor] = None
        self._pool = None
        self._chunk_items: list[list[int]] = []
        self._pending: list = []
        self._comm_stream = None
        self.bytes_received_per_run = sum(n for (r, _), (_, n) in self._region.items() if r != dst) if self.rank == dst else 0

    # ------------------------------------------------------------------------------------------------
    def bind(self, weights: dict) -> None:
        """``weights``: {index into specs: contiguous tensor on this rank's device} for ``local_indices``."""
        missing = [i for i in self.local_indices if i not in weights]
        if missing:
            msg = f"rank {self.rank} was not given the weights {missing[:5]}{'...' if len(missing) > 5 else ''}"
            raise ValueError(msg)
        items = [(self.specs[i][0], weights[i], self.specs[i][3]) for i in self.local_indices]
        own_bytes = sum(self.out_sizes[i] for i in self.local_indices)
        n_arena = self._arena_bytes if self.rank == self.dst else own_bytes
        arena = None
        if self.registered_buffers:
            pg = self.group if self.group is not None else dist.distributed_c10d._get_default_group()
            backend = pg._get_backend(self.device)
            self._pool = torch.cuda.MemPool(backend.mem_allocator)
            with torch.cuda.use_mem_pool(self._pool):
                arena = torch.empty(max(n_arena, 1), dtype=torch.uint8, device=self.device)
            backend.register_mem_pool(self._pool)
        if self.rank == self.dst:
            # one arena for the whole model; this rank's own region is where its kernels write
            self.arena = arena if arena is not None else torch.empty(self._arena_bytes, dtype=torch.uint8, device=self.device)
            start = self._region[(self.rank, 0)][0] if self.chunks[self.rank] else 0
            own = sum(self.out_sizes[i] for i in self.local_indices)
            self.plan = self._make_plan(items, self.arena[start:start + own]) if items else None
        if self.peer_stores:
            self.peer_stores = self._map_collecting_arena()
        self.peer_copies = self.peer_copies and self.peer_stores
        if self.rank != self.dst:
            if self.peer_stores and not self.peer_copies:
                start = self._region[(self.rank, 0)][0] if self.chunks[self.rank] else 0
                target = self._remote_arena[start:start + own_bytes]
            else:
                target = arena[:own_bytes] if arena is not None else None
            self.plan = self._make_plan(items, target) if items else None
            self.arena = self.plan.arena if self.plan is not None else None
        self._chunk_items, k = [], 0
        for chunk in self.chunks[self.rank]:
            self._chunk_items.append(list(range(k, k + len(chunk))))
            k += len(chunk)
        if self.device.type == "cuda":
            with torch.cuda.device(self.device):
                self._comm_stream = torch.cuda.Stream()

    def _map_collecting_arena(self) -> bool:
        """Maps the collecting rank's arena into this process (CUDA IPC) and lets this rank's GPU store into it.
        Collective over the group; True when every rank succeeded."""
        ok = 1
        payload = [None]
        try:
            if self.rank == self.dst:
                payload = [(torch.cuda.device_count(), self.arena.untyped_storage()._share_cuda_())]
        except Exception:  # noqa: BLE001  (an allocator that cannot export its blocks: every rank falls back together)
            ok = 0
        dist.broadcast_object_list(payload, src=dist.get_global_rank(self.group, self.dst) if self.group is not None else self.dst,
                                   group=self.group, device=self.device)
        try:
            if payload[0] is None:
                ok = 0
            elif self.rank != self.dst:
                n_devices, handle = payload[0]
                if n_devices != torch.cuda.device_count():
                    msg = "the ranks do not see the same set of GPUs"
                    raise RuntimeError(msg)
                # The handle is opened with THIS rank's device current, so the collecting GPU's memory is mapped
                # into this GPU's address space with peer access enabled for the mapping (what
                # cudaIpcOpenMemHandle does for a handle from another device); torch then labels the tensor with
                # this device although its bytes live on the collecting GPU.  Opened under the owner's device
                # index instead, the mapping belongs to that device's context in this process and this GPU's
                # kernels may not touch it.
                if not torch.cuda.can_device_access_peer(self.device.index, int(handle[0])):
                    msg = "the collecting rank's GPU is not a peer of this GPU"
                    raise RuntimeError(msg)
                with torch.cuda.device(self.device):
                    storage = torch.UntypedStorage._new_shared_cuda(self.device.index, *handle[1:])
                remote = torch.empty(0, dtype=torch.uint8, device=self.device).set_(storage)
                if remote.numel() < self._arena_bytes:
                    msg = "the collecting rank's arena is smaller than the model's results"
                    raise RuntimeError(msg)
                self._remote_arena = remote[: self._arena_bytes]
        except Exception:  # noqa: BLE001
            ok = 0
        flag = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        good = bool(int(flag.item()))
        if not good:
            self._remote_arena = None
        else:
            self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        return good

    def _make_plan(self, items: list, arena: Optional[torch.Tensor]):
        """The batched launch plan of this rank's weights with its outputs in one arena (a seam for the CPU
        tests of the protocol, which substitute a host-side stand-in for the kernels)."""
        return CompressionPlan(items, self.device, arena=arena, use_arena=True)

    def _chunk_view(self, c: int) -> torch.Tensor:
        first, last = self._chunk_items[c][0], self._chunk_items[c][-1] + 1
        off, nbytes = self.plan.item_range(first, last)
        base = self.plan.arena
        return base[off:off + nbytes]

    def run(self, compute: bool = True, transfer: bool = True) -> None:
        """Enqueue one pass: kernels on the current stream, sends / receives on a side stream ordered behind
        the kernel launch they depend on.  ``wait`` makes the current stream wait for all of it.
        ``compute=False`` / ``transfer=False`` leave one half out (for timing the halves on their own; the
        buffers then hold the previous pass's results)."""
        cuda = self.device.type == "cuda"
        self._pending = []
        if self.peer_stores:
            transfer = False  # the kernels' stores are the transfer
            if compute and self.world > 1:
                # nobody overwrites a byte range that the collecting rank may still be reading
                dist.all_reduce(self._flag, group=self.group)
        if transfer and self.world > 1 and self.rank == self.dst:
            # receives first: they only need the arena, and the senders' first chunks arrive while this rank works
            ops = []
            n_rounds = max((len(self.chunks[r]) for r in range(self.world) if r != self.dst), default=0)
            for c in range(n_rounds):
                for r in range(self.world):
                    if r == self.dst or c >= len(self.chunks[r]):
                        continue
                    off, nbytes = self._region[(r, c)]
                    if nbytes:
                        ops.append(dist.P2POp(dist.irecv, self.arena[off:off + nbytes], r, self.group))
            if ops:
                if cuda:
                    self._comm_stream.wait_stream(torch.cuda.current_stream(self.device))
                    with torch.cuda.stream(self._comm_stream):
                        self._pending += dist.batch_isend_irecv(ops)
                else:
                    self._pending += dist.batch_isend_irecv(ops)
        if self.plan is None:
            return
        for c, idx in enumerate(self._chunk_items):
            if compute:
                if cuda:
                    with torch.cuda.device(self.device):
                        self.plan.launch(idx)
                else:
                    self.plan.launch(idx)
            if self.peer_copies and compute and self.rank != self.dst:
                view = self._chunk_view(c)
                if view.numel():
                    off = self._region[(self.rank, c)][0]
                    done = torch.cuda.Event()
                    done.record(torch.cuda.current_stream(self.device))
                    self._comm_stream.wait_event(done)
                    with torch.cuda.stream(self._comm_stream):
                        self._remote_arena[off:off + view.numel()].copy_(view, non_blocking=True)
            if transfer and self.world > 1 and self.rank != self.dst:
                view = self._chunk_view(c)
                if view.numel() == 0:
                    continue
                if cuda:
                    done = torch.cuda.Event()
                    done.record(torch.cuda.current_stream(self.device))
                    self._comm_stream.wait_event(done)
                    with torch.cuda.stream(self._comm_stream):
                        self._pending += dist.batch_isend_irecv([dist.P2POp(dist.isend, view, self.dst, self.group)])
                else:
                    self._pending += dist.batch_isend_irecv([dist.P2POp(dist.isend, view, self.dst, self.group)])

    def wait(self) -> None:
        """Block the current stream (CUDA) or the caller (CPU) until every send / receive of the last ``run`` is
        complete.  No host synchronisation on CUDA."""
        for req in self._pending:
            req.wait()
        if self.peer_stores and self.world > 1:
            if self.peer_copies and self._comm_stream is not None:
                torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)
            # stream-ordered on every rank behind its kernels (and copies): when this completes on the collecting
            # rank, every other rank's stores into the arena have been performed
            dist.all_reduce(self._flag, group=self.group)
        if self.device.type == "cuda" and self._comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)
        self._pending = []

    def close(self) -> None:
        """Release the arenas.  With ``registered_buffers`` this must run before the process group is destroyed:
        the pool is deregistered from the communicator first, then its memory is returned."""
        self._pending = []
        self.plan = None
        if self.peer_stores and self.world > 1:
            # the mappings go before the memory: every rank drops its view, then the owner may free the arena
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            if self.rank != self.dst:
                self.arena = None
            self._remote_arena = None
            dist.barrier(group=self.group)
        self.arena = None
        if self._pool is not None:
            pg = self.group if self.group is not None else dist.distributed_c10d._get_default_group()
            if self.device.type == "cuda":
                torch.cuda.synchronize(self.device)
            pg._get_backend(self.device).deregister_mem_pool(self._pool)
            self._pool = None

    # ------------------------------------------------------------------------------------------------
    def results(self) -> dict:
        """On the collecting rank: {name: {field: tensor}} for every weight of the model (views into the arena).
        On other ranks: the same for the rank's own weights."""
        out = {}
        if self.rank == self.dst:
            for i, spec in enumerate(self.specs):
                off = self._tensor_offset[i]
                fields = {}
                for name, dt, numel in self.layouts[i]:
                    nb = numel * _itemsize(dt)
                    fields[name] = self.arena[off:off + nb].view(dt)
                    off += (nb + _ALIGN - 1) // _ALIGN * _ALIGN
                out[spec[0]] = fields
            return out
        if self.plan is not None:
            for it, lay in zip(self.plan.items, self.plan._layouts):
                out[it.name] = {name: getattr(it, name) for name, _, _ in lay}
        return out


# ------------------------------------------------------------------------------------------------------
# unstreamed form
# ------------------------------------------------------------------------------------------------------
def _manifest(named: dict) -> list:
    out = []
    for name, tensors in named.items():
        out.append((name, [(str(t.dtype).replace("torch.", ""), tuple(t.shape)) for t in tensors]))
    return out


def _nbytes(dtype: str, shape: Sequence[int]) -> int:
    n = 1
    for d in shape:
        n *= d
    return n * torch.empty(0, dtype=getattr(torch, dtype)).element_size()


def _padded(n: int) -> int:
    return (n + _ALIGN - 1) // _ALIGN * _ALIGN


def flat_size(manifest: list) -> int:
    return sum(_padded(_nbytes(dt, shp)) for _, ts in manifest for dt, shp in ts)


def pack_flat(named: dict, device) -> torch.Tensor:
    """One contiguous byte buffer holding every tensor of ``named`` at aligned offsets."""
    total = flat_size(_manifest(named))
    flat = torch.empty(total, dtype=torch.uint8, device=device)
    off = 0
    for tensors in named.values():
        for t in tensors:
            nb = t.numel() * t.element_size()
            flat[off:off + nb].copy_(t.contiguous().reshape(-1).view(torch.uint8))
            off += _padded(nb)
    return flat


def unpack_flat(flat: torch.Tensor, manifest: list) -> dict:
    out, off = {}, 0
    for name, ts in manifest:
        tensors = []
        for dt, shp in ts:
            nb = _nbytes(dt, shp)
            tensors.append(flat[off:off + nb].view(getattr(torch, dt)).reshape(shp))
            off += _padded(nb)
        out[name] = tensors
    return out


def gather_results(named: dict, dst: int = 0, group: Optional[dist.ProcessGroup] = None,
                   device: Optional[torch.device] = None) -> Optional[dict]:
    """Gather ``{name: [tensor, ...]}`` of every rank on rank ``dst`` (simple form, for callers whose results
    are not laid out in an arena: one extra copy into a flat buffer per rank, nothing overlapped).

    Step 1: manifests (names, dtypes, shapes) travel as Python objects; ``dst`` validates them (a name
    owned by two ranks is an error on every rank, before any payload moves).  Step 2: every other rank
    sends one flat byte buffer, ``dst`` receives each into its own memory and slices it back into
    tensors.  Returns the merged dict on ``dst`` and None elsewhere."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if device is None:
        first = next((t for ts in named.values() for t in ts), None)
        device = first.device if first is not None else torch.device("cpu")
    manifest = _manifest(named)
    manifests: list = [None] * world
    dist.all_gather_object(manifests, manifest, group=group)
    seen: dict = {}
    for r, m in enumerate(manifests):
        for name, _ in m:
            if name in seen:
                msg = f"tensor '{name}' was produced by rank {seen[name]} and rank {r}: the shards overlap"
                raise ValueError(msg)
            seen[name] = r
    if world == 1:
        return dict(named)
    if rank == dst:
        bufs = {r: torch.empty(flat_size(manifests[r]), dtype=torch.uint8, device=device)
                for r in range(world) if r != dst}
        ops = [dist.P2POp(dist.irecv, bufs[r], r, group) for r in bufs if bufs[r].numel() > 0]
        for req in (dist.batch_isend_irecv(ops) if ops else []):
            req.wait()
        merged = dict(named)
        for r, buf in bufs.items():
            merged.update(unpack_flat(buf, manifests[r]))
        return merged
    flat = pack_flat(named, device)
    if flat.numel() > 0:
        for req in dist.batch_isend_irecv([dist.P2POp(dist.isend, flat, dst, group)]):
            req.wait()
    return None
