"""Multi-GPU sharding of a compression job: one process per GPU, tensors split by source bytes,
results gathered on one rank.

The reference compresses sequentially in one process
(src/nncf/quantization/algorithms/weight_compression/algorithm.py:1198-1211) and has no collective
call site at all, so this layer is new.  Every weight (and every MoE expert) compresses
independently: ranks exchange nothing while compressing.  The only exchange step is the optional
gather of the stored results (packed codes, scales, zero points) to one rank, done with
``torch.distributed`` point-to-point operations - NCCL over NVLink for CUDA tensors, gloo for the CPU
tests of the protocol.  Received data always lands in the receiver's own memory; no kernel reads a
peer's memory.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .pipeline import partition_by_bytes

_ALIGN = 256  # every tensor starts on a 256-byte boundary inside a rank's flat buffer


def shard_indices(sizes: Sequence[int], rank: int, world_size: int) -> list[int]:
    """Indices of the tensors this rank compresses (identical partition on every rank)."""
    return partition_by_bytes(sizes, world_size)[rank]


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
    """Gather ``{name: [tensor, ...]}`` of every rank on rank ``dst``.

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
