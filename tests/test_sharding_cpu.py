"""Host-side logic of the multi-GPU path on CPU: the byte-balanced partition and the gather protocol
run as two gloo ranks (world_size 2)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nncf_b200.pipeline import llama3_8b_weight_shapes, partition_by_bytes


def test_partition_is_balanced_complete_and_deterministic():
    sizes = [s[0] * s[1] * 2 for _, s in llama3_8b_weight_shapes()]
    for world in (1, 2, 4, 8):
        parts = partition_by_bytes(sizes, world)
        assert sorted(i for p in parts for i in p) == list(range(len(sizes)))
        loads = [sum(sizes[i] for i in p) for p in parts]
        assert max(loads) - min(loads) <= max(sizes)
        assert parts == partition_by_bytes(sizes, world)
    # the two 1 GB embeddings never share a rank when there are at least two ranks
    big = [i for i, s in enumerate(sizes) if s == max(sizes)]
    parts = partition_by_bytes(sizes, 2)
    assert not any(set(big) <= set(p) for p in parts)


def test_partition_edge_cases():
    assert partition_by_bytes([], 3) == [[], [], []]
    assert partition_by_bytes([5], 2) == [[0], []]
    assert partition_by_bytes([1, 1, 1, 1], 2) == [[0, 2], [1, 3]]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, overlap, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nncf_b200.sharding import gather_results, shard_indices

        shapes = [(7, 128), (3, 64), (33, 256), (1, 128), (16, 32)]
        sizes = [a * b for a, b in shapes]
        mine = shard_indices(sizes, rank, world)
        gen = torch.Generator().manual_seed(100)
        everything = {}
        for i, (a, b) in enumerate(shapes):
            everything[f"w{i}"] = [torch.randint(0, 255, (a * b // 2,), dtype=torch.uint8, generator=gen),
                                   torch.randn(a, b // 32, generator=gen),
                                   torch.randint(0, 15, (a, b // 32), dtype=torch.int32, generator=gen)]
        local = {f"w{i}": everything[f"w{i}"] for i in mine}
        if overlap and rank == 1:
            stolen = f"w{shard_indices(sizes, 0, world)[0]}"  # a tensor of rank 0 claimed by rank 1 as well
            local[stolen] = everything[stolen]
        try:
            merged = gather_results(local, dst=0)
        except ValueError as e:
            q.put((rank, "error", str(e)))
            return
        if rank == 0:
            ok = sorted(merged) == sorted(everything) and all(
                all(torch.equal(x, y) and x.dtype == y.dtype for x, y in zip(merged[k], everything[k])) for k in everything)
            q.put((rank, "ok" if ok else "mismatch", ""))
        else:
            q.put((rank, "ok" if merged is None else "mismatch", ""))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("overlap", [False, True])
def test_gather_protocol_two_gloo_ranks(overlap):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, overlap, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    if overlap:
        assert all(r[1] == "error" and "overlap" in r[2] for r in results), results
    else:
        assert all(r[1] == "ok" for r in results), results
