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


def test_weighted_partition_gives_the_collecting_rank_its_share():
    sizes = [s[0] * s[1] * 2 for _, s in llama3_8b_weight_shapes()]
    total = sum(sizes)
    for world in (2, 4, 8):
        share = 0.6
        cap = [share] + [(1 - share) / (world - 1)] * (world - 1)
        parts = partition_by_bytes(sizes, world, cap)
        assert sorted(i for p in parts for i in p) == list(range(len(sizes)))
        loads = [sum(sizes[i] for i in p) for p in parts]
        assert abs(loads[0] / total - share) < 0.02
        assert max(loads[1:]) - min(loads[1:]) <= max(sizes)
    assert partition_by_bytes([4, 4, 4], 2, [1.0, 0.0]) == [[0, 1, 2], []]
    with pytest.raises(ValueError):
        partition_by_bytes([1], 2, [0.0, 0.0])


class _HostPlan:
    """Stand-in for CompressionPlan on CPU: same arena layout, and a "kernel" that fills every output of an item
    with bytes that depend only on the item's name and the position, so any rank can predict any result."""

    def __init__(self, items, arena):
        from types import SimpleNamespace

        from nncf_b200.pipeline import stored_bytes, stored_outputs

        self.items = [SimpleNamespace(name=n, weight=w, config=c) for n, w, c in items]
        self._layouts = [stored_outputs(n, w.shape, -1, c) for n, w, c in items]
        offs = [0]
        for lay in self._layouts:
            offs.append(offs[-1] + stored_bytes(lay))
        self._offs = offs
        self.arena = arena if arena is not None else torch.zeros(offs[-1], dtype=torch.uint8)
        for it, lay, off in zip(self.items, self._layouts, offs):
            for field, dt, numel in lay:
                nb = numel * torch.empty(0, dtype=dt).element_size()
                setattr(it, field, self.arena[off:off + nb].view(dt))
                off += (nb + 255) // 256 * 256

    def item_range(self, first, last):
        return self._offs[first], self._offs[last] - self._offs[first]

    @staticmethod
    def expected(name, field, numel, dt):
        seed = sum(name.encode()) * 7 + len(field)
        return ((torch.arange(numel, dtype=torch.int64) * 13 + seed) % 97).to(dt)

    def launch(self, idx):
        for k in idx:
            for field, dt, numel in self._layouts[k]:
                getattr(self.items[k], field).copy_(self.expected(self.items[k].name, field, numel, dt))


def _sharded_worker(rank, world, port, dst_share, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nncf_b200 import CompressWeightsMode, WeightCompressionConfig
        from nncf_b200.sharding import ShardedCompression

        class HostSharded(ShardedCompression):
            def _make_plan(self, items, arena):
                return _HostPlan(items, arena)

        i4 = WeightCompressionConfig(CompressWeightsMode.INT4_ASYM, 32)
        i8 = WeightCompressionConfig(CompressWeightsMode.INT8_ASYM, -1)
        mx = WeightCompressionConfig(CompressWeightsMode.MXFP4, 32)
        specs = [(f"w{i}", shp, torch.bfloat16, cfg) for i, (shp, cfg) in enumerate(
            [((64, 128), i8), ((16, 64), i4), ((48, 256), i4), ((8, 128), mx), ((32, 32), i4), ((24, 96), i4),
             ((40, 64), mx), ((12, 160), i8), ((20, 32), i4)])]
        sc = HostSharded(specs, "cpu", rank, world, dst=0, n_chunks=3, dst_share=dst_share)
        # every rank derives the same assignment; the union of the shares is the model
        assert sorted(i for a in sc.assignment for i in a) == list(range(len(specs)))
        sc.bind({i: torch.zeros(specs[i][1], dtype=torch.bfloat16) for i in sc.local_indices})
        for _ in range(2):   # a second pass reuses every buffer
            sc.run()
            sc.wait()
        dist.barrier()
        if rank == 0:
            res = sc.results()
            ok = sorted(res) == sorted(s[0] for s in specs)
            for name, fields in res.items():
                for field, t in fields.items():
                    ok = ok and torch.equal(t, _HostPlan.expected(name, field, t.numel(), t.dtype))
            received = sc.bytes_received_per_run
            q.put((rank, "ok" if ok else "mismatch", received))
        else:
            q.put((rank, "ok", len(sc.local_indices)))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,dst_share", [(2, None), (2, 0.3), (3, 0.5)])
def test_streamed_sharded_compression_collects_every_result_on_rank_0(world, dst_share):
    """The streamed gather as gloo ranks on CPU with a host-side stand-in for the kernels: every rank lays out
    every rank's results identically without exchanging a manifest, chunks are sent as they finish, and the
    collecting rank ends up with every tensor of the model at its final position."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sharded_worker, args=(r, world, port, dst_share, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] == "ok" for r in results), results
    assert [r for r in results if r[0] == 0][0][2] > 0   # something did cross between the ranks


def test_default_share_of_the_collecting_rank():
    """The collecting rank keeps the share at which its own work and its ingest end together: more of the model when
    results arrive slowly, never less than an even split, everything on one GPU."""
    from nncf_b200.sharding import default_dst_share

    src, out = 16.06e9, 4.76e9
    assert default_dst_share(1, src, out) == 1.0
    slow = default_dst_share(8, src, out, ingest_gbps=650.0)
    fast = default_dst_share(8, src, out, ingest_gbps=820.0)
    assert 0.6 < fast < slow < 0.7
    assert default_dst_share(2, src, out, ingest_gbps=1e6) == 0.5


def _gptq_ranks_worker(rank, world, port, q):
    import os
    from types import SimpleNamespace

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import nncf_b200 as nb
        from nncf_b200.compress_api import _GptqRanks
        from nncf_b200.config import WCTensorStatistic

        ranks = _GptqRanks(dist.group.WORLD)
        items = list(range(7))
        mine = ranks.share(items)
        # every rank accumulates the running average (2 / n_r) * sum x^T x over ITS items; the combination must be
        # the average over all of them
        gen = torch.Generator().manual_seed(0)
        xs = [torch.randn(5, 6, generator=gen, dtype=torch.float64) for _ in items]
        H = torch.zeros(6, 6, dtype=torch.float64)
        for i in mine:
            H += (2.0 / len(mine)) * xs[i].T @ xs[i]
        stat = WCTensorStatistic([xs[i].mean(0) for i in mine], [(1, 5, 6)] * len(mine))
        Hc, merged = ranks.combine(H, len(mine), stat)
        want = sum((2.0 / len(items)) * x.T @ x for x in xs)
        factor = torch.full((3, 3), float(rank + 1))
        factor._dead_columns, factor._cholesky_info = "dead", "info"
        factor = ranks.same_factor(factor)
        p = SimpleNamespace(compression_config=nb.WeightCompressionConfig(nb.CompressWeightsMode.INT4_ASYM, 2),
                            weight=torch.zeros(3, 4))
        owner = 1
        given = (torch.full((3, 4), 7.0), torch.full((3, 2, 1), 0.5), torch.full((3, 2, 1), 3, dtype=torch.int32)) \
            if rank == owner else (None, None, None)
        got = ranks.from_owner(owner, p, *given)
        q.put((rank, dict(
            mine=mine, h_err=float((Hc - want).abs().max()),
            means_in_item_order=all(torch.equal(m, xs[i].mean(0)) for i, m in enumerate(merged.mean_values)),
            n_means=len(merged.mean_values), factor=float(factor[0, 0]), kept=(factor._dead_columns, factor._cholesky_info),
            owner_values=(float(got[0][0, 0]), float(got[1][0, 0, 0]), int(got[2][0, 0, 0])))))
    except Exception as exc:  # noqa: BLE001
        q.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_gptq_exchange_steps_over_two_gloo_ranks():
    """The three exchange steps of distributed GPTQ on CPU tensors: calibration items dealt round-robin, per-rank
    running averages of the Hessian combined into the average over all items (weights n_r / n), per-item statistics
    back in item order, rank 0's factor on every rank, one layer's results from the rank that swept it."""
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gptq_ranks_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert all(isinstance(v, dict) for v in out.values()), out
    assert out[0]["mine"] == [0, 2, 4, 6] and out[1]["mine"] == [1, 3, 5]
    for r in (0, 1):
        assert out[r]["h_err"] < 1e-12
        assert out[r]["means_in_item_order"] and out[r]["n_means"] == 7
        assert out[r]["factor"] == 1.0 and out[r]["kept"] == ("dead", "info")
        assert out[r]["owner_values"] == (7.0, 0.5, 3)
