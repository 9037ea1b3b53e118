"""The streamed multi-GPU compression on real GPUs: one model's tensors split over two ranks (NCCL), results
collected in rank 0's arena while the other rank is still compressing, every byte checked against the oracle;
by NCCL send / receive (plain or registered arenas), by the other rank's kernels storing straight into rank 0's
arena over NVLink (CUDA IPC mapping), or by copies of finished chunks into that mapping.
Needs two GPUs (skipped otherwise); the protocol itself is covered on CPU by tests/test_sharding_cpu.py."""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [((512, 1024), "int4_sym", 128), ((1024, 512), "int8_asym", -1), ((256, 2048), "int4_asym", 128),
          ((384, 1024), "nf4", 128), ((640, 1024), "int4_sym", 128), ((128, 4096), "mxfp4", 32),
          ((2048, 1024), "int4_sym", 64), ((96, 1024), "int8_sym", -1)]


def _weight(k, shape, device):
    gen = torch.Generator(device=device).manual_seed(100 + k)
    w = torch.empty(shape, dtype=torch.bfloat16, device=device)
    w.normal_(0.0, 0.02, generator=gen)
    return w


def _worker(rank, world, port, variant, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from nncf_b200 import CompressWeightsMode, WeightCompressionConfig
        from nncf_b200.sharding import ShardedCompression

        specs = [(f"w{k}", shp, torch.bfloat16, WeightCompressionConfig(CompressWeightsMode(m), g))
                 for k, (shp, m, g) in enumerate(SHAPES)]
        sc = ShardedCompression(specs, device, rank, world, dst=0, n_chunks=3, dst_share=0.5,
                                registered_buffers=variant == "registered", peer_stores=variant == "peer_stores",
                                peer_copies=variant == "peer_copies")
        sc.bind({i: _weight(i, specs[i][1], device) for i in sc.local_indices})
        if variant in ("peer_stores", "peer_copies"):
            assert sc.peer_stores, "the collecting rank's arena could not be mapped"
        for _ in range(2):
            sc.run()
            sc.wait()
        torch.cuda.synchronize()
        out = None
        if rank == 0:
            out = {name: {f: t.cpu().numpy().copy() for f, t in fields.items()} for name, fields in sc.results().items()}
        sc.close()
        q.put((rank, out, sorted(sc.local_indices)))
    except Exception as exc:  # noqa: BLE001
        q.put((rank, repr(exc), None))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("variant", ["nccl", "registered", "peer_stores", "peer_copies"])
def test_two_ranks_compress_one_model_and_rank_0_holds_every_result(variant):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    from oracle import wc_oracle as O

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, variant, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {r: (out, idx) for r, out, idx in (q.get(timeout=300) for _ in procs)}
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert isinstance(got[0][0], dict), got[0][0]
    assert got[1][1] and got[0][1] and sorted(got[0][1] + got[1][1]) == list(range(len(SHAPES)))   # both ranks worked
    res = got[0][0]
    for k, (shape, mode, gs) in enumerate(SHAPES):
        w = _weight(k, shape, "cuda:0").float().cpu().numpy()
        ref = O.stored_form(w, mode, gs)
        for field, want in ref.items():
            have = res[f"w{k}"][field].reshape(-1)
            if have.dtype != want.dtype:
                have = have.view(want.dtype)
            np.testing.assert_array_equal(have, want, err_msg=f"w{k} {mode} {field}")
