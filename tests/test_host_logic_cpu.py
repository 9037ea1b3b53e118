"""Host-side logic that needs no GPU: the GEMM-based triangular inverse and the two routes to GPTQ's inverse
factor (pure torch), and the CPU-affinity helper against a fake NVML."""
import os
import sys
import types

import pytest
import torch


def _gptq_module():
    # nncf_b200/__init__ loads the CUDA library; the module under test only needs torch for these functions
    import importlib

    try:
        return importlib.import_module("nncf_b200.gptq")
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"nncf_b200 cannot be imported here: {exc}")


@pytest.mark.parametrize("n", [1, 37, 128, 300, 1000])
def test_lower_triangular_inverse_matches_dense_inverse(n, monkeypatch):
    g = _gptq_module()
    monkeypatch.setattr(g, "_TRI_LEAF", 64)  # force several levels of recursion at small sizes
    gen = torch.Generator().manual_seed(n)
    L = torch.tril(torch.randn(n, n, generator=gen, dtype=torch.float64)) * 0.1
    L.diagonal().copy_(1.0 + torch.rand(n, generator=gen, dtype=torch.float64))
    got = g.lower_triangular_inverse(L)
    assert torch.equal(got, torch.tril(got))
    torch.testing.assert_close(got @ L, torch.eye(n, dtype=torch.float64), rtol=0, atol=1e-10)


def test_inverse_factor_routes_agree_on_cpu(monkeypatch):
    """U with H^-1 = U^T U: the reversed-order route (one Cholesky + triangular inverse) against the reference's
    three calls (gptq.py:293-295), including dead columns and damping."""
    g = _gptq_module()
    monkeypatch.setattr(g, "_TRI_LEAF", 32)
    gen = torch.Generator().manual_seed(3)
    C = 200
    x = torch.randn(512, C, generator=gen, dtype=torch.float64)
    x[:, 7] = 0
    H = (2.0 / 4) * (x.T @ x)
    w = torch.randn(8, C, generator=gen, dtype=torch.float64)
    out = {}
    for route in ("reversed", "reference"):
        Hc, wc = H.clone(), w.clone()
        out[route] = g.GPTQ(0.01, inverse_factor=route).prepare_hessian_inverse(Hc, wc)
        assert torch.all(wc[:, 7] == 0)
        assert getattr(out[route], "_dead_columns")[7]
    torch.testing.assert_close(out["reversed"], out["reference"], rtol=0, atol=1e-9)
    Hd = H.clone()
    Hd[7, 7] = 1
    Hd.diagonal().add_(0.01 * Hd.diagonal().mean())
    torch.testing.assert_close(out["reversed"].T @ out["reversed"], torch.linalg.inv(Hd), rtol=0, atol=1e-8)


def test_bind_host_thread_near_uses_nvml_cpu_set(monkeypatch):
    try:
        from nncf_b200.pipeline import bind_host_thread_near
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"nncf_b200 cannot be imported here: {exc}")
    allowed = sorted(os.sched_getaffinity(0))
    if len(allowed) < 2:
        pytest.skip("needs at least two CPUs")
    want = set(allowed[: len(allowed) // 2])
    words = [0] * (max(allowed) // 64 + 1)
    for c in want:
        words[c // 64] |= 1 << (c % 64)
    calls = {}
    fake = types.SimpleNamespace(
        nvmlInit=lambda: None,
        nvmlDeviceGetHandleByIndex=lambda i: calls.setdefault("index", i) or "h",
        nvmlDeviceGetHandleByUUID=lambda u: "h",
        nvmlDeviceGetCpuAffinity=lambda h, n: (words + [0] * n)[:n],
    )
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    before = os.sched_getaffinity(0)
    try:
        msg = bind_host_thread_near(torch.device("cuda", 0))
        assert os.sched_getaffinity(0) == want, msg
        assert "bound to" in msg
        # an NVML failure leaves the affinity alone
        fake.nvmlDeviceGetCpuAffinity = lambda h, n: (_ for _ in ()).throw(RuntimeError("no nvml"))
        assert "unchanged" in bind_host_thread_near(torch.device("cuda", 0))
        assert os.sched_getaffinity(0) == want
    finally:
        os.sched_setaffinity(0, before)


def test_block_replay_reproduces_the_model_block_by_block():
    """The layer-wise engine of model-level GPTQ on CPU: blocks found as the ModuleList of callable modules that
    holds the targets, replayed with their recorded keyword arguments (stateful cache objects dropped), each
    block's output feeding the next; the last output equals the model's own."""
    try:
        from nncf_b200 import compress_api as api
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"nncf_b200 cannot be imported here: {exc}")
    from types import SimpleNamespace

    from torch import nn

    class FakeCache:
        def __init__(self):
            self.calls = 0

        def get_seq_length(self):
            return 0

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(8, 8, bias=False)
            self.b = nn.Linear(8, 8, bias=False)

        def forward(self, hidden_states, shift=None, past=None, use_cache=False):
            if past is not None:
                past.calls += 1
            return (hidden_states + self.b(torch.tanh(self.a(hidden_states))) + shift,)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.inp = nn.Linear(4, 8, bias=False)
            self.containers = nn.ModuleList([nn.ModuleDict({"x": nn.Linear(8, 8)}), nn.ModuleDict({"x": nn.Linear(8, 8)})])
            self.layers = nn.ModuleList([Block() for _ in range(3)])
            self.out = nn.Linear(8, 2, bias=False)
            self.cache = FakeCache()
            self.trace = []

        def forward(self, x):
            h = self.inp(x)
            shift = torch.full((1, 8), 0.25)
            for layer in self.layers:
                h = layer(h, shift=shift, past=self.cache, use_cache=True)[0]
                self.trace.append(h)
            return self.out(h)

    torch.manual_seed(0)
    model = Model()
    targets = [SimpleNamespace(module=m) for layer in model.layers for m in (layer.a, layer.b)] + \
              [SimpleNamespace(module=model.out)]
    blocks = api._decoder_blocks(model, targets)
    assert blocks is not None and [id(b) for b in blocks] == [id(b) for b in model.layers]
    assert api._decoder_blocks(model, [SimpleNamespace(module=model.out)]) is None
    items = [torch.randn(2, 4), torch.randn(3, 4)]
    with torch.no_grad():
        for item in items:
            model(item)
    want = [model.trace[0:3], model.trace[3:6]]
    replay = api._BlockReplay(model, blocks, items)
    # every block got the very same argument objects as the first one, so only the first item ran through the
    # whole model; the second one stopped at the first block
    assert len(model.trace) == 6 + 3
    calls_after_capture = model.cache.calls
    for bi in range(3):
        outs = [run() for run in replay.runners(bi)]
        for k in range(2):
            torch.testing.assert_close(outs[k][0], want[k][bi])
        replay.advance(bi)
    assert model.cache.calls == calls_after_capture  # the cache object was not passed to the replayed blocks
    # weights changed after the capture are seen by later blocks: the replay runs the live modules
    with torch.no_grad():
        model.layers[0].a.weight.mul_(2.0)
    replay2 = api._BlockReplay(model, blocks, items)
    out0 = replay2.runners(0)[0]()[0]
    assert not torch.allclose(out0, want[0][0])
    # items of one shape [1, T, C] whose other arguments are equal are stacked into micro-batches of at most
    # `batch_tokens` tokens; a stacked call equals the separate calls, and the runner says how to split it
    seq = [torch.randn(1, 5, 4) for _ in range(5)]
    single = api._BlockReplay(model, blocks, seq, batch_tokens=1)
    stacked = api._BlockReplay(model, blocks, seq, batch_tokens=10)
    assert [len(s) for s in single.splits] == [1] * 5 and [len(s) for s in stacked.splits] == [2, 2, 1]
    for bi in range(3):
        a = torch.cat([run()[0] for run in single.runners(bi)], 0)
        b = torch.cat([run()[0] for run in stacked.runners(bi)], 0)
        torch.testing.assert_close(a, b)
        assert [r.split for r in stacked.runners(bi)] == [[1, 1], [1, 1], [1]]
        single.advance(bi)
        stacked.advance(bi)


def test_tied_weights_are_listed_once_and_the_last_layer_counts_as_skipped():
    """A Parameter shared by the embedding and the output head (tied embeddings) must appear once, under the
    module that runs first, with the other holder recorded; the last layer then counts as skipped, so that
    the last *remaining* Linear is not demoted to the backup precision (algorithm.py:540-575, 992-1007)."""
    try:
        from nncf_b200 import CompressWeightsMode
        from nncf_b200.compress_api import _ratio_defining, get_weight_compression_parameters
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"nncf_b200 cannot be imported here: {exc}")

    class Tied(torch.nn.Module):
        def __init__(self, tie: bool):
            super().__init__()
            self.embed = torch.nn.Embedding(32, 16)
            self.a = torch.nn.Linear(16, 16, bias=False)
            self.b = torch.nn.Linear(16, 16, bias=False)
            self.head = torch.nn.Linear(16, 32, bias=False)
            if tie:
                self.head.weight = self.embed.weight

        def forward(self, ids):
            return self.head(self.b(self.a(self.embed(ids))))

    ids = torch.randint(0, 32, (1, 4))
    tied = get_weight_compression_parameters(Tied(True), None, ids)
    assert [p.weight_name for p in tied] == ["embed", "a", "b"]
    assert tied.is_last_layer_skipped
    assert [type(m).__name__ for m in tied[0].shared_modules] == ["Linear"]
    assert [p.weight_name for p in _ratio_defining(tied, CompressWeightsMode.INT4_SYM, False)] == ["a", "b"]
    plain = get_weight_compression_parameters(Tied(False), None, ids)
    assert [p.weight_name for p in plain] == ["embed", "a", "b", "head"]
    assert not plain.is_last_layer_skipped
    assert [p.weight_name for p in _ratio_defining(plain, CompressWeightsMode.INT4_SYM, False)] == ["a", "b"]
    assert [p.weight_name for p in _ratio_defining(plain, CompressWeightsMode.INT4_SYM, True)] == ["a", "b", "head", "embed"]


def test_resumable_block_pauses_at_every_target_and_continues_through_new_weights():
    """One forward per micro-batch, paused at each target layer: the Hessians equal those of separate partial
    runs, a weight replaced while the forwards are paused is the one they continue through, the outputs become
    the next block's inputs, and an error inside a forward reaches the caller."""
    try:
        from nncf_b200 import compress_api as api
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"nncf_b200 cannot be imported here: {exc}")
    from torch import nn

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(8, 8, bias=False)
            self.b = nn.Linear(8, 8, bias=False)

        def forward(self, hidden_states):
            return hidden_states + self.b(torch.tanh(self.a(hidden_states)))

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Block(), Block()])

        def forward(self, x):
            for layer in self.layers:
                x = layer(x)
            return x

    class StubGPTQ:   # the running Hessian of WC/gptq.py:229-236 in plain torch
        def accumulate_hessian(self, H, x, n, batch):
            x = x.reshape(-1, H.shape[-1]).float()
            H.mul_(n / (n + batch)).add_((2.0 / (n + batch)) * (x.T @ x))
            return n + batch

    torch.manual_seed(0)
    model = Model()
    items = [torch.randn(1, 5, 8) for _ in range(5)]
    replay = api._BlockReplay(model, list(model.layers), items, batch_tokens=10)   # micro-batches of 2, 2, 1 items
    inputs = [h.clone() for h in replay.hidden]
    workers = api._ReplayWorkers(len(replay.hidden), torch.device("cpu"))
    try:
        block = model.layers[0]
        run = api._ResumableBlock(workers, replay, 0, [block.a, block.b], StubGPTQ(), False, None)
        Ha, _, n_a = run.hessian(0)
        assert n_a == 5
        xa = torch.cat(inputs, 0).reshape(-1, 8)
        torch.testing.assert_close(Ha, (2.0 / 5) * (xa.T @ xa))
        with torch.no_grad():
            block.a.weight.mul_(0.5)               # "quantise" the first layer while the forwards are paused
        Hb, _, _ = run.hessian(1)
        xb = torch.tanh(block.a(xa))
        torch.testing.assert_close(Hb, (2.0 / 5) * (xb.T @ xb))
        with torch.no_grad():
            block.b.weight.mul_(2.0)
        run.finish()
        with torch.no_grad():
            want = [block(h) for h in inputs]
        for got, w in zip(replay.hidden, want):
            torch.testing.assert_close(got, w)
        # second block: an exception raised inside a paused forward surfaces in the caller, nothing is left hanging
        block2 = model.layers[1]

        def boom(mod, args):
            raise ValueError("broken layer")

        handle = block2.b.register_forward_pre_hook(boom)
        run2 = api._ResumableBlock(workers, replay, 1, [block2.a], StubGPTQ(), False, None)
        run2.hessian(0)
        with pytest.raises(ValueError, match="broken layer"):
            run2.finish()
        handle.remove()
        assert not any(run2.running)
    finally:
        workers.close()
    assert not any(t.is_alive() for t in workers.threads)


def test_same_input_groups_equal_the_reference_schedule():
    """The steps the reference's layer-wise scheduler produced for the toy decoder (stored with the model-level
    GPTQ fixture) are the groups of target layers that receive the identical input tensor."""
    from types import SimpleNamespace

    from conftest import golden
    from models import LAYERWISE, TinyGatedLM, layerwise_ids

    from nncf_b200.compress_api import _same_input_groups

    model = TinyGatedLM(**LAYERWISE["model"]).eval()
    names = [n for n, m in model.named_modules() if isinstance(m, torch.nn.Linear) and n != "head"]
    mods = dict(model.named_modules())
    targets = [SimpleNamespace(weight_name=n, module=mods[n], weight_shape=tuple(mods[n].weight.shape)) for n in names]
    groups = _same_input_groups(model, layerwise_ids()[0], targets)
    got = [",".join(p.weight_name for p in grp) for grp in groups]
    assert got == [str(s) for s in golden("layerwise")["layerwise/int4_sym/steps"]]


def test_factor_of_an_indefinite_hessian_is_reported_by_the_deferred_check():
    """The factorisation's error check does not read a flag back when it runs (the host keeps enqueueing); the
    status travels with the factor and ``check_factor`` raises what ``torch.linalg.cholesky`` would have."""
    from nncf_b200 import gptq as g

    good = torch.eye(64) * 2.0
    w = torch.randn(8, 64)
    hinv = g.GPTQ(0.01).prepare_hessian_inverse(good.clone(), w.clone())
    g.GPTQ.check_factor(hinv)
    bad = good.clone()
    bad[5, 5] = -3.0
    hinv = g.GPTQ(0.01).prepare_hessian_inverse(bad, w.clone())
    with pytest.raises(torch.linalg.LinAlgError):
        g.GPTQ.check_factor(hinv)
