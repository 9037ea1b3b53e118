"""Shared pytest configuration: the `gpu` marker, fixture loading and import paths."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"
if str(GOLDEN) not in sys.path:
    sys.path.insert(0, str(GOLDEN))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch

        have_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Read access to one fixture file written by tests/golden/make_golden.py."""

    def __init__(self, name: str):
        self._z = np.load(GOLDEN / f"{name}.npz", allow_pickle=False)

    def __contains__(self, key: str) -> bool:
        return key.replace("/", "|") in self._z.files

    def __getitem__(self, key: str) -> np.ndarray:
        return self._z[key.replace("/", "|")]

    def index(self, group: str) -> list[str]:
        return [str(s) for s in self[f"{group}/index"]]


_cache: dict[str, Golden] = {}


def golden(name: str) -> Golden:
    if name not in _cache:
        _cache[name] = Golden(name)
    return _cache[name]
