"""pytest configuration: the `gpu` marker, import paths, golden-vector loader."""

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    """GPU tests are skipped, loudly, when no device is visible (they never fall back to CPU)."""
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden(name: str) -> dict:
    """{case: {key: array}} of one committed .npz under tests/golden."""
    out = {}
    with np.load(GOLDEN / name) as z:
        for k in z.files:
            case, key = k.split("/") if "/" in k else ("", k)
            out.setdefault(case, {})[key] = z[k]
    return out
