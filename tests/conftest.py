import json
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (select with -m gpu)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Outputs of the reference's own oracles (tests/golden/make_golden.py)."""

    def __init__(self):
        base = ROOT / "tests" / "golden"
        self.index = json.loads((base / "reference_index.json").read_text())
        self.arrays = np.load(base / "reference_outputs.npz")

    def bf16(self, key):
        return torch.from_numpy(self.arrays[key].copy()).view(torch.bfloat16)

    def fp32(self, key):
        return torch.from_numpy(self.arrays[key].copy()).view(torch.float32)

    def int32(self, key):
        return torch.from_numpy(self.arrays[key].copy())


@pytest.fixture(scope="session")
def golden():
    return Golden()


def sha256(t: torch.Tensor) -> str:
    import hashlib
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


_moe_cache = {}


def moe_reference_case(case):
    """Materialising a reference MoE case draws ~1.4 G random numbers; keep the last one."""
    from oracle import moe
    if case not in _moe_cache:
        _moe_cache.clear()
        _moe_cache[case] = moe.materialize_reference_case(case)
    return _moe_cache[case]
