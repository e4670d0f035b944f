import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG_ROOT = os.path.join(ROOT, "titanmac-standalone_b200")
for p in (ROOT, PKG_ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


class Golden:
    """Read-only view of one .npz fixture: ``g[case, field]`` → torch tensor."""

    def __init__(self, path):
        self._z = np.load(path)
        self.cases = sorted({k.split("/")[0] for k in self._z.files})

    def has(self, case, field):
        return f"{case}/{field}" in self._z.files

    def np(self, case, field):
        return self._z[f"{case}/{field}"]

    def __getitem__(self, key):
        case, field = key
        return torch.from_numpy(self._z[f"{case}/{field}"])

    def meta(self, case):
        B, T, H, dh, w, Np, seed = (int(v) for v in self._z[f"{case}/meta"])
        return dict(B=B, T=T, H=H, dh=dh, w=w, Np=Np, seed=seed, L=Np + T, D=H * dh)


@pytest.fixture(scope="session")
def golden():
    return Golden(os.path.join(GOLDEN_DIR, "windowed_attention_golden.npz"))


@pytest.fixture(scope="session")
def golden_model():
    return Golden(os.path.join(GOLDEN_DIR, "titanmac_golden.npz"))


FULL_CASES = ["tiny_w3", "ragged_w16", "self_only_w0", "window_exceeds_len", "one_persistent_row_short",
              "dh64_multi_tile", "dh128_multi_tile", "dh64_np8_w129"]
CORE_CASES = ["tiny_w3", "ragged_w16", "dh64_multi_tile"]
