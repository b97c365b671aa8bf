"""pytest configuration: the `gpu` marker, import paths, and shared helpers."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "fused-layernorm-cuda-operator_b200"
for p in (str(ROOT), str(PKG)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


TORCH_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


class Golden:
    """tests/golden/torch_cpu_golden.npz as torch tensors."""

    def __init__(self, path):
        self.z = np.load(path)
        self.names = sorted({k.split("/")[0] for k in self.z.files})

    def case(self, name):
        dt = TORCH_DT[str(self.z[f"{name}/dtype"])]
        out = {"dtype": dt, "kind": str(self.z[f"{name}/kind"]), "eps": float(self.z[f"{name}/eps"])}
        for k in self.z.files:
            if not k.startswith(name + "/"):
                continue
            f = k.split("/", 1)[1]
            if f in ("dtype", "kind", "eps"):
                continue
            a = self.z[k]
            if a.dtype == np.uint16:
                t = torch.from_numpy(a.view(np.int16).copy()).view(dt)
            else:
                t = torch.from_numpy(a.copy())
            out[f] = t
        for f in ("gamma", "beta", "res", "sum", "mean", "dbeta", "dgamma"):
            out.setdefault(f, None)
        return out

    def raw(self, key):
        return self.z[key]


@pytest.fixture(scope="session")
def golden():
    return Golden(ROOT / "tests" / "golden" / "torch_cpu_golden.npz")
