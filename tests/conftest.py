import json
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "ml-dlr-lock_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def load_golden(name: str):
    """Fixture written by tests/golden/make_golden.py: meta dict, x, reference outputs."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    meta = json.loads(str(z["meta"]))
    out = dict(meta=meta, x=bf16_from_bits(z["x_bits"]), y_bf16=bf16_from_bits(z["y_bf16_bits"]),
               y_fp32=torch.from_numpy(z["y_fp32"].copy()))
    if "packed_Vs_bits" in z:
        out["packed_Vs"] = bf16_from_bits(z["packed_Vs_bits"])
        out["packed_Us"] = bf16_from_bits(z["packed_Us_bits"])
    return out


@pytest.fixture(scope="session")
def golden():
    return load_golden
