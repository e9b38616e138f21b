"""The C-ABI library loads and exports what include/dlr_b200.h declares (no GPU)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT

from dlr_lock_b200 import _lib
from dlr_lock_b200.build import build_library


@pytest.fixture(scope="module")
def lib():
    build_library()
    return _lib.load()


def _declared():
    text = open(os.path.join(ROOT, "include", "dlr_b200.h")).read()
    return sorted(set(re.findall(r"DLRB200_API[^;(]*?\b(dlrb200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared()
    assert len(names) >= 9
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_text(lib):
    assert lib.dlrb200_version() >= 100
    assert lib.dlrb200_strerror(0) == b"ok"
    for code in range(1, 9):
        assert lib.dlrb200_strerror(code) not in (b"ok", b"unknown error")
    assert lib.dlrb200_strerror(99) == b"unknown error"


def test_workspace_bytes_and_shape_rejection(lib):
    assert lib.dlrb200_workspace_bytes(8, 4096, 128, 143) % 256 == 0
    assert lib.dlrb200_workspace_bytes(8, 4096, 128, 143) > 0
    assert lib.dlrb200_workspace_bytes(8, 4096, 100, 143) == 0   # rank not supported
    assert lib.dlrb200_workspace_bytes(8, 4100, 128, 143) == 0   # width not a multiple of 16
    # argument checks come before any CUDA call
    null = ctypes.c_void_p(0)
    assert lib.dlrb200_forward(null, null, null, null, 8, 4096, 100, 143, 1e-6, null, 0, null, null) == 2
    assert lib.dlrb200_forward(null, null, null, null, -1, 4096, 128, 143, 1e-6, null, 0, null, null) == 1
    assert lib.dlrb200_forward(null, null, null, null, 8, 4096, 128, 143, 1e-6, null, 0, null, null) == 1
    assert lib.dlrb200_forward(null, null, null, null, 0, 4096, 128, 143, 1e-6, null, 0, null, null) == 0
