"""ctypes binding of ``libdlr_b200.so`` (the C ABI declared in include/dlr_b200.h).

There is no CPU or framework fallback behind this module: if the shared library
has not been built, loading raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdlr_b200.so")

OK = 0
ERR_TEXT_FALLBACK = "dlr_b200 error"


class Plan(ctypes.Structure):
    """Mirror of ``dlrb200_plan``."""

    _fields_ = [
        ("path", ctypes.c_int), ("grid", ctypes.c_int), ("cluster", ctypes.c_int),
        ("stripe_cols", ctypes.c_int), ("rows_per_pass", ctypes.c_int), ("passes", ctypes.c_int),
        ("stages", ctypes.c_int), ("smem_bytes", ctypes.c_size_t), ("workspace_bytes", ctypes.c_size_t),
    ]


# name -> (restype, argtypes); one entry per declaration in include/dlr_b200.h
_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
SIGNATURES = {
    "dlrb200_version": (_i, []),
    "dlrb200_strerror": (ctypes.c_char_p, [_i]),
    "dlrb200_last_cuda_error": (_i, []),
    "dlrb200_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "dlrb200_query": (_i, [_i, _i, _i, _i, ctypes.POINTER(Plan)]),
    "dlrb200_forward": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp, _sz, _vp, _vp]),
    "dlrb200_forward_host": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp, _sz, _vp, _vp]),
    "dlrb200_fold_weights": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "dlrb200_transpose_stack": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "dlrb200_status_to_host": (_i, [_vp, _vp, _vp]),
    "dlrb200_forward_static": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp, _vp]),
}

_lib = None
_lock = threading.Lock()


class DlrB200Error(RuntimeError):
    """A C-ABI call returned a non-zero code, or the device status word was set."""

    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(what)


def load() -> ctypes.CDLL:
    """Load the shared library (once) and declare every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dlr_lock_b200.build` "
                "(nvcc, sm_100a). There is no fallback path.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def strerror(code: int) -> str:
    try:
        return load().dlrb200_strerror(int(code)).decode()
    except Exception:  # pragma: no cover - only if the library itself is broken
        return ERR_TEXT_FALLBACK


def check(code: int, where: str) -> None:
    """Raise DlrB200Error for a non-zero return code."""
    if code != OK:
        lib = load()
        extra = ""
        if code == 6:
            extra = f" [cuda error {lib.dlrb200_last_cuda_error()}]"
        raise DlrB200Error(code, f"{where}: {strerror(code)}{extra}")
