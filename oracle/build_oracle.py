"""Compile oracle/dlrnet_oracle.c into oracle/liboracle_c.so with gcc.
TEST INFRASTRUCTURE ONLY (see the header of dlrnet_oracle.c)."""
import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "dlrnet_oracle.c")
LIB = os.path.join(HERE, "liboracle_c.so")


def build(force: bool = False) -> str:
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-o", LIB, SRC, "-lm"], check=True)
    return LIB


def load() -> ctypes.CDLL:
    lib = ctypes.CDLL(build())
    fp = ctypes.POINTER(ctypes.c_float)
    lib.dlrnet_forward_f32.restype = ctypes.c_int
    lib.dlrnet_forward_f32.argtypes = [fp, fp, fp, fp, fp, fp] + [ctypes.c_int] * 4 + [ctypes.c_float]
    return lib


def forward_f32(x, V, U, w, alpha, eps=1e-6):
    """numpy fp32 arrays: x (M,d), V (L,r,d), U (L,d,r), w (L,d), alpha (L,) -> y (M,d)."""
    import numpy as np

    lib = load()
    x, V, U, w, alpha = (np.ascontiguousarray(a, dtype=np.float32) for a in (x, V, U, w, alpha))
    M, d = x.shape
    L, r, _ = V.shape
    y = np.empty_like(x)
    fp = ctypes.POINTER(ctypes.c_float)
    rc = lib.dlrnet_forward_f32(*(a.ctypes.data_as(fp) for a in (x, y, V, U, w, alpha)), M, d, r, L, eps)
    if rc != 0:
        raise MemoryError("dlrnet_forward_f32 failed")
    return y


if __name__ == "__main__":
    print(build(force=True))
