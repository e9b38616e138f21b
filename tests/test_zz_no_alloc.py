"""dlrb200_forward_static: the small-batch forward for callers that cannot allocate.

A host whose device-memory budget is fixed at start-up (or a plain C caller with
no allocator) cannot provide the workspace dlrb200_forward asks for, and must
not trigger a cudaMalloc while serving; this entry point keeps its scratch in a
fixed array inside the library.  The test drives it through the C ABI and
checks it against the regular entry point on two consecutive calls, which share
that array.  Collected last on purpose (file name), runs alone as well.
"""
import ctypes

import pytest
import torch

from oracle import dlrnet_oracle as O

pytestmark = pytest.mark.gpu

TOL = 1e-3   # with the regular entry point held to the striped kernel both run the same code; only the order of fp32 atomics differs


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("d,r,L,M", [(1024, 32, 9, 5), (2048, 64, 7, 64), (512, 256, 4, 17)])
def test_static_entry_point_matches_regular_one_twice(d, r, L, M, monkeypatch):
    import dlr_lock_b200 as D
    monkeypatch.setenv("DLRB200_FORCE_PATH", "1")       # the regular entry point would pick another kernel for some of these shapes
    lib = D.ops._lib.load()
    dev = torch.device("cuda:0")
    p, x = O.seeded_case(d, r, L, 2 * M, seed=d + r + M, alpha=1.0, gain_jitter=0.1)
    Vp, Up = D.ops.fold_weights(p.V.to(dev), p.U.to(dev), p.w.to(dev), p.alpha.to(dev))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    xs = [x[:M].contiguous().to(dev), x[M:].contiguous().to(dev)]
    for call, xd in enumerate(xs):                      # two calls in a row share the built-in scratch
        want = D.ops.forward_folded(xd, Vp, Up, p.eps)
        got = torch.empty_like(xd)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)       # the driver's count: sees any cudaMalloc, torch's or not
        torch_before = torch.cuda.memory_allocated(dev)
        rc = lib.dlrb200_forward_static(_vp(xd), _vp(got), _vp(Vp), _vp(Up), M, d, r, L, ctypes.c_float(p.eps),
                                        _vp(status), stream)
        assert rc == 0, lib.dlrb200_strerror(rc)
        torch.cuda.synchronize()
        if call > 0:
            # the property in the entry point's name: no device memory was taken, by any allocator (the very
            # first call on a device may still load the kernel's module, which the driver accounts as memory)
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        assert torch.cuda.memory_allocated(dev) == torch_before
        assert int(status.item()) == 0
        assert O.rel_l2(got.cpu(), want.cpu()) <= TOL, f"call {call}"
        assert O.rel_l2(got.cpu(), O.forward_fp32(x[call * M:(call + 1) * M], p)) <= 5e-3


def test_static_entry_point_rejects_what_does_not_fit():
    import dlr_lock_b200 as D
    lib = D.ops._lib.load()
    null = ctypes.c_void_p(0)
    # 65 rows do not fit the built-in scratch: refused before anything is launched
    rc = lib.dlrb200_forward_static(null, null, null, null, 65, 1024, 32, 4, ctypes.c_float(1e-6), null, null)
    assert rc == 9
    assert b"built-in scratch" in lib.dlrb200_strerror(rc)
    assert lib.dlrb200_forward_static(null, null, null, null, 8, 1024, 100, 4, ctypes.c_float(1e-6), null, null) == 2
    assert lib.dlrb200_forward_static(null, null, null, null, 0, 1024, 32, 4, ctypes.c_float(1e-6), null, null) == 0
