"""Tensor-level entry points: torch supplies device memory and the stream, the
arithmetic happens in ``libdlr_b200.so``.

Calling conventions mirrored from the reference kernels:

* ``forward_folded(x, Vp, Up)``      - this library's own layouts
  (V' (L,r,d), U' (L,d,r)).
* ``forward_xvu(x, Vs, Us)``         - the reference CUDA wrappers' convention,
  e.g. ``cooperative_forward(x, Vs, Us)`` with both stacks (L, R, D)
  (kernels/kernels/cooperative.py:41-68).
* ``dlrnet_fused(x, weights)``       - the reference Triton convention, taking
  the dict of ``pack_dlrnet_weights`` (kernels/kernels/triton_fused.py:68-92).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Tuple

import torch

from . import _lib

EPS = 1e-6

class _Scratch:
    """Per (device, stream): workspace, device status word and its pinned host mirror."""

    __slots__ = ("ws", "status", "status_host", "retired")

    def __init__(self, device: torch.device, nbytes: int):
        self.ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        # workspaces that were outgrown: a CUDA graph captured earlier has their address in its nodes, so
        # they stay allocated for the life of the process (they are small: at most a few tens of MB)
        self.retired = []


_workspaces: Dict[Tuple[int, int], _Scratch] = {}
_derived: Dict[Tuple, Tuple[torch.Tensor, ...]] = {}
_MIN_WORKSPACE = 1 << 20


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _raise_status(ent: _Scratch, word: int):
    ent.status_host.zero_()
    ent.status.zero_()          # a non-zero word makes later calls give up early: clear it before reporting
    raise _lib.DlrB200Error(word & 0xff, f"device status: {_lib.strerror(word & 0xff)} at layer {word >> 8}")


def _workspace(device: torch.device, nbytes: int) -> _Scratch:
    """Scratch + status word for the current (device, stream); grown on demand.

    One workspace per stream, because calls that share one must not overlap.  A workspace that is outgrown
    is kept, not freed: a CUDA graph captured while it was current still clears and uses that memory on
    every replay.  Also the lazy error check: the status word of the calls before, mirrored to pinned host
    memory by a copy on the stream after every forward, is looked at here without synchronising.
    """
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    ent = _workspaces.get(key)
    if ent is None:
        ent = _Scratch(device, max(nbytes, _MIN_WORKSPACE))
        _workspaces[key] = ent
    else:
        word = int(ent.status_host[0])
        if word != 0 and not torch.cuda.is_current_stream_capturing():
            _raise_status(ent, word)
        if ent.ws.numel() < nbytes:
            ent.retired.append(ent.ws)
            ent.ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return ent


def _mirror_status(lib, ent: _Scratch, device: torch.device) -> None:
    """Queue the 4-byte copy of the status word to its pinned host mirror behind the forward."""
    rc = lib.dlrb200_status_to_host(_ptr(ent.status), ctypes.c_void_p(ent.status_host.data_ptr()),
                                    _stream_ptr(device))
    _lib.check(rc, "dlrb200_status_to_host")


def check_status(device=None) -> None:
    """Synchronise and raise if a bounded device-side wait gave up on `device`.

    Without this call a timeout still surfaces, one call late: every forward mirrors the status word to
    pinned host memory on its stream, and the next forward on that stream looks at the mirror first.
    """
    for (dev, _), ent in list(_workspaces.items()):
        if device is not None and torch.device(device).index not in (None, dev):
            continue
        word = int(ent.status.item())
        if word != 0:
            _raise_status(ent, word)


def _check_inputs(x, Vp, Up):
    if not (x.is_cuda and Vp.is_cuda and Up.is_cuda):
        raise ValueError("dlr_b200 runs on CUDA tensors only (there is no CPU path)")
    if not (x.dtype == Vp.dtype == Up.dtype == torch.bfloat16):
        raise TypeError("dlr_b200 takes bfloat16 activations and folded weights")
    if Vp.dim() != 3 or Up.dim() != 3:
        raise ValueError("folded weights must be V' (L,r,d) and U' (L,d,r)")
    L, r, d = Vp.shape
    if tuple(Up.shape) != (L, d, r):
        raise ValueError(f"U' has shape {tuple(Up.shape)}, expected {(L, d, r)}")
    if x.shape[-1] != d:
        raise ValueError(f"last dimension of x is {x.shape[-1]}, expected d={d}")
    if not (Vp.is_contiguous() and Up.is_contiguous()):
        raise ValueError("folded weights must be contiguous")
    return L, r, d


def forward_folded(x: torch.Tensor, Vp: torch.Tensor, Up: torch.Tensor, eps: float = EPS,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """y = DLRNet(x) on folded weights; x is (..., d) bf16 on CUDA, y is a new tensor.

    Asynchronous on the current stream.  A device-side timeout is reported by
    ``check_status`` (which synchronises) or, without a synchronisation, by the
    next forward on the same stream that runs after the failed one has finished.
    """
    L, r, d = _check_inputs(x, Vp, Up)
    lib = _lib.load()
    x2 = x.reshape(-1, d)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    M = x2.shape[0]
    y2 = torch.empty_like(x2) if out is None else out.view(-1, d)
    if M == 0:
        return y2.view(x.shape)
    with torch.cuda.device(x.device):
        need = lib.dlrb200_workspace_bytes(M, d, r, L)
        if need == 0:
            _lib.check(2, f"dlrb200_forward(M={M}, d={d}, r={r}, L={L})")
        ent = _workspace(x.device, need)
        rc = lib.dlrb200_forward(_ptr(x2), _ptr(y2), _ptr(Vp), _ptr(Up), M, d, r, L, float(eps),
                                 _ptr(ent.ws), ent.ws.numel(), _ptr(ent.status), _stream_ptr(x.device))
        _lib.check(rc, f"dlrb200_forward(M={M}, d={d}, r={r}, L={L})")
        _mirror_status(lib, ent, x.device)
    return y2.view(x.shape)


def forward_host(x_host: torch.Tensor, y_host: torch.Tensor, x_dev: torch.Tensor, y_dev: torch.Tensor,
                 Vp: torch.Tensor, Up: torch.Tensor, eps: float = EPS) -> None:
    """Forward with activations in (pinned) host memory; copies ride the current stream."""
    L, r, d = Vp.shape
    M = x_host.numel() // d
    lib = _lib.load()
    with torch.cuda.device(Vp.device):
        need = lib.dlrb200_workspace_bytes(M, d, r, L)
        ent = _workspace(Vp.device, need)
        rc = lib.dlrb200_forward_host(_ptr(x_host), _ptr(y_host), _ptr(x_dev), _ptr(y_dev), _ptr(Vp), _ptr(Up),
                                      M, d, r, L, float(eps), _ptr(ent.ws), ent.ws.numel(), _ptr(ent.status),
                                      _stream_ptr(Vp.device))
        _lib.check(rc, "dlrb200_forward_host")
        _mirror_status(lib, ent, Vp.device)


def query(M: int, d: int, r: int, L: int) -> _lib.Plan:
    """How a forward of this shape would run on the current CUDA device."""
    plan = _lib.Plan()
    _lib.check(_lib.load().dlrb200_query(M, d, r, L, ctypes.byref(plan)), "dlrb200_query")
    return plan


def fold_weights(V: torch.Tensor, U: torch.Tensor, gain: torch.Tensor, alpha: torch.Tensor):
    """Stacked (L,r,d)/(L,d,r)/(L,d)/(L,) parameters -> folded bf16 (V', U') on the device.

    Same rounding as the reference packer (kernels/reference.py:73-79): V, U and
    the gain are rounded to bf16 first, alpha goes through the parameter dtype to
    fp32, products are formed in fp32 and rounded once.
    """
    if not V.is_cuda:
        raise ValueError("fold_weights runs on CUDA tensors only")
    L, r, d = V.shape
    Vb = V.detach().to(torch.bfloat16).contiguous()
    Ub = U.detach().to(torch.bfloat16).contiguous()
    gb = gain.detach().to(torch.bfloat16).contiguous()
    af = alpha.detach().to(torch.float32).contiguous()
    Vp = torch.empty_like(Vb)
    Up = torch.empty_like(Ub)
    with torch.cuda.device(V.device):
        rc = _lib.load().dlrb200_fold_weights(_ptr(Vb), _ptr(Ub), _ptr(gb), _ptr(af), _ptr(Vp), _ptr(Up),
                                              d, r, L, _stream_ptr(V.device))
    _lib.check(rc, "dlrb200_fold_weights")
    return Vp, Up


def transpose_stack(src: torch.Tensor) -> torch.Tensor:
    """(L, rows, cols) bf16 -> (L, cols, rows), on the device."""
    L, rows, cols = src.shape
    src = src.contiguous()
    dst = torch.empty((L, cols, rows), dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        rc = _lib.load().dlrb200_transpose_stack(_ptr(src), _ptr(dst), L, rows, cols, _stream_ptr(src.device))
    _lib.check(rc, "dlrb200_transpose_stack")
    return dst


def _cached_transpose(t: torch.Tensor) -> torch.Tensor:
    key = ("T", t.data_ptr(), t._version, tuple(t.shape), t.device.index)
    hit = _derived.get(key)
    if hit is None:
        if len(_derived) > 64:
            _derived.clear()
        hit = (transpose_stack(t),)
        _derived[key] = hit
    return hit[0]


def forward_xvu(x: torch.Tensor, Vs: torch.Tensor, Us: torch.Tensor) -> torch.Tensor:
    """Reference CUDA-wrapper convention: Vs (L,R,D) and Us (L,R,D), both folded.

    Us is U'^T there; its transpose is derived on the device once per weight
    tensor and cached.  Any B >= 1 is accepted (no padding needed).
    """
    if Vs.dim() != 3 or Us.shape != Vs.shape:
        raise ValueError("expected Vs (L,R,D) and Us (L,R,D)")
    return forward_folded(x, Vs.contiguous(), _cached_transpose(Us))


def dlrnet_fused(x: torch.Tensor, weights: dict, **_ignored) -> torch.Tensor:
    """Reference Triton convention: `weights` is the dict of pack_dlrnet_weights
    with Vs (L,D,R) = V'^T and Us (L,R,D) = U'^T, premultiplied."""
    if not weights.get("premultiplied", False):
        raise ValueError("dlrnet_fused needs premultiplied weights (pack with premultiply=True)")
    return forward_folded(x, _cached_transpose(weights["Vs"]), _cached_transpose(weights["Us"]))
