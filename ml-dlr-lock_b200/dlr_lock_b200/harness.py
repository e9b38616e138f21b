"""Per-cell parity gate and timing protocol for the DLR-Net forward, in the form of the
reference's kernel benchmark (kernels/bench/bench_paper.py, kernels/bench/_protocol.py).

    python -m dlr_lock_b200.harness --models Qwen3-8B --batch-sizes 1 64 8192 --out cells.json

For every (model, batch size) cell: build the benchmark twin of the net
(``build_models(name, seed=42)``, kernels/reference.py:94-102: alpha 0.01, gains 1, bf16),
run the torch module on the GPU as the reference output, run the registry's callable for the
cell, gate it on relative L2 error (``ok`` / ``WRONG`` / ``OOM`` / ``ERROR``, bench_paper.py:122-147)
and time it with the reference's protocol: after a warm-up, the minimum over ``n_iters`` single
calls is one pass, and the mean and standard deviation over ``n_passes`` passes are reported
(_protocol.py:83-142).  Clocks are not locked here (a shared machine): the sampled SM clock is
recorded instead.

The module also builds the two library-only baselines the reference measures its kernels
against on the same machine: the torch module under ``torch.compile(mode="reduce-overhead")``
(bench_paper.py:178) and the cuBLAS + elementwise loop captured in one CUDA graph
(kernels/kernels/orchestrated.py:95-126).  They are comparison figures, not part of the product
path.
"""
from __future__ import annotations

import argparse
import gc
import importlib
import json
import math
import statistics
from typing import Callable, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import registry
from .model import DLRNet, compute_depth

DTYPE = torch.bfloat16
REL_ERR_TOL = 2e-2          # kernels/bench/bench_paper.py:43
N_WARMUP, N_ITERS, N_PASSES = 100, 100, 10      # kernels/bench/_protocol.py:28
DEFAULT_B = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384, 32768, 65536, 131072]


class SwiGLU(nn.Module):
    """The MLP a DLR-Net replaces (kernels/reference.py:35-43): down(silu(gate(x)) * up(x))."""

    def __init__(self, d: int, d_ff: int):
        super().__init__()
        self.gate_proj = nn.Linear(d, d_ff, bias=False)
        self.up_proj = nn.Linear(d, d_ff, bias=False)
        self.down_proj = nn.Linear(d_ff, d, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


def build_models(name: str = "Qwen3-0.6B", seed: int = 42, device="cuda"):
    """(swiglu, dlrnet, cfg) for one benchmark shape, as kernels/reference.py:94-102.

    The benchmark twin of the net draws all U first, then all V (kernels/reference.py:50-53), with
    alpha 0.01 and unit gains; the same seed therefore gives the same weights as the reference's bench.
    """
    cfg = registry.MODEL_CONFIGS[name]
    d, d_ff, r = cfg["d"], cfg["d_ff"], cfg["r"]
    depth = compute_depth(d, d_ff, r)
    torch.manual_seed(seed)
    swiglu = SwiGLU(d, d_ff).to(DTYPE).to(device)
    torch.manual_seed(seed)
    u_scale, v_scale = 1.0 / math.sqrt(r * depth), 1.0 / math.sqrt(d)
    us = [torch.randn(d, r) * u_scale for _ in range(depth)]
    vs = [torch.randn(r, d) * v_scale for _ in range(depth)]
    net = DLRNet(d, r, depth, alpha_init=0.01)
    with torch.no_grad():
        for i in range(depth):
            net.Us[i].copy_(us[i])
            net.Vs[i].copy_(vs[i])
    net = net.to(DTYPE).to(device).eval()
    for p in net.parameters():
        p.requires_grad_(False)
    return swiglu.eval(), net, {"d": d, "d_ff": d_ff, "r": r, "depth": depth}


@torch.no_grad()
def pack_dlrnet_weights(net: nn.Module, premultiply: bool = True) -> Dict:
    """The reference's packed-weights dict (kernels/reference.py:68-91): ``Vs`` (L, D, R) = V^T,
    ``Us`` (L, R, D) = U^T, ``Ws`` (L, D), ``As`` (L,), and ``L``, ``D``, ``R``, ``premultiplied``;
    with ``premultiply`` the gain is folded into V and alpha into U in fp32, rounded once."""
    V = torch.stack([p.detach() for p in net.Vs]).to(DTYPE)
    U = torch.stack([p.detach() for p in net.Us]).to(DTYPE)
    W = torch.stack([p.detach() for p in net.rms_w]).to(DTYPE)
    A = torch.stack([p.detach() for p in net.alphas]).float()
    if premultiply:
        V = (V.float() * W.float()[:, None, :]).to(DTYPE)
        U = (U.float() * A[:, None, None]).to(DTYPE)
    L, R, D = V.shape
    return {"Vs": V.transpose(1, 2).contiguous(), "Us": U.transpose(1, 2).contiguous(), "Ws": W.contiguous(),
            "As": A.contiguous(), "L": L, "D": D, "R": R, "premultiplied": premultiply}


# --------------------------------------------------------------------------- #
# timing protocol
# --------------------------------------------------------------------------- #
def bench_pass(fn: Callable[[], object], n: int, warmup: int):
    """Per-call device times (microseconds) of ``n`` calls after ``warmup`` untimed ones."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(n):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    return times


def measure(fn: Callable[[], object], passes: int = N_PASSES, n_iters: int = N_ITERS, n_warmup: int = N_WARMUP) -> Dict:
    """Minimum of ``n_iters`` calls per pass; mean and spread over ``passes`` passes."""
    mins, every = [], []
    for _ in range(passes):
        ts = bench_pass(fn, n_iters, n_warmup)
        mins.append(min(ts))
        every.extend(ts)
    return {"mean_us": statistics.fmean(mins), "std_us": statistics.pstdev(mins) if len(mins) > 1 else 0.0,
            "median_us": sorted(mins)[len(mins) // 2], "pass_mins_us": mins,
            "iter_mean_us": statistics.fmean(every), "iter_std_us": statistics.pstdev(every)}


def free_all():
    gc.collect()
    torch.cuda.empty_cache()
    torch.cuda.synchronize()


def rel_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    return float((out.float() - ref.float()).norm() / ref.float().norm())


def update_err(out: torch.Tensor, ref: torch.Tensor, x: torch.Tensor) -> float:
    """Error of the update ``y - x`` relative to the reference's update: with the benchmark's alpha the
    stack moves its input by well under a percent, so a kernel that returns its input passes the
    total-error gate; here it scores 1."""
    den = float((ref.float() - x.float()).norm())
    return float((out.float() - ref.float()).norm()) / den if den > 0 else 0.0


# --------------------------------------------------------------------------- #
# cells
# --------------------------------------------------------------------------- #
def _import_callable(path: str):
    mod, fn = path.rsplit(".", 1)
    return getattr(importlib.import_module(mod), fn)


def build_run(entry: Dict, x: torch.Tensor, weights: Dict) -> Callable[[], torch.Tensor]:
    """Zero-argument callable for a registry entry: the ``fn(x, Vs, Us)`` convention with both stacks
    (L, R, D) (kernels/bench/bench_paper.py:97-101); set-up happens here, outside the timed region."""
    fn = _import_callable(entry["callable"])
    Vs = weights["Vs"].transpose(-1, -2).contiguous()      # (L, D, R) -> (L, R, D)
    Us = weights["Us"]
    fn(x, Vs, Us)                                           # derived layouts are cached by the callable
    return lambda: fn(x, Vs, Us)


def run_cell(kernel: str, run_factory: Callable[[], Callable[[], torch.Tensor]], x: torch.Tensor, ref: torch.Tensor,
             baseline_us: Optional[float] = None, ref32: Optional[torch.Tensor] = None, **measure_kw) -> Dict:
    """Build, gate and time one cell (kernels/bench/bench_paper.py:126-147).  ``ref`` is the torch module's
    bf16 output (the reference's gate); ``ref32`` its fp32 output on the same bf16 weights, against which the
    update error is also reported: the bf16 module itself is most of the small update away from the fp32 one,
    so a kernel that carries the activation in fp32 is judged against the latter."""
    try:
        run = run_factory()
        out = run()
        torch.cuda.synchronize()
        err = rel_err(out, ref)
        if not err <= REL_ERR_TOL:
            return {"kernel": kernel, "status": "WRONG", "rel_err": err}
        stats = measure(run, **measure_kw)
        stats.update({"kernel": kernel, "status": "ok", "rel_err": err, "update_err": update_err(out, ref, x),
                      "ratio": stats["mean_us"] / baseline_us if baseline_us else None})
        if ref32 is not None:
            stats["update_err_fp32_ref"] = update_err(out, ref32.to(out.dtype), x)
        return stats
    except torch.cuda.OutOfMemoryError:
        free_all()
        return {"kernel": kernel, "status": "OOM"}
    except Exception as e:  # noqa: BLE001 - the harness reports, it does not stop the sweep
        free_all()
        return {"kernel": kernel, "status": f"ERROR: {type(e).__name__}: {e}"}
    finally:
        free_all()


# --------------------------------------------------------------------------- #
# library-only baselines on the same machine
# --------------------------------------------------------------------------- #
def compiled_reduce_overhead(net: nn.Module):
    """The torch layer loop under ``torch.compile(mode="reduce-overhead")``: fused elementwise kernels and
    the whole stack replayed from a CUDA graph (kernels/bench/bench_paper.py:174-178)."""
    loop = _TorchLoop(net)
    return torch.compile(loop, mode="reduce-overhead")


class _TorchLoop(nn.Module):
    """``DLRNet._forward_impl`` as a module of its own, so that compiling it does not touch the product's
    dispatch in ``DLRNet.forward``."""

    def __init__(self, net: nn.Module):
        super().__init__()
        self.net = net

    def forward(self, x):
        return self.net._forward_impl(x)


def orchestrated_graph(x: torch.Tensor, weights: Dict, eps: float = 1e-6):
    """Per layer one library GEMM into ``z``, one elementwise step ``z = silu(z * rstd(h))``, one library GEMM
    accumulating into ``h`` (``addmm_``), the whole stack captured in one CUDA graph
    (kernels/kernels/orchestrated.py:95-126; the reference's elementwise step is a Triton kernel, here it is
    torch ops inside the graph).  Returns (graph, output buffer)."""
    if not weights.get("premultiplied", False):
        raise ValueError("orchestrated_graph needs premultiplied weights")
    Vs, Us, L = weights["Vs"], weights["Us"], weights["L"]
    h = x.clone()
    z = torch.empty(x.shape[0], weights["R"], device=x.device, dtype=x.dtype)

    def step():
        h.copy_(x)
        for l in range(L):
            torch.matmul(h, Vs[l], out=z)
            rstd = torch.rsqrt(h.float().pow(2).mean(dim=-1, keepdim=True) + eps)
            z.copy_(F.silu(z.float() * rstd))
            h.addmm_(z, Us[l])

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph), torch.no_grad():
        step()
    return graph, h


# --------------------------------------------------------------------------- #
# sweep
# --------------------------------------------------------------------------- #
def sweep(models, batch_sizes, passes=N_PASSES, n_iters=N_ITERS, n_warmup=N_WARMUP, baselines=("swiglu",)):
    """{model: {B: row}}: per cell the SwiGLU baseline (eager module), the optional library-only DLR-Net
    baselines, and the registry's kernel for the cell, each gated and timed."""
    kw = dict(passes=passes, n_iters=n_iters, n_warmup=n_warmup)
    results = {}
    for model in models:
        swiglu, net, cfg = build_models(model)
        weights = pack_dlrnet_weights(net, premultiply=True)
        results[model] = {}
        compiled = compiled_reduce_overhead(net) if "compile" in baselines else None
        import copy
        net32 = copy.deepcopy(net).float()
        for B in batch_sizes:
            free_all()
            row = {"cells": []}
            try:
                x = torch.randn(B, cfg["d"], device="cuda", dtype=DTYPE)
                with torch.no_grad():
                    net.fast = False
                    ref = net(x)
                    net.fast = True
                    ref32 = net32._forward_impl(x.float())
                    sw = measure(lambda: swiglu(x), **kw) if "swiglu" in baselines else None
            except torch.cuda.OutOfMemoryError:
                results[model][B] = {"status": "OOM building baseline"}
                free_all()
                continue
            row["SwiGLU"] = sw
            base = sw["mean_us"] if sw else None
            if compiled is not None:
                with torch.no_grad():
                    row["cells"].append(run_cell("torch_compile_reduce_overhead", lambda: (lambda: compiled(x)), x, ref, base, ref32, **kw))
            if "orchestrated" in baselines:
                def make():
                    g, hbuf = orchestrated_graph(x, weights)
                    return lambda: (g.replay(), hbuf)[1]
                row["cells"].append(run_cell("cublas_graph_loop", make, x, ref, base, ref32, **kw))
            entry = registry.describe(model, B, cfg["depth"])
            row["cells"].append(run_cell(entry["kernel"], lambda: build_run(entry, x, weights), x, ref, base, ref32, **kw))
            row["cells"][-1]["config"] = entry["config"]
            results[model][B] = row
            del x, ref, ref32
        del swiglu, net, net32, weights, compiled
        free_all()
    return results


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--models", nargs="+", default=list(registry.REGISTRY))
    ap.add_argument("--batch-sizes", nargs="+", type=int, default=DEFAULT_B)
    ap.add_argument("--passes", type=int, default=N_PASSES)
    ap.add_argument("--iters", type=int, default=N_ITERS)
    ap.add_argument("--warmup", type=int, default=N_WARMUP)
    ap.add_argument("--baselines", nargs="*", default=["swiglu"], choices=["swiglu", "compile", "orchestrated"])
    ap.add_argument("--out", default="cells.json")
    args = ap.parse_args(argv)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    print(f"GPU: {torch.cuda.get_device_name(0)}")
    res = sweep(args.models, args.batch_sizes, args.passes, args.iters, args.warmup, tuple(args.baselines))
    for model, rows in res.items():
        print(f"\n########## {model} ##########")
        for B, row in rows.items():
            if "cells" not in row:
                print(f"  B={B:>6}: {row.get('status')}")
                continue
            line = f"  B={B:>6}:"
            if row.get("SwiGLU"):
                line += f" SwiGLU {row['SwiGLU']['mean_us']:>9.1f}±{row['SwiGLU']['std_us']:.1f}us"
            for c in row["cells"]:
                line += (f" | {c['kernel']} {c['mean_us']:>9.1f}±{c['std_us']:.1f}us" if c["status"] == "ok"
                         else f" | {c['kernel']} [{c['status']}]")
            print(line)
    with open(args.out, "w") as f:
        json.dump(res, f, indent=2)
    print(f"\nSaved -> {args.out}")


if __name__ == "__main__":
    main()
