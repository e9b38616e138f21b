"""Benchmark of the DLR-Net forward on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward of the whole L-layer stack over one batch of M
synthetic token rows.  The default workload is the shape the headline metric
is quoted on: d=4096, r=128, L=143 (kernels/reference.py:18-23, "Qwen3-8B"),
M=8192 rows per GPU, bf16, seeded N(0,1) inputs and the reference's
initialisation scales with alpha=0.01 (kernels/reference.py:46-55).  With N
GPUs every rank runs the same number of rows on its own replica of the weights
(rows are independent, so there is no collective in the timed region) and the
reported value is the total rows per second, timed on the device and taken as
the maximum over ranks.

The single JSON line also carries: the tensor-core roofline of the large-batch
kernel, the same forward measured through the host-buffer C-ABI entry point
(``e2e``), the small-batch (decode) latencies with their weight-streaming
bandwidth, the clocks sampled during the run, and a CPU baseline (the oracle's
restatement of the reference's torch loop, timed on this machine's cores).

``--impl reference`` times that CPU restatement alone, on bounded samples of the
same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [ROOT, os.path.join(ROOT, "ml-dlr-lock_b200")]

import torch  # noqa: E402

METRIC = "DLR-Net fwd tokens/s at d=4096 r=128 L=143 (M=1..8192); % HBM/TC roofline"
WORKLOADS = {
    # name: d, d_ff, r, L, seed  (BASELINE configs 1-4)
    "cfg1": (1024, 3072, 32, 141, 0),
    "cfg2": (2048, 6144, 64, 142, 1),
    "cfg3": (4096, 12288, 128, 143, 2),
    "cfg4": (5120, 25600, 256, 149, 3),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tf_burst=p["bf16_tflops"], tf_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tf_burst=1590.0, tf_sustained=1400.0, source="fallback")


# --------------------------------------------------------------------------- #
# clocks
# --------------------------------------------------------------------------- #
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the bench runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake"}

    def __init__(self, device: int):
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._mark = None
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self._nv = pynvml
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # pragma: no cover - depends on the box
            self._nv = None
            self.error = repr(e)

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                self.samples.append((time.perf_counter(), mhz, mask))
            except Exception:
                pass
            time.sleep(0.02)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def mark(self):
        self._mark = time.perf_counter()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        end = time.perf_counter()
        inside = [s for s in self.samples if self._mark is not None and self._mark <= s[0] <= end]
        use = inside or self.samples
        reasons = set()
        for _, _, mask in use:
            for bit, name in self.REASONS.items():
                if mask & bit:
                    reasons.add(name)
        return {"sm_mhz": statistics.median([s[1] for s in use]) if use else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons), "samples": len(use)}


# --------------------------------------------------------------------------- #
# synthetic problem
# --------------------------------------------------------------------------- #
def make_weights(d, r, L, seed, device, alpha=0.01):
    """Folded bf16 weights with the reference's initialisation scales
    (dlr_lock/model.py:65-68): V ~ N(0, 1/d), U ~ N(0, 1/(rL)), gain 1."""
    from dlr_lock_b200 import ops
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    V = torch.randn(L, r, d, device=device, generator=g) * (1.0 / math.sqrt(d))
    U = torch.randn(L, d, r, device=device, generator=g) * (1.0 / math.sqrt(r * L))
    gain = torch.ones(L, d, device=device)
    a = torch.full((L,), alpha, device=device)
    Vp, Up = ops.fold_weights(V, U, gain, a)
    del V, U
    return Vp, Up


def time_steps(fn, steps, warmup, dist_barrier=None):
    """Device time of `steps` calls after `warmup`, ms total."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_barrier:
        dist_barrier()
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    if dist_barrier:
        dist_barrier()
    return a.elapsed_time(b)


def min_latency_us(fn, iters=200, warmup=20):
    """Minimum single-call device time (kernels/bench/_protocol.py:83-105 form)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    best = float("inf")
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = [a.elapsed_time(b) * 1e3 for a, b in evs]
    return min(ts), statistics.median(ts)


# --------------------------------------------------------------------------- #
# CPU baseline (oracle port of the reference's torch loop)
# --------------------------------------------------------------------------- #
def cpu_forward_sampler(d, r, L, seed, rows):
    from oracle import dlrnet_oracle as O
    # torchrun pins OMP_NUM_THREADS to 1 for every rank; the CPU arm runs on one rank only and may use the host
    n = os.cpu_count() or 1
    if torch.get_num_threads() < n:
        torch.set_num_threads(min(n, 64))
    p, x = O.seeded_case(d, r, L, rows, seed, alpha=0.01)
    return lambda: O.forward_eager(x, p)


def torch_loop_same_box(x, Vp, Up, eps=1e-6):
    """The layer loop in eager torch ops on the same GPU, on the folded weights (the arithmetic of
    dlr_lock/model.py:96-100 with the gain and alpha pre-multiplied: about six launches per layer).  A
    comparison figure only: nothing of the product path runs here."""
    import torch.nn.functional as F

    def fwd():
        h = x
        for l in range(Vp.shape[0]):
            rstd = torch.rsqrt(h.float().pow(2).mean(dim=-1, keepdim=True) + eps).to(h.dtype)
            h = h + F.silu((h * rstd) @ Vp[l].T) @ Up[l].T
        return h

    with torch.no_grad():
        fwd()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            fwd()
        b.record()
        torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 3
    return {"ms_per_step": ms, "tokens_per_s": x.shape[0] / (ms * 1e-3), "what": "eager torch bf16 layer loop on folded weights, same GPU, same input"}


def locked_decoder_loop(dev, batch=8, prompt=512, steps=256, eager_steps=2, fused=True):
    """The locked decoder loop on synthetic shapes: a randomly initialised Qwen3-shaped decoder (28 layers,
    hidden 1024, 16 query / 8 key-value heads of 128, d_ff 3072, vocabulary 151936) whose MLPs are DLR-Nets of
    rank 32 (depth 141), batch 8, 512 uniform-random prompt ids, 256 greedy steps on the KV cache.  Timed with
    the CUDA library under the nets, and for a few steps with the torch layer loop under them (the
    reference's own arithmetic: about 31000 kernel launches per token)."""
    import time

    from transformers import AutoConfig

    import dlr_lock_b200 as D
    torch.manual_seed(5)
    cfg = AutoConfig.for_model("qwen3", vocab_size=151936, hidden_size=1024, intermediate_size=3072,
                               num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128,
                               max_position_embeddings=2048, tie_word_embeddings=True)
    model = D.locked_model_from_config(cfg, rank=32, device=dev, alpha_init=0.01).eval()
    ids = torch.randint(0, 151936, (batch, prompt), device=dev)

    def run(n_steps):
        # plain loop: the host framework's eager decode on a growing cache (host-bound: about 2 ms of
        # Python per decoder layer)
        with torch.no_grad():
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = model(ids, use_cache=True)
            tok = out.logits[:, -1:].argmax(-1)
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            past = out.past_key_values
            for _ in range(n_steps):
                out = model(tok, past_key_values=past, use_cache=True)
                past = out.past_key_values
                tok = out.logits[:, -1:].argmax(-1)
            torch.cuda.synchronize()
            t2 = time.perf_counter()
        return (t1 - t0) * 1e3, (t2 - t1) * 1e3 / max(1, n_steps)

    def run_graph(n_steps):
        # one decode step captured in a CUDA graph on a static KV cache, replayed n_steps times
        from transformers import StaticCache
        with torch.no_grad():
            cache = StaticCache(config=model.config, max_cache_len=prompt + n_steps + 8)
            out = model(ids, past_key_values=cache, use_cache=True, cache_position=torch.arange(prompt, device=dev))
            tok = out.logits[:, -1:].argmax(-1).clone()
            pos = torch.tensor([prompt], device=dev)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    model(tok, past_key_values=cache, use_cache=True, cache_position=pos)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                out = model(tok, past_key_values=cache, use_cache=True, cache_position=pos)
                nxt = out.logits[:, -1:].argmax(-1)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(n_steps):
                graph.replay()
                tok.copy_(nxt)
                pos.add_(1)
            torch.cuda.synchronize()
            return (time.perf_counter() - t0) * 1e3 / n_steps

    D.set_fast_path(model, True)
    if fused:
        D.fuse_decoder_layers(model)          # the net's output is the layer's output: no "- h" / "+ h" passes
    run(2)                                    # warm-up: weights folded, workspaces allocated
    pre_ms, step_ms = run(32)
    try:
        graph_ms = run_graph(steps)
        graph_note = "one decode step captured in a CUDA graph on a static KV cache"
    except Exception as e:                    # host framework without a capturable static cache
        graph_ms, graph_note = None, f"not captured: {type(e).__name__}"
    D.ops.check_status()
    torch_loop = None
    if eager_steps > 0:
        D.set_fast_path(model, False)
        if fused:
            D.fuse_decoder_layers(model, False)
        run(1)
        pre_eager, step_eager = run(eager_steps)
        torch_loop = {"prefill_ms": pre_eager, "decode_ms_per_step": step_eager, "steps_timed": eager_steps}
    del model
    torch.cuda.empty_cache()
    best = graph_ms if graph_ms is not None else step_ms
    return {"batch": batch, "fused_residual": bool(fused), "config": f"qwen3-shaped random init, 28 layers, d=1024, r=32, L=141, batch {batch}, prompt {prompt}, {steps} greedy steps",
            "prefill_ms": pre_ms, "prefill_tokens_per_s": batch * prompt / (pre_ms * 1e-3),
            "decode_ms_per_step": best, "decode_tokens_per_s": batch / (best * 1e-3),
            "decode_mode": graph_note, "decode_ms_per_step_plain_loop": step_ms,
            "torch_loop": torch_loop,
            "timing": "host clock around synchronised regions (the loop includes the host framework's attention and sampling)"}


def cpu_baseline_cfg1(rows=2048, budget_s=8.0):
    """The stated CPU baseline configuration: d=1024, r=32, L=141, M=2048 rows, seed 0, the reference's
    torch loop (oracle port) in fp32 and in bf16 on this machine's cores, best of up to 5 after one warm-up."""
    from oracle import dlrnet_oracle as O
    n = os.cpu_count() or 1
    if torch.get_num_threads() < n:
        torch.set_num_threads(min(n, 64))
    d, _, r, L, seed = WORKLOADS["cfg1"]
    p, x = O.seeded_case(d, r, L, rows, seed, alpha=0.01)
    out = {"config": f"cfg1: d={d} r={r} L={L}, M={rows} rows, seed {seed}", "cores": torch.get_num_threads(),
           "nproc": n, "kind": "port"}
    for name, fn in (("fp32", lambda: O.forward_fp32(x, p)), ("bf16", lambda: O.forward_eager(x, p))):
        fn()
        best, spent, reps = float("inf"), 0.0, 0
        while spent < budget_s / 2 and reps < 5:
            t0 = time.perf_counter()
            fn()
            dt = time.perf_counter() - t0
            best, spent, reps = min(best, dt), spent + dt, reps + 1
        out[name] = {"seconds": best, "tokens_per_s": rows / best, "best_of": reps}
    return out


def cpu_baseline(d, r, L, seed, rows=512, budget_s=12.0):
    fn = cpu_forward_sampler(d, r, L, seed, rows)
    fn()
    best, spent, reps = float("inf"), 0.0, 0
    while spent < budget_s and reps < 8:
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        best = min(best, dt)
        spent += dt
        reps += 1
    return {"value": rows / best, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{rows} rows of the same d/r/L, bf16 torch CPU loop (oracle.forward_eager), best of {reps}"}


def run_reference_arm(args, d, r, L, seed):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 256
    fn = cpu_forward_sampler(d, r, L, seed, rows)
    for _ in range(min(args.warmup, 2)):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = time.perf_counter() - t0
    v = rows * args.steps / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 2), "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: d={d} r={r} L={L}, {rows}-row sample per step on host cores"},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{rows} rows per step, bf16 torch CPU loop (oracle.forward_eager)"},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# --------------------------------------------------------------------------- #
_REAL_STDOUT = None


def quiet_stdout():
    """Send everything libraries print on stdout (NCCL's version banner, the host framework's notices) to
    stderr: stdout carries the one JSON line and nothing else."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    sys.stdout.flush()
    if _REAL_STDOUT is not None:
        os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())
    else:
        print(json.dumps(line), flush=True)


def _max_over_ranks(vals, dev, world):
    if world == 1:
        return [float(v) for v in vals]
    import torch.distributed as dist
    t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def sharded_block(dev, world, rank, barrier, Vp, Up, d, r, L, steps):
    """ONE batch of M rows split over the ranks in contiguous row blocks (weights replicated, rows are
    independent: dlr_lock/model.py:93-101 has no cross-row op), forward per rank, one all-gather of the output
    blocks.  Reported per M: time of the single-GPU forward of the whole batch (every rank measures it on its own
    GPU: the N = 1 reference of the strong-scaling figure), time of the sharded forward alone and with the gather
    inside the timed region (device time, maximum over ranks), and that the gathered output equals the single-GPU
    output bit for bit."""
    from dlr_lock_b200 import ops, sharding
    fwd = sharding.RowShardedForward(lambda x: ops.forward_folded(x, Vp, Up), tile=128)
    out = []
    for M in (8192, 4096, 1024):
        g = torch.Generator(device=dev)
        g.manual_seed(4242 + M)                         # same batch on every rank
        x = torch.randn(M, d, device=dev, generator=g).to(torch.bfloat16)
        y_full = ops.forward_folded(x, Vp, Up)
        a, b = fwd.local_rows(M)
        xl = x[a:b].contiguous()
        y_all = fwd.gather(ops.forward_folded(xl, Vp, Up), M) if b > a or world > 1 else y_full
        torch.cuda.synchronize()
        same = bool(torch.equal(y_all, y_full))
        n = max(3, min(steps, 10))
        t_full = time_steps(lambda: ops.forward_folded(x, Vp, Up), n, 3, barrier) / n
        t_local = time_steps(lambda: ops.forward_folded(xl, Vp, Up), n, 3, barrier) / n
        t_gather = time_steps(lambda: fwd.gather(ops.forward_folded(xl, Vp, Up), M), n, 3, barrier) / n
        t_full, t_local, t_gather = _max_over_ranks([t_full, t_local, t_gather], dev, world)
        plan = ops.query(max(b - a, 1), d, r, L)
        out.append({"M": M, "rows_per_gpu": b - a, "ms_single_gpu_whole_batch": t_full, "ms_sharded_forward": t_local,
                    "ms_sharded_forward_and_gather": t_gather, "tokens_per_s_no_gather": M / (t_local * 1e-3),
                    "tokens_per_s_with_gather": M / (t_gather * 1e-3),
                    "strong_scaling_efficiency_no_gather": t_full / (world * t_local),
                    "strong_scaling_efficiency_with_gather": t_full / (world * t_gather),
                    "gathered_equals_single_gpu_bits": same,
                    "per_gpu_plan": {"path": plan.path, "grid": plan.grid, "cluster": plan.cluster, "passes": plan.passes}})
        del x, y_full, y_all, xl
    ops.check_status()
    return {"what": "one batch split in contiguous row blocks, final all_gather_into_tensor (NCCL)", "n_gpus": world, "cases": out,
            "limit": "at 1024 rows per GPU the cluster kernel runs one wave of row tiles on part of the SMs: the per-GPU time "
                     "stops falling with the row count, which bounds strong scaling; the gather itself is NVLink-bound"}


def decode_sweep(dev, name, Ms, peaks):
    from dlr_lock_b200 import ops
    d, _, r, L, seed = WORKLOADS[name]
    Vp, Up = make_weights(d, r, L, seed, dev)
    g = torch.Generator(device=dev)
    g.manual_seed(77 + seed)
    x = torch.randn(max(Ms), d, device=dev, generator=g).to(torch.bfloat16)
    wbytes = 4.0 * L * d * r
    rows = []
    for m in Ms:
        xm, ym = x[:m].contiguous(), torch.empty(m, d, device=dev, dtype=torch.bfloat16)
        plan = ops.query(m, d, r, L)
        if m <= 64:
            lo, med = min_latency_us(lambda: ops.forward_folded(xm, Vp, Up, out=ym))
            gbs = (wbytes + 4.0 * m * d) / (lo * 1e-6) / 1e9
            rows.append({"M": m, "path": plan.path, "min_us": lo, "median_us": med, "us_per_layer": lo / L,
                         "algorithmic_GBps": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "tokens_per_s": m / (lo * 1e-6)})
        else:
            lo, med = min_latency_us(lambda: ops.forward_folded(xm, Vp, Up, out=ym), iters=10, warmup=3)
            tf = 4.0 * L * m * d * r / (lo * 1e-6) / 1e12
            rows.append({"M": m, "path": plan.path, "cluster": plan.cluster, "grid": plan.grid, "min_us": lo,
                         "tokens_per_s": m / (lo * 1e-6), "TFLOPs": tf, "frac_of_measured_bf16_burst": tf / peaks["tf_burst"]})
    ops.check_status()
    del Vp, Up, x
    torch.cuda.empty_cache()
    return {"config": f"{name}: d={d} r={r} L={L}", "weights_MB": wbytes / 1e6, "cases": rows}


def same_box_comparisons(dev, x, Vp, Up, d, r, L, seed, workload, rows):
    """Library-only ways of running the same stack on this GPU (comparison figures; nothing of the product path):
    the eager torch loop, the cuBLAS + elementwise loop captured in one CUDA graph (the form of
    kernels/kernels/orchestrated.py:95-126) and the torch module under torch.compile(mode="reduce-overhead")
    (kernels/bench/bench_paper.py:178), the last in a child process with a time limit."""
    import subprocess
    from dlr_lock_b200 import harness
    out = {"eager_torch_loop": torch_loop_same_box(x, Vp, Up)}
    try:
        weights = {"Vs": Vp.transpose(1, 2).contiguous(), "Us": Up.transpose(1, 2).contiguous(), "L": L, "D": d, "R": r,
                   "premultiplied": True}
        graph, hbuf = harness.orchestrated_graph(x, weights)
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 3
        out["cublas_graph_loop"] = {"ms_per_step": ms, "tokens_per_s": x.shape[0] / (ms * 1e-3),
                                    "what": "per layer cuBLAS GEMM, elementwise rstd*SiLU, cuBLAS addmm_; one CUDA graph"}
        del graph, hbuf, weights
    except Exception as e:  # noqa: BLE001
        out["cublas_graph_loop"] = {"status": f"{type(e).__name__}: {e}"[:200]}
    torch.cuda.empty_cache()
    try:
        cmd = [sys.executable, os.path.abspath(__file__), "--compare-child", "compile", "--workload", workload, "--rows", str(rows)]
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
        line = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
        out["torch_compile_reduce_overhead"] = json.loads(line[-1]) if line else {"status": "no output", "stderr": res.stderr[-300:]}
    except subprocess.TimeoutExpired:
        out["torch_compile_reduce_overhead"] = {"status": "not finished within 240 s (compilation of the unrolled stack)"}
    except Exception as e:  # noqa: BLE001
        out["torch_compile_reduce_overhead"] = {"status": f"{type(e).__name__}: {e}"[:200]}
    out["triton_fused"] = {"status": "not run: the reference's Triton source is not on this machine and is not reproduced here"}
    return out


def compare_child(args):
    """Child process of same_box_comparisons: the torch module of the workload under
    torch.compile(mode="reduce-overhead")."""
    import dlr_lock_b200 as D
    from dlr_lock_b200 import harness
    d, _, r, L, seed = WORKLOADS[args.workload]
    dev = torch.device("cuda", 0)
    torch.manual_seed(seed)
    net = D.DLRNet(d, r, L, alpha_init=0.01).to(torch.bfloat16).to(dev).eval()
    for p in net.parameters():
        p.requires_grad_(False)
    x = torch.randn(args.rows, d, device=dev).to(torch.bfloat16)
    t0 = time.perf_counter()
    fn = harness.compiled_reduce_overhead(net)
    with torch.no_grad():
        for _ in range(3):
            y = fn(x)
        torch.cuda.synchronize()
        compile_s = time.perf_counter() - t0
        net.fast = False
        err = harness.rel_err(y, net(x))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            fn(x)
        b.record()
        torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 3
    print(json.dumps({"ms_per_step": ms, "tokens_per_s": args.rows / (ms * 1e-3), "compile_s": compile_s,
                      "rel_err_vs_eager": err, "what": "torch.compile(mode='reduce-overhead') of the eager module"}), flush=True)


def main():
    quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=8192, help="token rows per GPU per step")
    ap.add_argument("--no-extras", action="store_true", help="headline only: skip e2e, sharding, decode sweeps, comparisons, CPU baseline")
    ap.add_argument("--compare-child", default=None, help=argparse.SUPPRESS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    d, d_ff, r, L, seed = WORKLOADS[args.workload]

    if args.compare_child:
        global _REAL_STDOUT
        os.dup2(_REAL_STDOUT, 1)
        _REAL_STDOUT = None
        compare_child(args)
        return
    if args.impl == "reference":
        run_reference_arm(args, d, r, L, seed)
        return

    from dlr_lock_b200 import ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    barrier = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        barrier = dist.barrier
    ops._lib.load()
    peaks = measured_peaks()

    M = args.rows
    Vp, Up = make_weights(d, r, L, seed, dev)
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + seed + rank)
    xs = [torch.randn(M, d, device=dev, generator=g).to(torch.bfloat16) for _ in range(2)]
    ys = [torch.empty_like(x) for x in xs]
    plan = ops.query(M, d, r, L)
    it = [0]

    def step():
        i = it[0] & 1
        it[0] += 1
        ops.forward_folded(xs[i], Vp, Up, out=ys[i])

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    ops.check_status()
    sampler.mark()
    ms = time_steps(step, args.steps, args.warmup, barrier)
    clocks = sampler.stop()
    ops.check_status()
    (ms,) = _max_over_ranks([ms], dev, world)
    ms_step = ms / args.steps
    value = world * M * 1e3 / ms_step

    path_name = {1: "striped", 2: "cluster", 3: "cluster_small", 4: "streamed", 5: "streamed_pairs", 6: "striped_clusters"}.get(plan.path, "?")
    launches_per_step = plan.passes if plan.path == 1 else 1   # the striped path launches once per 64 rows
    kernel_ms = ms_step / launches_per_step
    timed_s = ms / 1e3
    if plan.path in (1, 3, 6):
        # small-batch kernels stream the weights once per launch: HBM-bound by design
        bytes_alg = 4.0 * L * d * r + 4.0 * min(M, 64) * d
        achieved = bytes_alg / (kernel_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": bytes_alg,
                    "traffic_note": "ncu capture of the striped kernel (profiles/): DRAM bytes equal the algorithmic bytes",
                    "peak_source": f"{peaks['source']} (copy bandwidth)", "kernel": path_name, "kernel_ms": kernel_ms}
    else:
        flops = 4.0 * L * M * d * r
        peak_tf = peaks["tf_sustained"] if timed_s > 1.0 else peaks["tf_burst"]
        achieved_tf = flops / launches_per_step / (kernel_ms * 1e-3) / 1e12
        alg_bytes = 4.0 * L * d * r + 4.0 * M * d
        if args.workload == "cfg3" and M == 8192 and plan.path == 5:
            # one ncu capture of this very launch (profiles/streamed_pairs_kernel_cfg3_M8192.md)
            traffic, note = 0.707e9 + 0.924e9, ("measured: dram__bytes_read + dram__bytes_write of one captured launch of this "
                                                "configuration (a second capture: 1.06 + 1.57 GB); the activations (134 MB through "
                                                "L2 per layer) do not stay in L2 entirely")
        else:
            traffic, note = plan.passes * 4.0 * L * d * r + 4.0 * M * d, "not captured at this size: waves x weights + activations"
        roofline = {"bound": "tensor", "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s",
                    "frac": achieved_tf / peak_tf, "traffic": traffic, "traffic_note": note, "algorithmic_bytes": alg_bytes,
                    "peak_source": f"{peaks['source']} ({'sustained' if timed_s > 1.0 else 'burst'})",
                    "kernel": path_name, "kernel_ms": kernel_ms, "frac_of_nominal_2250": achieved_tf / 2250.0}

    line = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: DLR-Net forward d={d} r={r} L={L}, M={M} rows per GPU, alpha=0.01",
                   "rows_per_gpu": M, "l2": "inputs exceed L2 (weights %.0f MB + two alternating %d MB batches)"
                   % (4.0 * L * d * r / 1e6, M * d * 2 // 1000000),
                   "parallelism": f"rows x{world}, weights replicated"},
        "roofline": roofline, "clocks": clocks, "gpu_launches": launches_per_step * args.steps,
        "plan": {"path": plan.path, "grid": plan.grid, "cluster": plan.cluster, "stripe_cols": plan.stripe_cols,
                 "passes": plan.passes},
    }

    # ---- the same step for at least two seconds: what the kernel sustains under the power cap
    if not args.no_extras and plan.path not in (1, 3, 6):
        n_long = int(math.ceil(2200.0 / ms_step))
        s2 = ClockSampler(local)
        s2.start()
        s2.mark()
        ms_long = time_steps(step, n_long, 3, barrier)
        clk = s2.stop()
        (ms_long,) = _max_over_ranks([ms_long], dev, world)
        tf = 4.0 * L * M * d * r / (ms_long / n_long * 1e-3) / 1e12
        line["sustained"] = {"steps": n_long, "seconds": ms_long / 1e3, "ms_per_step": ms_long / n_long,
                             "tokens_per_s": world * M * n_long * 1e3 / ms_long, "TFLOPs_per_gpu": tf,
                             "frac_of_measured_sustained_bf16": tf / peaks["tf_sustained"], "clocks": clk}
        ops.check_status()

    # ---- end to end through the host-buffer entry point (every rank, max over ranks)
    if not args.no_extras:
        xh = [x.cpu().pin_memory() for x in xs]
        yh = [torch.empty_like(x).pin_memory() for x in xh]
        jt = [0]

        def step_host():
            i = jt[0] & 1
            jt[0] += 1
            ops.forward_host(xh[i], yh[i], xs[i], ys[i], Vp, Up)

        # (1) one stream: H2D, kernel, D2H of a step strictly one after the other
        ms_serial = time_steps(step_host, args.steps, 3, barrier)
        # (2) two streams, steps alternate: each step is still H2D -> kernel -> D2H on its own stream and its own
        # buffers, but the copies of one step overlap the kernel of the other (what a serving loop does)
        side = [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)]

        def run_piped(n):
            for k in range(n):
                with torch.cuda.stream(side[k & 1]):
                    ops.forward_host(xh[k & 1], yh[k & 1], xs[k & 1], ys[k & 1], Vp, Up)

        for st in side:
            st.wait_stream(torch.cuda.current_stream())
        run_piped(4)
        torch.cuda.synchronize()
        if barrier:
            barrier()
        torch.cuda.synchronize()
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record()
        for st in side:
            st.wait_stream(torch.cuda.current_stream())
        run_piped(args.steps)
        for st in side:
            torch.cuda.current_stream().wait_stream(st)
        eb.record()
        torch.cuda.synchronize()
        if barrier:
            barrier()
        ms_h = ea.elapsed_time(eb)
        ms_h, ms_serial = _max_over_ranks([ms_h, ms_serial], dev, world)
        line["e2e"] = {"value": world * M * args.steps * 1e3 / ms_h, "unit": "tokens/s",
                       "h2d_bytes_per_step": M * d * 2, "d2h_bytes_per_step": M * d * 2,
                       "ms_per_step": ms_h / args.steps,
                       "mode": "dlrb200_forward_host from pinned host buffers, steps alternating between two streams",
                       "one_stream": {"value": world * M * args.steps * 1e3 / ms_serial, "ms_per_step": ms_serial / args.steps}}
        ops.check_status()
        del xh, yh

    # ---- one batch sharded by rows over the ranks, with the final gather (every N; at N = 1 it is the reference point)
    if not args.no_extras and args.workload == "cfg3":
        line["sharded"] = sharded_block(dev, world, rank, barrier, Vp, Up, d, r, L, args.steps)

    # ---- the locked decoder loop over N GPUs, batch-sharded: the sequences of a batch are independent, every rank
    # runs its own sequences on its own replica of the model and KV cache, no collective in the loop
    if not args.no_extras and args.workload == "cfg3":
        if world == 1:
            line["locked_decoder"] = locked_decoder_loop(dev)
        else:
            steps_n = 64
            strong_b = max(1, 8 // world)
            strong = locked_decoder_loop(dev, batch=strong_b, steps=steps_n, eager_steps=0) if world <= 8 else None
            weak = locked_decoder_loop(dev, batch=8, steps=steps_n, eager_steps=0)
            vals = _max_over_ranks([strong["decode_ms_per_step"], strong["prefill_ms"], weak["decode_ms_per_step"], weak["prefill_ms"]],
                                   dev, world)
            line["locked_decoder"] = {
                "config": strong["config"].split(", batch")[0] + f", prompt 512, {steps_n} greedy steps, {world} GPUs, batch-sharded",
                "strong": {"batch_total": strong_b * world, "batch_per_gpu": strong_b, "decode_ms_per_step": vals[0], "prefill_ms": vals[1],
                           "decode_tokens_per_s": strong_b * world / (vals[0] * 1e-3),
                           "prefill_tokens_per_s": strong_b * world * 512 / (vals[1] * 1e-3)},
                "weak": {"batch_total": 8 * world, "batch_per_gpu": 8, "decode_ms_per_step": vals[2], "prefill_ms": vals[3],
                         "decode_tokens_per_s": 8 * world / (vals[2] * 1e-3),
                         "prefill_tokens_per_s": 8 * world * 512 / (vals[3] * 1e-3)},
                "decode_mode": weak["decode_mode"], "fused_residual": weak["fused_residual"],
                "timing": "host clock around synchronised regions, maximum over ranks"}

    # ---- small-batch latencies, other sizes and shapes, comparisons, CPU baselines (rank 0, N=1 only)
    if not args.no_extras and world == 1:
        wbytes = 4.0 * L * d * r
        dec = []
        for m in (1, 4, 16, 64):
            xm, ym = xs[0][:m].contiguous(), torch.empty(m, d, device=dev, dtype=torch.bfloat16)
            lo, med = min_latency_us(lambda: ops.forward_folded(xm, Vp, Up, out=ym))
            gbs = (wbytes + 4.0 * m * d) / (lo * 1e-6) / 1e9
            dec.append({"M": m, "path": ops.query(m, d, r, L).path, "min_us": lo, "median_us": med, "us_per_layer": lo / L,
                        "algorithmic_GBps": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "tokens_per_s": m / (lo * 1e-6)})
        line["decode"] = dec
        pre = []
        for m in (1024, 2048, 3840, 4096, 16384):
            if m == M:
                continue
            if m < M:
                xm = xs[0][:m].contiguous()
            else:       # more rows than stay in L2 between two layers: walked in rounds
                xm = torch.cat([xs[0]] * ((m + M - 1) // M))[:m].contiguous()
            ym = torch.empty(m, d, device=dev, dtype=torch.bfloat16)
            lo, med = min_latency_us(lambda: ops.forward_folded(xm, Vp, Up, out=ym), iters=10, warmup=3)
            pl = ops.query(m, d, r, L)
            pre.append({"M": m, "path": pl.path, "grid": pl.grid, "cluster": pl.cluster, "rounds": pl.passes, "min_us": lo,
                        "tokens_per_s": m / (lo * 1e-6), "TFLOPs": 4.0 * L * m * d * r / (lo * 1e-6) / 1e12})
            del xm, ym
        line["prefill_other"] = pre
        ops.check_status()
        line["same_box"] = same_box_comparisons(dev, xs[0], Vp, Up, d, r, L, seed, args.workload, M)
        line["same_box_torch_loop"] = line["same_box"]["eager_torch_loop"]
        del xs, ys, Vp, Up
        torch.cuda.empty_cache()
        if args.workload == "cfg3":
            line["other_configs"] = {
                "cfg1": decode_sweep(dev, "cfg1", (1, 16, 64, 2048), peaks),
                "cfg2": decode_sweep(dev, "cfg2", (1, 4, 16, 64, 8192), peaks),
                "cfg4": decode_sweep(dev, "cfg4", (1, 64, 4096), peaks),
            }
            line["cpu_baseline_cfg1"] = cpu_baseline_cfg1()
        line["cpu_baseline"] = cpu_baseline(d, r, L, seed)

    if rank == 0:
        emit(line)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
