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


def locked_decoder_loop(dev, batch=8, prompt=512, steps=256, eager_steps=2):
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
    run(2)                                    # warm-up: weights folded, workspaces allocated
    pre_ms, step_ms = run(32)
    try:
        graph_ms = run_graph(steps)
        graph_note = "one decode step captured in a CUDA graph on a static KV cache"
    except Exception as e:                    # host framework without a capturable static cache
        graph_ms, graph_note = None, f"not captured: {type(e).__name__}"
    D.ops.check_status()
    D.set_fast_path(model, False)
    run(1)
    pre_eager, step_eager = run(eager_steps)
    del model
    torch.cuda.empty_cache()
    best = graph_ms if graph_ms is not None else step_ms
    return {"config": f"qwen3-shaped random init, 28 layers, d=1024, r=32, L=141, batch {batch}, prompt {prompt}, {steps} greedy steps",
            "prefill_ms": pre_ms, "prefill_tokens_per_s": batch * prompt / (pre_ms * 1e-3),
            "decode_ms_per_step": best, "decode_tokens_per_s": batch / (best * 1e-3),
            "decode_mode": graph_note, "decode_ms_per_step_plain_loop": step_ms,
            "torch_loop": {"prefill_ms": pre_eager, "decode_ms_per_step": step_eager, "steps_timed": eager_steps},
            "timing": "host clock around synchronised regions (the loop includes the host framework's attention and sampling)"}


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


def main():
    quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=8192, help="token rows per GPU per step")
    ap.add_argument("--no-extras", action="store_true", help="skip decode sweep, e2e and CPU baseline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    d, d_ff, r, L, seed = WORKLOADS[args.workload]

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
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / args.steps
    value = world * M * 1e3 / ms_step

    flops = 4.0 * L * M * d * r
    launches_per_step = plan.passes if plan.path == 1 else 1   # the striped path launches once per 64 rows
    kernel_ms = ms_step / launches_per_step
    timed_s = ms / 1e3
    peak_tf = peaks["tf_sustained"] if timed_s > 1.0 else peaks["tf_burst"]
    achieved_tf = flops / launches_per_step / (kernel_ms * 1e-3) / 1e12
    # DRAM traffic per launch: one ncu capture of a one-wave launch (profiles/) showed traffic equal to the
    # algorithmic bytes; weights exceed L2, so a launch of several waves re-reads them once per wave.
    tiles = (M + 127) // 128
    waves = plan.passes          # cluster / streamed paths: waves of row tiles inside the one launch
    traffic = waves * 4.0 * L * d * r + 4.0 * M * d
    roofline = {"bound": "tensor", "achieved": achieved_tf, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": achieved_tf / peak_tf, "traffic": traffic,
                "traffic_note": "bytes per launch, scaled by waves from a one-wave ncu capture",
                "peak_source": f"{peaks['source']} ({'sustained' if timed_s > 1.0 else 'burst'})",
                "kernel": {1: "striped", 2: "cluster", 3: "cluster_small", 4: "streamed"}.get(plan.path, "?"), "kernel_ms": kernel_ms,
                "frac_of_nominal_2250": achieved_tf / 2250.0}

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
        if world > 1:
            t = torch.tensor([ms_h, ms_serial], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_h, ms_serial = float(t[0].item()), float(t[1].item())
        line["e2e"] = {"value": world * M * args.steps * 1e3 / ms_h, "unit": "tokens/s",
                       "h2d_bytes_per_step": M * d * 2, "d2h_bytes_per_step": M * d * 2,
                       "ms_per_step": ms_h / args.steps,
                       "mode": "dlrb200_forward_host from pinned host buffers, steps alternating between two streams",
                       "one_stream": {"value": world * M * args.steps * 1e3 / ms_serial, "ms_per_step": ms_serial / args.steps}}
        ops.check_status()

    # ---- small-batch latencies and other prefill sizes (rank 0, N=1 only)
    if not args.no_extras and world == 1:
        wbytes = 4.0 * L * d * r
        dec = []
        for m in (1, 4, 16, 64):
            xm, ym = xs[0][:m].contiguous(), torch.empty(m, d, device=dev, dtype=torch.bfloat16)
            lo, med = min_latency_us(lambda: ops.forward_folded(xm, Vp, Up, out=ym))
            gbs = (wbytes + 4.0 * m * d) / (lo * 1e-6) / 1e9
            dec.append({"M": m, "min_us": lo, "median_us": med, "us_per_layer": lo / L, "algorithmic_GBps": gbs,
                        "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "tokens_per_s": m / (lo * 1e-6)})
        line["decode"] = dec
        pre = []
        for m in (1024, 4096):
            if m >= M:
                continue
            xm, ym = xs[0][:m].contiguous(), torch.empty(m, d, device=dev, dtype=torch.bfloat16)
            lo, med = min_latency_us(lambda: ops.forward_folded(xm, Vp, Up, out=ym), iters=10, warmup=3)
            pre.append({"M": m, "min_us": lo, "tokens_per_s": m / (lo * 1e-6),
                        "TFLOPs": 4.0 * L * m * d * r / (lo * 1e-6) / 1e12})
        line["prefill_other"] = pre
        ops.check_status()
        line["same_box_torch_loop"] = torch_loop_same_box(xs[0], Vp, Up)
        if args.workload == "cfg3":
            line["locked_decoder"] = locked_decoder_loop(dev)
        line["cpu_baseline"] = cpu_baseline(d, r, L, seed)

    if rank == 0:
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
