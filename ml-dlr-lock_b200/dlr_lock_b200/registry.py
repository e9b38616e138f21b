"""(model, batch size) -> implementation table, in the format of the reference's
``kernels/registry.py:17-135``: a list of entries per model with ``B_lo``,
``B_hi``, ``kernel``, ``callable`` (importable dotted path), ``config`` and
``note``.  This build has one backend behind one callable; it covers every batch
size of all four model shapes.  The library picks among its device paths per
call (``dlrb200_query`` reports the choice for a shape on the current device);
the ranges below name the path that serves most of each range on a B200, and
``describe`` fills an entry from the library's own answer.
"""

MODEL_CONFIGS = {  # kernels/reference.py:18-23
    "Qwen3-0.6B": {"d": 1024, "d_ff": 3072, "r": 32},
    "Qwen3-1.7B": {"d": 2048, "d_ff": 6144, "r": 64},
    "Qwen3-8B": {"d": 4096, "d_ff": 12288, "r": 128},
    "Qwen3-32B": {"d": 5120, "d_ff": 25600, "r": 256},
}

_CALLABLE = "dlr_lock_b200.ops.forward_xvu"

PATH_NAMES = {1: "b200_striped", 2: "b200_cluster", 3: "b200_cluster_small", 4: "b200_streamed",
              5: "b200_streamed_pairs", 6: "b200_striped_clusters"}
PATH_CONFIGS = {
    1: "width-striped cooperative grid, TMA weight ring, one exchange per layer through L2",
    2: "128-row tiles on clusters of d/512 CTAs, activations resident in tensor memory, tcgen05",
    3: "one cluster of d/256 CTAs per two rows, exchange in distributed shared memory",
    4: "128-row tiles, one cluster of 1/2/4 CTAs each, activations streamed through shared and tensor memory, tcgen05",
    5: "256-row tiles on CTA pairs (tcgen05 cta_group::2), activations streamed, exchange in distributed shared memory",
    6: "width-striped cooperative grid in clusters of 8: reduction inside a cluster in distributed shared memory, "
       "cluster sums through counted words in L2",
}


def _entry(lo, hi, path, note):
    return {"B_lo": lo, "B_hi": hi, "kernel": PATH_NAMES[path], "callable": _CALLABLE,
            "config": PATH_CONFIGS[path] + "; picked per call by dlrb200_query", "note": note}


def _entries(name):
    d, r = MODEL_CONFIGS[name]["d"], MODEL_CONFIGS[name]["r"]
    small = 3 if d <= 1024 else 1
    big = 2 if r < 64 or d <= 2048 else 4
    rows = [_entry(1, 64, small, "Small batch: one launch walks all layers, one exchange per layer.")]
    if d >= 2048:
        split = 17 if d >= 4096 else 29          # from where the two-level exchange is the faster one
        rows = [_entry(1, split - 1, small, "Small batch: one launch walks all layers, one exchange per layer."),
                _entry(split, 64, 6, "Small batch, more rows: the exchange in two levels.")]
    big_pairs = 5 if r in (64, 128) else big
    return rows + [
        _entry(65, 4095, big, "Large batch: row tiles on tensor cores, one launch for all layers."),
        _entry(4096, 131072, big_pairs, "Largest batches: 256-row tiles on CTA pairs where the shape allows."),
    ]


REGISTRY = {name: _entries(name) for name in MODEL_CONFIGS}


def resolve(model: str, batch_size: int):
    """Entry serving ``(model, batch_size)``, or None (kernels/registry.py:130-135)."""
    for entry in REGISTRY.get(model, []):
        if entry["B_lo"] <= batch_size <= entry["B_hi"]:
            return entry
    return None


def describe(model: str, batch_size: int, depth: int):
    """``resolve`` with ``kernel`` and ``config`` filled from what the library would run for this exact
    cell on the current CUDA device (needs the built library and a GPU)."""
    from . import ops
    entry = resolve(model, batch_size)
    if entry is None:
        return None
    cfg = MODEL_CONFIGS[model]
    plan = ops.query(batch_size, cfg["d"], cfg["r"], depth)
    out = dict(entry)
    out["kernel"] = PATH_NAMES.get(plan.path, f"path{plan.path}")
    out["config"] = (f"{PATH_CONFIGS.get(plan.path, '')}; grid {plan.grid}, cluster {plan.cluster}, "
                     f"{plan.passes} pass(es), {plan.smem_bytes} B shared memory")
    return out
