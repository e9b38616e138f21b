"""(model, batch size) -> implementation table, in the format of the reference's
``kernels/registry.py:17-135``: a list of entries per model with ``B_lo``,
``B_hi``, ``kernel``, ``callable`` (importable dotted path), ``config`` and
``note``.  This build has one backend; it covers every batch size of all four
model shapes, split only by which of its two device paths serves the range.
"""

MODEL_CONFIGS = {  # kernels/reference.py:18-23
    "Qwen3-0.6B": {"d": 1024, "d_ff": 3072, "r": 32},
    "Qwen3-1.7B": {"d": 2048, "d_ff": 6144, "r": 64},
    "Qwen3-8B": {"d": 4096, "d_ff": 12288, "r": 128},
    "Qwen3-32B": {"d": 5120, "d_ff": 25600, "r": 256},
}

_CALLABLE = "dlr_lock_b200.ops.forward_xvu"


def _entries():
    return [
        {
            "B_lo": 1, "B_hi": 64,
            "kernel": "b200_striped",
            "callable": _CALLABLE,
            "config": "width-striped cooperative grid, TMA weight ring, mma.sync; picked by dlrb200_query",
            "note": "Small batch: one launch walks all layers, one exchange per layer.",
        },
        {
            "B_lo": 65, "B_hi": 131072,
            "kernel": "b200_cluster",
            "callable": _CALLABLE,
            "config": "128-row tiles on CTA clusters, tcgen05 + tensor memory; picked by dlrb200_query",
            "note": "Large batch: activations stay on chip for all layers.",
        },
    ]


REGISTRY = {name: _entries() for name in MODEL_CONFIGS}


def resolve(model: str, batch_size: int):
    """Entry serving ``(model, batch_size)``, or None (kernels/registry.py:130-135)."""
    for entry in REGISTRY.get(model, []):
        if entry["B_lo"] <= batch_size <= entry["B_hi"]:
            return entry
    return None
