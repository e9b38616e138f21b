"""dlr_lock_b200: the DLR-Net forward pass on NVIDIA B200 (sm_100a).

Public names follow the reference package ``dlr_lock`` (dlr_lock/__init__.py:13-41)
so that a user of the reference can switch imports; the forward itself runs in
hand-written CUDA behind a C ABI (include/dlr_b200.h).
"""
from .model import (  # noqa: F401
    DLRNet,
    ResidualDLRNet,
    accelerate_locked_model,
    build_locked_model,
    compute_depth,
    dlrnet_config,
    dlrnet_param_count,
    fuse_decoder_layers,
    load_dlrnet_weights,
    locked_model_from_config,
    replace_layer_mlp,
    save_dlrnet_weights,
    set_checkpointing,
    set_fast_path,
    write_config,
)
from . import evaluate, harness, ops, packed, registry, sharding  # noqa: F401
from .evaluate import evaluate_ppl, synthetic_token_stream  # noqa: F401
from .packed import PackedNet, load_packed_weights, pack_state_dict  # noqa: F401

__version__ = "0.1.0"
