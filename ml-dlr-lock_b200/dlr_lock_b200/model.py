"""Host-side mirror of the reference module API around the B200 forward.

``DLRNet`` here has the constructor, attributes, parameter names and
``state_dict`` keys of ``dlr_lock.model.DLRNet`` (dlr_lock/model.py:38-101), so
reference checkpoints load unchanged.  Its ``forward`` runs the CUDA library
when the call is inference on bf16 CUDA tensors, and otherwise (CPU, fp32,
gradients needed) evaluates the same layer loop with torch ops so that the
reference's training scripts keep working on top of it.

``accelerate_locked_model`` swaps the DLR-Nets of a model built by the
reference's own ``build_locked_model`` for this class, sharing the parameters.
"""
from __future__ import annotations

import json
import math
import os
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as _checkpoint

from . import ops


def dlrnet_param_count(d: int, r: int, depth: int) -> int:
    """Parameters of one DLR-Net: per layer U and V (2dr), the gain (d), alpha (1).
    Mirrors dlr_lock/model.py:125-127."""
    return depth * (2 * d * r + d + 1)


def compute_depth(d: int, d_ff: int, r: int, multiplier: float = 1.0) -> int:
    """Depth that fits ``multiplier`` x the 3*d*d_ff parameters of a SwiGLU MLP
    (dlr_lock/model.py:130-139); at least 2."""
    return max(int(3 * d * d_ff * multiplier) // (2 * d * r + d + 1), 2)


def dlrnet_config(d: int, d_ff: int, r: int, multiplier: float = 1.0) -> dict:
    """JSON-serialisable summary with the keys of dlr_lock/model.py:142-153."""
    depth = compute_depth(d, d_ff, r, multiplier)
    return {"d": d, "d_ff": d_ff, "rank": r, "multiplier": multiplier, "depth": depth,
            "params": dlrnet_param_count(d, r, depth), "swiglu_params": 3 * d * d_ff}


def write_config(path, d, d_ff, r, multiplier=1.0):
    """dlr_lock/model.py:282-285."""
    with open(path, "w") as f:
        json.dump(dlrnet_config(d, d_ff, r, multiplier), f, indent=2)


class DLRNet(nn.Module):
    """Depth-``depth`` stack of rank-``r`` residual updates over a width-``d`` state.

    h <- h + alpha_i * U_i silu(V_i RMSNorm_i(h)), i = 0..depth-1
    (dlr_lock/model.py:93-101).  Parameters: ``Vs[i]`` (r,d), ``Us[i]`` (d,r),
    ``rms_w[i]`` (d,), ``alphas[i]`` scalar; initialisation as
    dlr_lock/model.py:65-81.
    """

    def __init__(self, d, r, depth, alpha_init=0.0, eps=1e-6):
        super().__init__()
        self.d, self.r, self.depth, self.eps = d, r, depth, eps
        sv = 1.0 / math.sqrt(d)
        su = 1.0 / math.sqrt(r * depth)
        self.Vs = nn.ParameterList([nn.Parameter(torch.randn(r, d) * sv) for _ in range(depth)])
        self.Us = nn.ParameterList([nn.Parameter(torch.randn(d, r) * su) for _ in range(depth)])
        self.rms_w = nn.ParameterList([nn.Parameter(torch.ones(d)) for _ in range(depth)])
        self.alphas = nn.ParameterList([nn.Parameter(torch.tensor(float(alpha_init))) for _ in range(depth)])
        self.use_checkpoint = True
        self._folded = None       # (key, V', U') derived cache, rebuilt when parameters change
        self.fast = True          # set False to force the torch loop

    # ---- adoption of an existing (reference) module's parameters -------------
    @classmethod
    def adopt(cls, other: nn.Module) -> "DLRNet":
        """Wrap the parameters of a reference-style DLR-Net without copying them."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.d, self.r, self.depth = other.d, other.r, other.depth
        self.eps = getattr(other, "eps", 1e-6)
        self.Vs, self.Us, self.rms_w, self.alphas = other.Vs, other.Us, other.rms_w, other.alphas
        self.use_checkpoint = getattr(other, "use_checkpoint", True)
        self._folded = None
        self.fast = True
        self.train(other.training)
        return self

    # ---- derived folded weights ----------------------------------------------
    def _cache_key(self):
        # every parameter of every layer: storage address and in-place version counter.  A write through
        # ``p.data`` (``p.data.copy_(...)``) bumps neither: call ``invalidate()`` after such an edit.
        key = []
        for plist in (self.Vs, self.Us, self.rms_w, self.alphas):
            for p in plist:
                key.append(p.data_ptr())
                key.append(p._version)
        return tuple(key)

    def invalidate(self):
        """Drop the folded weights; they are rebuilt on the next fast forward.  Needed after writes
        that bypass autograd's version counter (``p.data.copy_``, ``p.data[...] = ``)."""
        self._folded = None

    def folded_weights(self):
        """(V' (L,r,d), U' (L,d,r)) bf16 on the parameters' device, cached."""
        key = self._cache_key()
        if self._folded is None or self._folded[0] != key:
            V = torch.stack([p.detach() for p in self.Vs])
            U = torch.stack([p.detach() for p in self.Us])
            w = torch.stack([p.detach() for p in self.rms_w])
            a = torch.stack([p.detach() for p in self.alphas])
            Vp, Up = ops.fold_weights(V, U, w, a)
            self._folded = (key, Vp, Up)
        return self._folded[1], self._folded[2]

    def _load_from_state_dict(self, *args, **kwargs):
        self.invalidate()
        return super()._load_from_state_dict(*args, **kwargs)

    def _apply(self, fn, *args, **kwargs):
        self.invalidate()
        return super()._apply(fn, *args, **kwargs)

    def train(self, mode: bool = True):
        if mode:
            self.invalidate()
        return super().train(mode)

    # ---- forward ---------------------------------------------------------------
    def _fast_ok(self, x: torch.Tensor) -> bool:
        if not self.fast or not x.is_cuda or x.dtype != torch.bfloat16:
            return False
        if self.Vs[0].dtype != torch.bfloat16:
            return False
        # the library returns a tensor without an autograd graph: whenever a gradient could be asked for,
        # towards the input or towards any parameter, in train or eval mode, the torch loop runs
        # (the reference's forward always builds the graph, dlr_lock/model.py:88-101)
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            return False
        return True

    def forward(self, x):
        if self._fast_ok(x):
            Vp, Up = self.folded_weights()
            return ops.forward_folded(x, Vp, Up, self.eps)
        if self.use_checkpoint and torch.is_grad_enabled() and x.requires_grad:
            return _checkpoint(self._forward_impl, x, use_reentrant=False)
        return self._forward_impl(x)

    def _forward_impl(self, x):
        """The layer loop in torch ops, one op per line of dlr_lock/model.py:96-100.
        Taken for training, fp32 and CPU tensors; never used as a fallback for a
        failed CUDA call."""
        h = x
        for V, U, w, a in zip(self.Vs, self.Us, self.rms_w, self.alphas):
            rstd = torch.rsqrt(h.pow(2).mean(dim=-1, keepdim=True) + self.eps)
            z = (h * w * rstd) @ V.T
            h = h + a * (F.silu(z) @ U.T)
        return h


class ResidualDLRNet(nn.Module):
    """``dlrnet(h) - h``: with the layer's post-attention norm replaced by the
    identity, the host decoder layer's ``h + mlp(h)`` becomes ``dlrnet(h)``
    (dlr_lock/model.py:104-122)."""

    def __init__(self, dlrnet):
        super().__init__()
        self.dlrnet = dlrnet

    def forward(self, h):
        return self.dlrnet(h) - h


def _strip_compile_prefix(sd: dict) -> dict:
    if any(k.startswith("_orig_mod.") for k in sd):
        return {k.removeprefix("_orig_mod."): v for k, v in sd.items()}
    return sd


def replace_layer_mlp(model, layer_idx, d, rank, depth, state_dict=None, alpha_init=0.0):
    """Swap one decoder layer's MLP for a DLR-Net in place (dlr_lock/model.py:156-176)."""
    net = DLRNet(d, rank, depth, alpha_init=alpha_init)
    if state_dict is not None:
        net.load_state_dict(_strip_compile_prefix(state_dict))
    layer = model.model.layers[layer_idx]
    like = next(layer.parameters())
    net = net.to(device=like.device, dtype=like.dtype)
    layer.post_attention_layernorm = nn.Identity()
    layer.mlp = ResidualDLRNet(net)
    return net


def build_locked_model(model_name, rank, multiplier=1.0, state_dicts=None, device="cpu", device_map=None,
                       torch_dtype=torch.bfloat16, attn_implementation="sdpa", alpha_init=0.0, verbose=True,
                       revision=None):
    """Load a causal LM and replace every MLP by a DLR-Net (dlr_lock/model.py:179-229).

    The loading itself is the host framework's ``from_pretrained``; only the
    surgery is this package's concern.
    """
    from transformers import AutoModelForCausalLM

    kw = dict(dtype=torch_dtype, attn_implementation=attn_implementation)
    if revision is not None:
        kw["revision"] = revision
    if device_map is not None:
        model = AutoModelForCausalLM.from_pretrained(model_name, device_map=device_map, **kw)
    else:
        model = AutoModelForCausalLM.from_pretrained(model_name, **kw).to(device)
    d, d_ff = model.config.hidden_size, model.config.intermediate_size
    depth = compute_depth(d, d_ff, rank, multiplier)
    n_layers = len(model.model.layers)
    if verbose:
        cfg = dlrnet_config(d, d_ff, rank, multiplier)
        print(f"Replacing {n_layers} MLPs with DLRNet(d={d}, r={rank}, depth={depth}); "
              f"{cfg['params']:,} params each ({cfg['params'] / cfg['swiglu_params']:.2f}x SwiGLU)")
    for li in range(n_layers):
        sd = state_dicts.get(li) if state_dicts is not None else None
        replace_layer_mlp(model, li, d, rank, depth, state_dict=sd, alpha_init=alpha_init)
    return model


def locked_model_from_config(config, rank, multiplier=1.0, device="cpu", torch_dtype=torch.bfloat16,
                             alpha_init=0.0):
    """A randomly initialised causal LM of ``config`` with every MLP replaced by a DLR-Net: what
    ``build_locked_model`` returns, minus the checkpoint (no files, no network).  Used where only the
    shapes matter: timing and parity of the whole decoder loop."""
    from transformers import AutoModelForCausalLM

    with torch.device(device):
        model = AutoModelForCausalLM.from_config(config, dtype=torch_dtype)
    d, d_ff = model.config.hidden_size, model.config.intermediate_size
    depth = compute_depth(d, d_ff, rank, multiplier)
    for li in range(len(model.model.layers)):
        replace_layer_mlp(model, li, d, rank, depth, alpha_init=alpha_init)
    return model


def set_fast_path(model, enabled: bool) -> int:
    """Switch every DLR-Net of ``model`` between the CUDA library and the torch layer loop."""
    n = 0
    for m in model.modules():
        if isinstance(m, DLRNet):
            m.fast = bool(enabled)
            n += 1
    return n


def load_dlrnet_weights(model, checkpoint_dir, n_layers=None):
    """Read ``layerNN.pt`` files into the model's DLR-Nets (dlr_lock/model.py:232-248)."""
    n = len(model.model.layers) if n_layers is None else n_layers
    for li in range(n):
        sd = torch.load(os.path.join(checkpoint_dir, f"layer{li:02d}.pt"), map_location="cpu", weights_only=True)
        model.model.layers[li].mlp.dlrnet.load_state_dict(_strip_compile_prefix(sd))
    return n


def save_dlrnet_weights(model, checkpoint_dir, n_layers=None):
    """Write every DLR-Net's ``state_dict`` as ``layerNN.pt`` (dlr_lock/model.py:251-262)."""
    os.makedirs(checkpoint_dir, exist_ok=True)
    n = len(model.model.layers) if n_layers is None else n_layers
    for li in range(n):
        sd = {k: v.cpu() for k, v in model.model.layers[li].mlp.dlrnet.state_dict().items()}
        torch.save(sd, os.path.join(checkpoint_dir, f"layer{li:02d}.pt"))
    return n


def _is_dlrnet_like(m) -> bool:
    return all(hasattr(m, a) for a in ("Vs", "Us", "rms_w", "alphas", "d", "r", "depth"))


def set_checkpointing(model, enabled):
    """Toggle activation checkpointing of every DLR-Net (dlr_lock/model.py:265-279)."""
    n = 0
    for layer in model.model.layers:
        net = getattr(layer.mlp, "dlrnet", layer.mlp)
        if _is_dlrnet_like(net):
            net.use_checkpoint = enabled
            n += 1
    return n


def _fused_locked_layer_forward(self, hidden_states, **kwargs):
    """A locked pre-norm decoder layer with the MLP branch's residual arithmetic cancelled.

    The host framework computes ``h = x + attn(norm(x))`` and then ``h + mlp(post_norm(h))``; in a locked
    layer ``post_norm`` is the identity and ``mlp`` is ``ResidualDLRNet``, i.e. ``dlrnet(h) - h``
    (dlr_lock/model.py:104-122, 174-175), so the layer's output is ``dlrnet(h)``.  Here the attention
    output goes straight into the net and the net's output is the layer's output: the ``- h`` and the
    ``+ h`` (two passes over the activations and two launches per layer) never run.  Arguments are passed
    through to the layer's own attention module unchanged.
    """
    attn = self.self_attn(hidden_states=self.input_layernorm(hidden_states), **kwargs)
    if isinstance(attn, tuple):
        attn = attn[0]
    return self.mlp.dlrnet(hidden_states + attn)


def _fusable(layer) -> bool:
    return (isinstance(getattr(layer, "mlp", None), ResidualDLRNet)
            and isinstance(getattr(layer, "post_attention_layernorm", None), nn.Identity)
            and hasattr(layer, "input_layernorm") and hasattr(layer, "self_attn"))


def fuse_decoder_layers(model, enabled: bool = True) -> int:
    """Switch every locked decoder layer of ``model`` between the host framework's own forward (the
    reference composition ``h + (dlrnet(h) - h)``) and the fused one (``dlrnet(h)``).  Only layers of the
    standard pre-norm form are touched (``input_layernorm``, ``self_attn``, an identity
    ``post_attention_layernorm`` and a ``ResidualDLRNet`` as ``mlp``).  Returns how many were switched."""
    import types
    n = 0
    for layer in model.model.layers:
        if not _fusable(layer):
            continue
        if enabled:
            layer.forward = types.MethodType(_fused_locked_layer_forward, layer)
        elif "forward" in layer.__dict__:
            del layer.__dict__["forward"]
        n += 1
    return n


def accelerate_locked_model(model, fuse_layers: bool = False) -> int:
    """Route every DLR-Net of a locked model through the B200 library.

    Works on models built by this package or by the reference's
    ``build_locked_model``: each ``layers[i].mlp.dlrnet`` that is not already a
    :class:`DLRNet` of this package is replaced by one that shares its
    parameters, so ``load_dlrnet_weights`` / ``save_dlrnet_weights`` /
    ``set_checkpointing`` keep working.  With ``fuse_layers`` the decoder layers also
    take the fused forward of ``fuse_decoder_layers``.  Returns the number of nets routed.
    """
    n = 0
    for layer in model.model.layers:
        mlp = layer.mlp
        net = getattr(mlp, "dlrnet", None)
        if net is None or not _is_dlrnet_like(net):
            continue
        if not isinstance(net, DLRNet):
            mlp.dlrnet = DLRNet.adopt(net)
        n += 1
    if fuse_layers:
        # layers built by the reference carry its own wrapper class: same shape, re-wrapped so that the
        # fused forward recognises them
        for layer in model.model.layers:
            mlp = getattr(layer, "mlp", None)
            if mlp is not None and not isinstance(mlp, ResidualDLRNet) and _is_dlrnet_like(getattr(mlp, "dlrnet", None) or object()):
                layer.mlp = ResidualDLRNet(mlp.dlrnet)
        fuse_decoder_layers(model, True)
    return n
