"""Checkpoint -> packed device weights, without building the modules.

The reference loads ``layerNN.pt`` files into ``nn.Module`` parameters
(dlr_lock/model.py:232-248) and packs them for its kernels afterwards
(kernels/reference.py:68-91): 4L small tensors per net on the way.  A serving process
needs only the folded stacks V' (L, r, d) and U' (L, d, r) on the device.  This module
reads each file once, stacks and folds on the device, and can keep the packed form
beside the checkpoint so that the next start skips the stacking and folding.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import ops

_KEY = re.compile(r"^(?:_orig_mod\.)?(Vs|Us|rms_w|alphas)\.(\d+)$")


@dataclass
class PackedNet:
    """One DLR-Net as the CUDA library takes it."""
    Vp: torch.Tensor          # (L, r, d) bf16, V * rms_w
    Up: torch.Tensor          # (L, d, r) bf16, alpha * U
    eps: float = 1e-6

    @property
    def depth(self) -> int:
        return self.Vp.shape[0]

    @property
    def r(self) -> int:
        return self.Vp.shape[1]

    @property
    def d(self) -> int:
        return self.Vp.shape[2]

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return ops.forward_folded(x, self.Vp, self.Up, self.eps)


def pack_state_dict(sd: dict, device, eps: float = 1e-6, dtype: torch.dtype = torch.bfloat16) -> PackedNet:
    """Fold one net's ``state_dict`` (keys ``Vs.i``, ``Us.i``, ``rms_w.i``, ``alphas.i``) on ``device``.

    Every tensor, alpha included, is first rounded to ``dtype``, the dtype the serving module would hold
    it in: the reference writes fp32 ``layerNN.pt`` files (dlr_lock/distill_logits.py:196-200) and loads
    them into a bf16 module (``replace_layer_mlp`` casts to the layer's dtype, dlr_lock/model.py:171-172)
    before its packer runs, so alpha reaches the fold as a bf16 value.  The result is then bit-identical to
    ``DLRNet.folded_weights()`` of a module loaded from the same file."""
    groups = {"Vs": {}, "Us": {}, "rms_w": {}, "alphas": {}}
    for k, v in sd.items():
        m = _KEY.match(k)
        if m:
            groups[m.group(1)][int(m.group(2))] = v
    L = len(groups["Vs"])
    if L == 0 or any(len(g) != L or sorted(g) != list(range(L)) for g in groups.values()):
        raise ValueError("not a DLR-Net state dict: need Vs.i, Us.i, rms_w.i, alphas.i for i = 0..L-1")
    stack = lambda name: torch.stack([groups[name][i] for i in range(L)]).to(dtype).to(device, non_blocking=True)
    Vp, Up = ops.fold_weights(stack("Vs"), stack("Us"), stack("rms_w"), stack("alphas"))
    return PackedNet(Vp, Up, eps)


def _cache_path(checkpoint_dir: str, li: int) -> str:
    return os.path.join(checkpoint_dir, "packed_b200", f"layer{li:02d}.pt")


def load_packed_weights(checkpoint_dir: str, device, n_layers: Optional[int] = None, eps: float = 1e-6,
                        use_cache: bool = True, write_cache: bool = False) -> List[PackedNet]:
    """Read ``layerNN.pt`` (dlr_lock/model.py:251-262 wrote them) into packed nets on ``device``.

    With ``write_cache`` the folded stacks are saved under ``<dir>/packed_b200/``; with ``use_cache`` a saved
    stack is taken instead of the checkpoint file when it is at least as new.
    """
    device = torch.device(device)
    if n_layers is None:
        n_layers = len([f for f in os.listdir(checkpoint_dir) if re.fullmatch(r"layer\d+\.pt", f)])
    nets = []
    for li in range(n_layers):
        src = os.path.join(checkpoint_dir, f"layer{li:02d}.pt")
        cached = _cache_path(checkpoint_dir, li)
        if use_cache and os.path.exists(cached) and os.path.getmtime(cached) >= os.path.getmtime(src):
            blob = torch.load(cached, map_location=device, weights_only=True)
            # the folded stacks do not depend on epsilon: the caller's value applies, not the one stored
            nets.append(PackedNet(blob["Vp"], blob["Up"], eps))
            continue
        sd = torch.load(src, map_location="cpu", weights_only=True)
        net = pack_state_dict(sd, device, eps)
        if write_cache:
            os.makedirs(os.path.dirname(cached), exist_ok=True)
            torch.save({"Vp": net.Vp.cpu(), "Up": net.Up.cpu(), "eps": torch.tensor(net.eps)}, cached)
        nets.append(net)
    return nets
