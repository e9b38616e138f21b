"""Row-sharded multi-GPU driver.

Token rows never interact in a DLR-Net (dlr_lock/model.py:93-101 has no
cross-row op), so N GPUs split the rows into contiguous blocks, each rank runs
the single-GPU forward on its block against its own replica of the folded
weights, and the only communication is the final gather of the output rows.
One process per GPU; ``torch.distributed`` (NCCL on GPUs, gloo in CPU tests)
supplies the gather.
"""
from __future__ import annotations

from typing import Callable, List, Tuple

import torch
import torch.distributed as dist


def row_blocks(M: int, world: int, tile: int = 1) -> List[Tuple[int, int]]:
    """Contiguous [start, stop) row ranges, one per rank.

    Blocks are multiples of ``tile`` rows except the last non-empty one; ranks
    beyond the work get empty ranges (M < world: independent requests are better
    served as replicas).
    """
    if M < 0 or world <= 0 or tile <= 0:
        raise ValueError("row_blocks needs M >= 0, world > 0, tile > 0")
    tiles = -(-M // tile)
    base, extra = divmod(tiles, world)
    out, start = [], 0
    for rank in range(world):
        n = (base + (1 if rank < extra else 0)) * tile
        stop = min(M, start + n)
        out.append((start, stop))
        start = stop
    return out


class RowShardedForward:
    """Run ``forward(x_block)`` on this rank's rows; optionally gather the result.

    ``forward`` is the single-GPU callable (e.g. ``DLRNet.forward`` or
    ``ops.forward_folded`` bound to this rank's weights).
    """

    def __init__(self, forward: Callable[[torch.Tensor], torch.Tensor], tile: int = 128, group=None):
        self.forward = forward
        self.tile = tile
        self.group = group

    @property
    def world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group) if dist.is_initialized() else 0

    def local_rows(self, M: int) -> Tuple[int, int]:
        return row_blocks(M, self.world, self.tile)[self.rank]

    def run_local(self, x_full: torch.Tensor) -> torch.Tensor:
        """Forward of this rank's block of a replicated (M, d) input."""
        a, b = self.local_rows(x_full.shape[0])
        return self.forward(x_full[a:b])

    def gather(self, y_local: torch.Tensor, M: int) -> torch.Tensor:
        """All ranks receive the full (M, d) output (blocks may differ in size)."""
        if self.world == 1:
            return y_local
        blocks = row_blocks(M, self.world, self.tile)
        d = y_local.shape[-1]
        longest = max(b - a for a, b in blocks)
        pad = torch.zeros((longest, d), dtype=y_local.dtype, device=y_local.device)
        pad[: y_local.shape[0]] = y_local
        out = torch.empty((self.world * longest, d), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(out, pad, group=self.group)
        parts = [out[i * longest: i * longest + (b - a)] for i, (a, b) in enumerate(blocks)]
        return torch.cat(parts, dim=0)

    def __call__(self, x_full: torch.Tensor, gather: bool = True) -> torch.Tensor:
        y = self.run_local(x_full)
        return self.gather(y, x_full.shape[0]) if gather else y
