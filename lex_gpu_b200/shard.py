"""Column-parallel `gemm_fp4` over several GPUs, one process per GPU.

The reference is single-GPU (crates/lex-cuda/src/device.rs:358-359 opens device 0); this is new.
W's rows are independent, so rank r owns the rows lexb_shard_rows gives it - whole 128-row tiles of
wq, ws and wg - and computes y[:, n0:n1] from all of x with no reduction.  Only when a caller needs
full rows is anything exchanged: an all-gather of the y shards (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .device import shard_rows


@dataclass(frozen=True)
class RowShard:
    n: int
    world: int
    rank: int
    n0: int
    n1: int

    @classmethod
    def of(cls, n: int, world: int, rank: int) -> "RowShard":
        n0, n1 = shard_rows(n, world, rank)
        return cls(n, world, rank, n0, n1)

    @property
    def rows(self) -> int:
        return self.n1 - self.n0

    def spans(self) -> list[tuple[int, int]]:
        return [shard_rows(self.n, self.world, r) for r in range(self.world)]

    def max_rows(self) -> int:
        return max(b - a for a, b in self.spans())

    def slice_weights(self, wq: np.ndarray, ws: np.ndarray, wg: np.ndarray):
        """This rank's slab of each weight array (views: contiguous row ranges)."""
        return wq[self.n0:self.n1], ws[self.n0:self.n1], wg[self.n0:self.n1]


def all_gather_y(y_local, shard: RowShard, group=None):
    """All-gather of the y shards into [world][m][max_rows] (shards shorter than the longest are
    padded with zeros on the right).  y_local: torch tensor [m, rows] on the device the process
    group's backend works with."""
    import torch
    import torch.distributed as dist
    m = y_local.shape[0]
    width = shard.max_rows()
    if y_local.shape[1] != width:
        padded = torch.zeros((m, width), dtype=y_local.dtype, device=y_local.device)
        padded[:, :y_local.shape[1]] = y_local
        y_local = padded
    out = torch.empty((shard.world * m, width), dtype=y_local.dtype, device=y_local.device)   # concatenated on dim 0
    dist.all_gather_into_tensor(out, y_local.contiguous(), group=group)
    return out.view(shard.world, m, width)


def assemble(gathered, shard: RowShard):
    """[world][m][max_rows] -> y[m, n] (a copy; callers that can consume the gathered layout should)."""
    import torch
    m = gathered.shape[1]
    y = torch.empty((m, shard.n), dtype=gathered.dtype, device=gathered.device)
    for r, (a, b) in enumerate(shard.spans()):
        y[:, a:b] = gathered[r, :, :b - a]
    return y


class SymmetricY:
    """A gathered y[m, n] on every rank (f32 by default; f16 for the gathered activation silu(gate) * up), allocated
    as symmetric memory so that each rank holds the device addresses of all ranks' buffers (`ptrs`), which is what
    lexb_gemm_fp4_launch_gather and lexb_gemm_fp4_silu_launch_gather store to."""

    def __init__(self, m: int, n: int, group, dtype=None):
        import torch
        import torch.distributed._symmetric_memory as symm
        self.tensor = symm.empty((m, n), dtype=dtype or torch.float32, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]

    def barrier(self) -> None:
        """All ranks' work queued so far on the current stream is done before any rank continues."""
        self.handle.barrier()
