"""Row-sharded (column-parallel) weights across the GPUs of one node.

The reference runs on a single device and has no counterpart for this file.
Output rows of W are independent, so rank g of G keeps rows
[g*M/G, (g+1)*M/G) -- one contiguous byte range of the tensor, because rows are
contiguous (LLM/Gemma/Gemma4Quant.swift:259,268) -- and computes its slice of
the output with the same kernels as the single-GPU path.  One all-gather over
NCCL reassembles the output on every rank.  Activations are replicated.

One process per GPU; `torch.distributed` provides the process group.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from .gguf_types import row_byte_count


def shard_bounds(m: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [lo, hi) owned by `rank`.  M must divide evenly so that every rank's
    slice of the gathered output has the same length."""
    if m % world:
        raise ValueError(f"M={m} is not divisible by the world size {world}")
    per = m // world
    return rank * per, (rank + 1) * per


def shard_rows(ty: int, blocks, k: int, m: int, rank: int, world: int) -> np.ndarray:
    """The bytes of this rank's rows, as a view of the full tensor's bytes."""
    b = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
    rb = row_byte_count(ty, k)
    assert b.size >= rb * m
    lo, hi = shard_bounds(m, rank, world)
    return b[lo * rb:hi * rb]


def gather_rows(local: torch.Tensor, n: int, m_local: int, group=None) -> torch.Tensor:
    """All-gather per-rank outputs local[n][m_local] into [world][n][m_local].

    For n == 1 the result, flattened, is the full output vector out[M].  For
    n > 1 the rank-major layout is returned as is; `to_token_major` turns it
    into the operator's out[n*M + m] layout when a consumer needs that."""
    world = dist.get_world_size(group)
    full = torch.empty((world, n, m_local), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(full.view(-1), local.reshape(-1).contiguous(), group=group)
    return full


def to_token_major(gathered: torch.Tensor) -> torch.Tensor:
    """[world][n][m_local] -> [n][world*m_local] (the reference's out[n*M + m])."""
    world, n, m_local = gathered.shape
    return gathered.permute(1, 0, 2).reshape(n, world * m_local)


class ShardedLinear:
    """One weight matrix W[M][K], rows split across the ranks of `group`.

    `compute(x, n, out_local)` runs the local slice: out_local[n][M/G] =
    X[n][K] . W_local^T.  On GPUs it is CudaEnc.gemm on this rank's shard; the
    CPU tests plug in another callable to exercise the sharding and the gather
    over gloo."""

    def __init__(self, ty: int, k: int, m: int, compute, group=None):
        self.ty, self.k, self.m = int(ty), int(k), int(m)
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.lo, self.hi = shard_bounds(self.m, self.rank, self.world)
        self.m_local = self.hi - self.lo
        self.compute = compute

    def forward(self, x: torch.Tensor, n: int, out_local: torch.Tensor | None = None,
                token_major: bool = True) -> torch.Tensor:
        if out_local is None:
            out_local = torch.empty((n, self.m_local), dtype=torch.float32, device=x.device)
        self.compute(x, n, out_local)
        full = gather_rows(out_local, n, self.m_local, self.group)
        if n == 1:
            return full.view(1, self.m)
        return to_token_major(full) if token_major else full
