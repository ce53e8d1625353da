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

import ctypes

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


def slot_layout(sizes: list[tuple[int, int]]) -> tuple[list[int], int]:
    """Byte offsets of the [n][m_total] fp32 outputs in one shared buffer, each on a
    256-byte boundary, and the buffer's size.  `sizes` holds (n, m_total) per slot."""
    offs, at = [], 0
    for n, m_total in sizes:
        offs.append(at)
        at += (n * m_total * 4 + 255) // 256 * 256
    return offs, at


class PeerOutputs:
    """Output buffers of the row-sharded decode matvec that every rank's kernel writes
    into directly (okf_gemm_gather), instead of an all-gather after the kernel.

    Every rank allocates one shared buffer holding all its output slots plus one
    arrival counter, publishes the two IPC handles through the process
    group, and maps every other rank's pair.  `slot(i, m_local)` is the okf_gather
    record of output i for this rank's rows.  All ranks must create the object
    with the same `sizes` and run the same sequence of gathered calls."""

    def __init__(self, ctx, sizes: list[tuple[int, int]], group=None, free: bool = False):
        """`free`: the slots carry OKF_GATHER_FREE (no launch waits for the exchange before
        it; the caller ends a batch of calls with CudaEnc.gather_wait())."""
        from . import _lib

        self.free = bool(free)

        self.ctx, self.group = ctx, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.sizes = list(sizes)
        self.offs, out_bytes = slot_layout(self.sizes)
        lib = ctx.lib
        self._mine, handles = [], []
        # one arrival counter (and one pair of epoch words) for all slots: a wait on it covers
        # every exchange launched so far
        for nbytes in (out_bytes, 256):
            p, h = ctypes.c_void_p(), _lib.IpcHandle()
            ctx._check(lib.okf_shared_alloc(ctx.h, nbytes, ctypes.byref(p), ctypes.byref(h)), "okf_shared_alloc")
            self._mine.append(p.value)
            handles.append(bytes(h.bytes))
        # the library's own two words for the counter (okf_gather.epoch)
        self.epochs = torch.zeros(2, dtype=torch.int32, device=f"cuda:{ctx.device}")
        everyone = [None] * self.world
        dist.all_gather_object(everyone, handles, group=group)
        self._opened = []
        self.out_base, self.cnt_base = [0] * self.world, [0] * self.world
        for r, (h_out, h_cnt) in enumerate(everyone):
            if r == self.rank:
                self.out_base[r], self.cnt_base[r] = self._mine
                continue
            ptrs = []
            for raw in (h_out, h_cnt):
                h, p = _lib.IpcHandle(), ctypes.c_void_p()
                ctypes.memmove(h.bytes, raw, 64)
                ctx._check(lib.okf_shared_open(ctx.h, ctypes.byref(h), ctypes.byref(p)), "okf_shared_open")
                ptrs.append(p.value)
                self._opened.append(p.value)
            self.out_base[r], self.cnt_base[r] = ptrs
        self._slots = {}

    def slot(self, i: int, m_local: int):
        """okf_gather for output slot i; this rank owns rows [rank * m_local, +m_local)."""
        from . import _lib

        key = (i, m_local)
        if key not in self._slots:
            n, m_total = self.sizes[i]
            g = _lib.Gather()
            g.nranks, g.rank, g.m_total, g.row_first = self.world, self.rank, m_total, self.rank * m_local
            for r in range(self.world):
                g.out[r] = self.out_base[r] + self.offs[i]
                g.arrivals[r] = self.cnt_base[r]
            g.epoch = self.epochs.data_ptr()
            g.flags = 1 if self.free else 0
            self._slots[key] = g
        return self._slots[key]

    def read(self, i: int) -> np.ndarray:
        """This rank's copy of output slot i as a host array [n][m_total]."""
        n, m_total = self.sizes[i]
        host = np.empty((n, m_total), dtype=np.float32)
        self.ctx._check(self.ctx.lib.okf_copy_to_host(self.ctx.h, self.out_base[self.rank] + self.offs[i],
                                                      host.ctypes.data, host.nbytes), "okf_copy_to_host")
        return host

    def read_into(self, i: int, host: torch.Tensor):
        """Copy this rank's copy of output slot i into a host tensor of the same size."""
        n, m_total = self.sizes[i]
        assert host.numel() * host.element_size() == n * m_total * 4 and host.is_contiguous()
        self.ctx._check(self.ctx.lib.okf_copy_to_host(self.ctx.h, self.out_base[self.rank] + self.offs[i],
                                                      host.data_ptr(), n * m_total * 4), "okf_copy_to_host")

    def close(self):
        """Unmap the other ranks' buffers, then (after a barrier) free this rank's."""
        lib = self.ctx.lib
        for p in self._opened:
            lib.okf_shared_close(self.ctx.h, p)
        self._opened = []
        dist.barrier(group=self.group)
        for p in self._mine:
            lib.okf_shared_free(self.ctx.h, p)
        self._mine = []
