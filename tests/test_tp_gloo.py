"""Row sharding + all-gather on two CPU ranks over gloo.  The local compute is
the CPU oracle here (tests may use it); on GPUs it is CudaEnc.gemm."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from chatokf_b200 import tp
from chatokf_b200.gguf_types import GGUFType, row_byte_count
from helpers import make_weights


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ty, k, m, n, blocks, x, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shard = tp.shard_rows(ty, blocks, k, m, rank, world)

        def compute(xt, nn, out_local):
            y = oracle.matmul(ty, shard, k, m // world, xt.numpy(), nn, threads=1)
            out_local.copy_(torch.from_numpy(y))

        lin = tp.ShardedLinear(ty, k, m, compute)
        full = lin.forward(torch.from_numpy(x), n)
        q.put((rank, full.numpy().copy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ty,n", [(GGUFType.Q4_K, 1), (GGUFType.IQ2_XXS, 4), (GGUFType.Q2_0, 3)])
def test_sharded_linear_two_ranks(ty, n):
    k, m, world = 512, 16, 2
    blocks = make_weights(ty, m, k, seed=1)
    x = np.random.default_rng(0).normal(size=(n, k)).astype(np.float32)
    want = oracle.matmul(ty, blocks, k, m, x, n, threads=1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, int(ty), k, m, n, blocks, x, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        assert np.array_equal(got[r], want), "every rank holds the full, identical output"


def test_shard_bounds_and_bytes():
    ty, k, m = GGUFType.IQ2_XXS, 5120, 1024
    rb = row_byte_count(ty, k)
    blocks = np.arange(rb * m, dtype=np.uint64).astype(np.uint8)
    parts = [tp.shard_rows(ty, blocks, k, m, r, 8) for r in range(8)]
    assert all(p.size == rb * m // 8 for p in parts)
    assert np.array_equal(np.concatenate(parts), blocks)
    with pytest.raises(ValueError):
        tp.shard_bounds(1001, 0, 8)


def test_token_major_layout():
    g = torch.arange(2 * 3 * 4).reshape(2, 3, 4)  # [world][n][m_local]
    t = tp.to_token_major(g)
    assert t.shape == (3, 8)
    assert t[1].tolist() == [4, 5, 6, 7, 16, 17, 18, 19]


def test_slot_layout_of_shared_outputs():
    """Outputs that other ranks write into share one buffer: 256-byte aligned slots."""
    from chatokf_b200.tp import slot_layout

    offs, total = slot_layout([(1, 9728), (1, 9728), (4, 2560), (1, 3)])
    assert offs == [0, 38912, 77824, 118784]
    assert total == 118784 + 256
    assert all(o % 256 == 0 for o in offs)
