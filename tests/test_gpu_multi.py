"""Decode matvec on row shards with the gather fused into the kernel.

The two-GPU case runs as child processes (one per GPU) and is skipped on a
single-GPU machine; the bounded wait is checked on one GPU with a peer that never
arrives, which costs about a second and faults nothing."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import oracle
from chatokf_b200 import _lib
from chatokf_b200.enc import Context, CudaEnc, GGUFTensor
from chatokf_b200.gguf_types import GGUFType
from helpers import lcg_fill, make_weights, rel_err

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_that_never_arrives_times_out_and_data_is_in_place():
    """nranks = 2 with both ranks' buffers on this GPU and nobody playing rank 1:
    the rows are stored into both copies and the launch ends without waiting; the wait
    that follows gives up after about a second, the status word says so and the
    context stays usable."""
    ctx = Context(0)  # its own status word
    enc = CudaEnc(ctx)
    ty, k, m_total = GGUFType.Q4_K, 1024, 512
    m = m_total // 2
    blocks = make_weights(ty, m_total, k, seed=3)
    x = lcg_fill(k, 9)
    ref = oracle.matvec(ty, blocks, k, m_total, x)
    rb = blocks.view(np.uint8).reshape(-1).size // m_total
    shard0 = ctx.upload(blocks.view(np.uint8).reshape(-1)[: rb * m])
    outs = [torch.full((m_total,), float("nan"), device="cuda") for _ in range(2)]
    counters = torch.zeros(4, dtype=torch.int32, device="cuda")  # two arrival counters and the two epoch words
    g = _lib.Gather()
    g.nranks, g.rank, g.m_total, g.row_first = 2, 0, m_total, 0
    for r in range(2):
        g.out[r] = outs[r].data_ptr()
        g.arrivals[r] = counters.data_ptr() + 4 * r
    g.epoch = counters.data_ptr() + 8
    xd = torch.from_numpy(x).cuda()
    enc.gemm_gather(GGUFTensor("w", (k, m), ty), xd, g, shard0, 1)
    torch.cuda.synchronize()
    assert ctx.device_status() == 0  # nobody has waited yet
    # the exchange is launched (two counts expected on this rank's counter) but not announced yet
    assert counters.cpu().tolist() == [0, 0, 2, 0]
    enc.gather_wait()
    torch.cuda.synchronize()
    assert counters.cpu().tolist() == [1, 1, 2, 0]  # announced on both counters; rank 1 never comes
    assert ctx.device_status() == 4
    for o in outs:
        got = o.cpu().numpy()
        assert rel_err(got[:m], ref[:m]) <= 1e-4
        assert np.isnan(got[m:]).all()  # the other rank's rows were never written
    # a second gathered call, standing in for rank 1, completes both exchanges' count: no wait gives up
    ctx2 = Context(0)
    enc2 = CudaEnc(ctx2)
    shard1 = ctx2.upload(blocks.view(np.uint8).reshape(-1)[rb * m:])
    g1 = _lib.Gather()
    g1.nranks, g1.rank, g1.m_total, g1.row_first = 2, 1, m_total, m
    scratch = torch.zeros(2, dtype=torch.int32, device="cuda")
    for r in range(2):
        g1.out[r] = outs[r].data_ptr()
        g1.arrivals[r] = counters.data_ptr() + 4 * r
    g1.epoch = scratch.data_ptr()
    enc2.gemm_gather(GGUFTensor("w", (k, m), ty), xd, g1, shard1, 1)
    enc2.gather_wait()
    torch.cuda.synchronize()
    assert ctx2.device_status() == 0
    for o in outs:
        assert rel_err(o.cpu().numpy(), ref) <= 1e-4
    # the first context still works
    out = torch.empty(m, device="cuda")
    enc.gemv(GGUFTensor("w", (k, m), ty), xd, out, shard0)
    torch.cuda.synchronize()
    assert rel_err(out.cpu().numpy(), ref[:m]) <= 1e-4
    ctx2.close()


def test_gather_argument_checks(ctx):
    g = _lib.Gather()
    g.nranks = 1
    w = ctx.upload(make_weights(GGUFType.Q8_0, 16, 256, seed=1))
    x = torch.zeros(256, device="cuda")
    rc = ctx.lib.okf_gemm_gather(ctx.h, int(GGUFType.Q8_0), w.h, 0, 256, 16, x.data_ptr(), 0, 1, ctypes.byref(g), None)
    assert rc == -1


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_store_into_each_other():
    n = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    sys.stdout.write(r.stdout[-3000:])
    sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0
    assert r.stdout.count(": OK") == n
