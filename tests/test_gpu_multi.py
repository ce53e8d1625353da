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
    the rows are stored into both copies, the wait gives up after about a second,
    the status word says so and the context stays usable."""
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
    counters = torch.zeros(3, dtype=torch.int32, device="cuda")  # two arrival counters and the epoch
    g = _lib.Gather()
    g.nranks, g.rank, g.m_total, g.row_first = 2, 0, m_total, 0
    for r in range(2):
        g.out[r] = outs[r].data_ptr()
        g.arrivals[r] = counters.data_ptr() + 4 * r
    g.epoch = counters.data_ptr() + 8
    enc.gemm_gather(GGUFTensor("w", (k, m), ty), torch.from_numpy(x).cuda(), g, shard0, 1)
    torch.cuda.synchronize()
    assert ctx.device_status() == 4
    for o in outs:
        got = o.cpu().numpy()
        assert rel_err(got[:m], ref[:m]) <= 1e-4
        assert np.isnan(got[m:]).all()  # the other rank's rows were never written
    assert counters.cpu().tolist()[2] == 1
    # the context still works
    out = torch.empty(m, device="cuda")
    enc.gemv(GGUFTensor("w", (k, m), ty), torch.from_numpy(x).cuda(), out, shard0)
    torch.cuda.synchronize()
    assert rel_err(out.cpu().numpy(), ref[:m]) <= 1e-4


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
