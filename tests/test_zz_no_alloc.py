"""okf_gemm_noalloc: the matmul for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is off limits once work has
started -- inside a stream capture, in a decode loop with a latency budget, in a
host process that hands out a fixed memory budget.  For them the split-K matmul
has a twin whose partial-sum scratch is a fixed array inside the library instead
of a buffer the context grows on demand.  This file checks, through the C ABI,
that the twin gives what okf_gemm gives, twice in a row (the array is shared and
keeps the previous call's contents), and that it refuses shapes beyond its fixed
size.  It is named to be collected last, so a stop-at-first-failure run has
already been through every other test.
"""
import numpy as np
import pytest
import torch

import oracle
from chatokf_b200.enc import CudaEnc, GGUFTensor, OkfError
from chatokf_b200.gguf_types import GGUFType
from helpers import lcg_fill, make_weights, rel_err

pytestmark = pytest.mark.gpu

# the two entry points may cut K into a different number of ranges, so their fp32
# sums differ in rounding only; 1e-5 is the bound the narrow-vs-matvec test uses
SAME_TOL = 1e-5
ORACLE_TOL = 1e-2  # the tensor-core matmul's bound with bf16 operands (tests/test_gpu_parity.py)


def test_noalloc_matches_gemm_twice_in_a_row(ctx):
    enc = CudaEnc(ctx)
    cases = [(GGUFType.Q4_K, 4096, 200, 40), (GGUFType.IQ2_XXS, 2048, 131, 77)]
    for ty, k, m, n in cases:
        blocks = make_weights(ty, m, k, seed=n)
        w = ctx.upload(blocks)
        t = GGUFTensor("w", (k, m), ty)
        for call in range(2):  # second call: the shared array still holds the first call's partials
            X = np.stack([lcg_fill(k, 100 * call + c) for c in range(n)])
            Xd = torch.from_numpy(X).cuda().to(torch.bfloat16)
            want = torch.empty(n, m, dtype=torch.float32, device="cuda")
            enc.gemm(t, Xd, want, w, n)
            got = torch.full((n * m + 8,), float("nan"), dtype=torch.float32, device="cuda")
            enc.gemm_noalloc(t, Xd, got, w, n)
            torch.cuda.synchronize()
            g = got.cpu().numpy()
            assert np.isnan(g[n * m:]).all(), "wrote past the N * M outputs"
            assert rel_err(g[:n * m].reshape(n, m), want.cpu().numpy()) <= SAME_TOL, (ty, call)
            # and, since both run the same tile kernel, against the CPU oracle as well
            ref = oracle.matmul(ty, blocks, k, m, Xd.float().cpu().numpy(), n)
            assert rel_err(g[:n * m].reshape(n, m), ref) <= ORACLE_TOL, (ty, call)
    assert ctx.device_status() == 0


def test_noalloc_rejects_what_does_not_fit(ctx):
    enc = CudaEnc(ctx)
    ty, k = GGUFType.Q4_K, 256
    m, n = 4096, 520  # N * M = 2 129 920 outputs: just above the 2 Mi the fixed array can serve
    w = ctx.upload(make_weights(ty, m, k, seed=1))
    X = torch.zeros(n, k, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(n, m, dtype=torch.float32, device="cuda")
    with pytest.raises(OkfError) as e:
        enc.gemm_noalloc(GGUFTensor("w", (k, m), ty), X, out, w, n)
    assert e.value.status == -9  # OKF_E_LIMIT
    with pytest.raises(OkfError) as e:  # a single 64-wide k-block leaves nothing to split
        enc.gemm_noalloc(GGUFTensor("w", (64, m), GGUFType.Q8_0), X[:, :64].contiguous(), out, w, 16)
    assert e.value.status == -3  # OKF_E_SHAPE
    enc.gemm(GGUFTensor("w", (k, m), ty), X, out, w, n)  # the ordinary entry point still takes it
    torch.cuda.synchronize()
