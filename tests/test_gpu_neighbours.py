"""The linears' neighbours on the GPU against the CPU oracle: embedding-row gather,
arg-max over logits rows, residual add + RMS norm, SiLU gating, the clamp around
gemma's linears.  Integer / byte / index work is bit-exact; the two reductions in
floating point have their tolerance stated where they are checked."""
import numpy as np
import pytest
import torch

import oracle
from chatokf_b200.enc import CudaEnc, GGUFTensor, OkfError
from chatokf_b200.gguf_types import GGUFType, row_byte_count
from helpers import ALL_TYPES, MORE_TYPES, lcg_fill, make_weights, rel_err

pytestmark = pytest.mark.gpu

NORM_TOL = 2e-6   # fp32 sum of squares reduced in parallel instead of one after the other
SILU_TOL = 1e-6   # expf on the device vs the host's libm


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


@pytest.mark.parametrize("ty", ALL_TYPES + MORE_TYPES)
def test_embed_batch_rows_are_bit_exact(ctx, ty):
    """MetalEnc.embedBatch (LLM/Base/MetalEnc.swift:1096-1147): N token rows of a quantized
    embedding matrix, repeated and out-of-order ids included."""
    k, rows = 1024, 50
    blocks = make_weights(ty, rows, k, seed=17)
    full = oracle.dequant(ty, blocks).reshape(rows, k)
    ids = np.array([3, 49, 0, 3, 17, 48, 1], dtype=np.int32)
    out = torch.full((ids.size * k + 8,), float("nan"), dtype=torch.float32, device="cuda")
    CudaEnc(ctx).embedBatch(dev(ids), ctx.upload(blocks), out, k, ids.size, ty, rows)
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.isnan(o[ids.size * k:]).all()
    assert np.array_equal(o[:ids.size * k].reshape(-1, k).view(np.uint32), full[ids].view(np.uint32))
    assert ctx.device_status() == 0


def test_embed_batch_inside_a_larger_buffer_and_bad_ids():
    """woff addresses the embedding matrix inside the weights buffer; an id outside the
    matrix gives a row of zeros and status 8 (its own context: the status word sticks)."""
    from chatokf_b200.enc import Context

    ctx = Context(0)
    ty, k, rows = GGUFType.Q4_K, 512, 9
    a = make_weights(ty, 4, k, seed=1)
    b = make_weights(ty, rows, k, seed=2)
    w = ctx.upload(np.concatenate([a, b]))
    full = oracle.dequant(ty, b).reshape(rows, k)
    ids = np.array([8, -1, 2, rows], dtype=np.int32)
    out = torch.full((4, k), float("nan"), dtype=torch.float32, device="cuda")
    CudaEnc(ctx).embedBatch(dev(ids), w, out, k, 4, ty, rows, weight_off=a.size)
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.array_equal(o[0], full[8]) and np.array_equal(o[2], full[2])
    assert (o[1] == 0).all() and (o[3] == 0).all()
    assert ctx.device_status() == 8
    ctx.close()


@pytest.mark.parametrize("n", [7, 1000, 151936, 248320])
def test_argmax_rows_ties_and_nans(ctx, n):
    """argmax_rows (LLM/metal/Kernels.metal:2756-2794): the draft only needs the index.  Ties
    go to the lower index; NaNs never win; rows whose length is not a multiple of four."""
    rng = np.random.default_rng(n)
    rows = 5
    x = rng.normal(size=(rows, n)).astype(np.float32)
    x[1, rng.integers(0, n, size=3)] = x[1].max() + 1      # the same maximum three times
    x[2, ::3] = np.nan
    x[3] = -np.inf
    x[4, :] = 2.5                                          # all equal: index 0
    want = oracle.argmax_rows(x)
    out = torch.full((rows + 2,), -7, dtype=torch.int32, device="cuda")
    CudaEnc(ctx).argmaxRows(dev(x), out, n, rows)
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert (o[rows:] == -7).all()
    assert np.array_equal(o[:rows], want)
    assert o[4] == 0 and o[3] == 0


@pytest.mark.parametrize("n,rows", [(2560, 1), (5120, 4), (2049, 3)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_add_rmsnorm(ctx, n, rows, with_residual):
    """add_rmsnorm_batch / rmsnorm_batch (LLM/metal/Kernels.metal:2811-2864) against
    Kernels.rmsnorm (LLM/Base/Kernels.swift:12-20); strided rows."""
    rng = np.random.default_rng(n + rows)
    xs = n + 16
    x = rng.normal(size=(rows, xs)).astype(np.float32) * 3
    r = rng.normal(size=(rows, xs)).astype(np.float32)
    w = rng.normal(1.0, 0.2, size=n).astype(np.float32)
    x_after, y_ref = oracle.add_rmsnorm(x[:, :n], r[:, :n] if with_residual else None, w, 1e-6)
    xd, rd = dev(x), dev(r)
    yd = torch.full((rows, n), float("nan"), dtype=torch.float32, device="cuda")
    CudaEnc(ctx).addRmsnormBatch(xd, rd if with_residual else None, dev(w), yd, n, rows, 1e-6, x_stride=xs)
    torch.cuda.synchronize()
    xo = xd.cpu().numpy()
    assert np.array_equal(xo[:, :n], x_after)          # the add is exact
    assert np.array_equal(xo[:, n:], x[:, n:])          # nothing past the row was touched
    assert rel_err(yd.cpu().numpy(), y_ref) <= NORM_TOL


def test_silu_mul(ctx):
    rng = np.random.default_rng(3)
    n = 9728 * 3 + 5
    a = (rng.normal(size=n) * 4).astype(np.float32)
    a[:4] = [0.0, -100.0, 100.0, -0.0]
    b = rng.normal(size=n).astype(np.float32)
    want = oracle.silu_mul(a, b)
    ad = dev(a)
    CudaEnc(ctx).siluMul(ad, dev(b), n)
    torch.cuda.synchronize()
    got = ad.cpu().numpy()
    assert np.isfinite(got).all()
    assert rel_err(got, want) <= SILU_TOL


@pytest.mark.parametrize("side", [(0.05, 0.0, 0.0), (1.0, 0.0, 0.0), (0.0, -1.5, 2.25), (0.0, 0.0, 0.0)])
def test_srq_is_bit_exact(ctx, side):
    """srq_to / srq_inplace against SRQ.apply (LLM/Gemma/Gemma4Quant.swift:413-427): round
    half to even on exact .5, saturation at -128 / 127, the plain two-sided clamp, and the
    inactive side (a copy)."""
    rng = np.random.default_rng(5)
    x = (rng.normal(size=4099) * 3).astype(np.float32)
    x[:8] = [0.5, 1.5, 2.5, -0.5, -1.5, 1e9, -1e9, 0.025]
    want = oracle.srq(x, *side)
    enc = CudaEnc(ctx)
    dst = torch.full((x.size,), float("nan"), dtype=torch.float32, device="cuda")
    xd = dev(x)
    enc.srq(xd, dst, x.size, side)
    enc.srq(xd, xd, x.size, side)  # in place
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert np.array_equal(xd.cpu().numpy().view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("ty", [GGUFType.Q4_0, GGUFType.Q8_0, GGUFType.Q4_K])
@pytest.mark.parametrize("n", [1, 3])
def test_linear_with_clamps(ctx, ty, n):
    """MetalEnc.linear (LLM/Base/MetalEnc.swift:762-794): clamp the input, multiply, clamp the
    output, against the same three steps on the CPU oracle."""
    k, m = 1024, 200
    blocks = make_weights(ty, m, k, seed=21)
    X = np.stack([lcg_fill(k, 80 + c) for c in range(n)]) * np.float32(3)
    sin, sout = (0.02, 0.0, 0.0), (0.0, -0.05, 0.04)
    xin = oracle.srq(X, *sin).reshape(n, k)
    ref = oracle.srq(oracle.matmul(ty, blocks, k, m, xin, n), *sout).reshape(n, m)
    enc = CudaEnc(ctx)
    out = torch.full((n, m), float("nan"), dtype=torch.float32, device="cuda")
    scratch = torch.empty(n * k, dtype=torch.float32, device="cuda")
    Xd = dev(X)
    enc.linear(GGUFTensor("w", (k, m), ty), Xd, out, ctx.upload(blocks), n, sin, sout, scratch)
    torch.cuda.synchronize()
    assert np.array_equal(Xd.cpu().numpy(), X)  # the shared input is left alone
    assert rel_err(out.cpu().numpy(), ref) <= 1e-4
    with enc.parallel():
        with pytest.raises(OkfError):
            enc.linear(GGUFTensor("w", (k, m), ty), Xd, out, ctx.upload(blocks), n, sin, sout, scratch)


def test_ffn_chain_gate_up_silu_down(ctx):
    """QwenEngine.ffn (LLM/Qwen/QwenEngine.swift:78-87) as the engines issue it: rmsnorm ->
    gate || up -> silu_mul -> down, every step from this library, against the oracle."""
    ty, k, ff = GGUFType.Q4_K, 1024, 2560
    rng = np.random.default_rng(9)
    wg, wu, wd = (make_weights(ty, ff, k, seed=1), make_weights(ty, ff, k, seed=2), make_weights(ty, k, ff, seed=3))
    h = rng.normal(size=k).astype(np.float32)
    nw = rng.normal(1.0, 0.1, size=k).astype(np.float32)
    _, xn = oracle.add_rmsnorm(h, None, nw, 1e-6)
    g = oracle.matvec(ty, wg, k, ff, xn[0])
    u = oracle.matvec(ty, wu, k, ff, xn[0])
    ref = oracle.matvec(ty, wd, ff, k, oracle.silu_mul(g, u))
    enc = CudaEnc(ctx)
    hd, xd = dev(h), torch.empty(k, dtype=torch.float32, device="cuda")
    gd, ud = (torch.empty(ff, dtype=torch.float32, device="cuda") for _ in range(2))
    od = torch.empty(k, dtype=torch.float32, device="cuda")
    ug, uu, ud_w = ctx.upload(wg), ctx.upload(wu), ctx.upload(wd)
    enc.addRmsnormBatch(hd, None, dev(nw), xd, k, 1, 1e-6)
    with enc.parallel():
        enc.gemv(GGUFTensor("gate", (k, ff), ty), xd, gd, ug)
        enc.gemv(GGUFTensor("up", (k, ff), ty), xd, ud, uu)
    enc.siluMul(gd, ud, ff)
    enc.gemv(GGUFTensor("down", (ff, k), ty), gd, od, ud_w)
    torch.cuda.synchronize()
    assert rel_err(od.cpu().numpy(), ref) <= 1e-3
