"""Parity of the CUDA path (through the C ABI) with the CPU oracle.

Integer / byte work (dequant) must be bit-exact.  Dot products follow the
tolerance the task states: max|y - ref| / max|ref| <= 1e-3 against the fp32
oracle; the tensor-core matmul, which rounds activations and weights to bf16
tiles, has its own bound (GEMM_TOL) stated below.
"""
import numpy as np
import pytest
import torch

import oracle
from chatokf_b200 import synth
from chatokf_b200.enc import BF16, F16, F32, CudaEnc, GGUFTensor, OkfError, QB
from chatokf_b200.gguf_types import GGUFType, block_bytes, block_elems, row_byte_count
from helpers import ALL_TYPES, MORE_TYPES, golden, lcg_fill, make_weights, rel_err

pytestmark = pytest.mark.gpu

GEMV_TOL = 1e-3   # stated tolerance for fp32-accumulated dot products
GEMV_TIGHT = 1e-4  # what the reference's own self-test asks of its GPU gemv (QwenMetalSelfTest.swift:580)
GEMM_TOL = 1e-2   # bf16 operands, fp32 accumulate
GEMM_TOL_F16 = 2e-3  # fp16 operands: the bound the reference sets for its own fp16 tile (QwenMetalSelfTest.swift:443-445)


def gemm_tol(xdt, odt=F32):
    """Bound for the tensor-core matmul: by operand type, plus bf16 rounding of a bf16 result."""
    return (GEMM_TOL_F16 if xdt in (F16, torch.float16) else GEMM_TOL) + (8e-3 if odt in (BF16, torch.bfloat16) else 0.0)

TORCH_DT = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16}


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


# ---- dequant: bit-exact ------------------------------------------------------

@pytest.mark.parametrize("ty", ALL_TYPES + MORE_TYPES)
def test_dequant_golden_bits(ctx, ty):
    g = golden(ty)
    enc = CudaEnc(ctx)
    for blocks, bits in ((g["blocks"], g["dequant_bits"]), (g["edge_blocks"], g["edge_dequant_bits"])):
        w = ctx.upload(blocks)
        n = blocks.size // block_bytes(ty) * block_elems(ty)
        out = torch.empty(n, dtype=torch.float32, device="cuda")
        enc.dequantRow(w, out, n, ty)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint32), bits)


@pytest.mark.parametrize("ty", ALL_TYPES + MORE_TYPES)
def test_dequant_random_blocks_bit_exact(ctx, ty):
    rng = np.random.default_rng(11)
    nblk = 100_000 if block_elems(ty) > 32 else 400_000
    blocks = synth.random_blocks(ty, nblk, rng)
    want = oracle.dequant(ty, blocks)
    got = QB(ctx).dequant(GGUFTensor("t", (nblk * block_elems(ty), 1), ty), ctx.upload(blocks), 0, want.size)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("ty", ALL_TYPES + MORE_TYPES)
def test_dequant_row_slice(ctx, ty):
    """dequantRow at a row offset inside a larger buffer (embedding-row read)."""
    k, m = 1024, 7
    blocks = make_weights(ty, m, k, seed=5)
    w = ctx.upload(blocks)
    t = GGUFTensor("emb", (k, m), ty)
    full = oracle.dequant(ty, blocks).reshape(m, k)
    for row in (0, 3, 6):
        got = QB(ctx).dequant(t, w, row, k)
        assert np.array_equal(got.view(np.uint32), full[row].view(np.uint32))


# ---- matvec ------------------------------------------------------------------

SHAPES = {
    GGUFType.Q8_0: [(2048, 2048), (96, 37), (32, 5)],
    GGUFType.Q4_K: [(2560, 512), (9728, 64), (256, 3)],
    GGUFType.IQ2_XXS: [(5120, 256), (17408, 40), (17408, 301), (256, 1)],
    GGUFType.Q2_0: [(2048, 384), (6144, 130), (9728, 50), (128, 9)],
}


@pytest.mark.parametrize("ty", ALL_TYPES)
@pytest.mark.parametrize("xdt", [F32, F16, BF16])
def test_gemv_vs_oracle(ctx, ty, xdt):
    enc = CudaEnc(ctx)
    for k, m in SHAPES[ty]:
        blocks = make_weights(ty, m, k, seed=k + m)
        x = np.random.default_rng(k).normal(size=k).astype(np.float32)
        xd = dev(x, TORCH_DT[xdt])
        xr = xd.float().cpu().numpy()  # the oracle sees exactly the rounded activations
        ref = oracle.matvec(ty, blocks, k, m, xr)
        out = torch.full((m + 8,), float("nan"), dtype=torch.float32, device="cuda")
        enc.gemv(GGUFTensor("w", (k, m), ty), xd, out, ctx.upload(blocks))
        torch.cuda.synchronize()
        o = out.cpu().numpy()
        assert np.isnan(o[m:]).all(), "wrote past the M outputs"
        assert rel_err(o[:m], ref) <= GEMV_TIGHT, (ty, k, m)


@pytest.mark.parametrize("ty", ALL_TYPES)
def test_gemv_golden_fixture(ctx, ty):
    g = golden(ty)
    k, m = int(g["k"]), int(g["m"])
    got = QB(ctx).matvec(GGUFTensor("w", (k, m), ty), ctx.upload(g["blocks"]), g["x"])
    assert rel_err(got, g["matvec"]) <= GEMV_TIGHT


def test_host_operator_with_page_locked_output(ctx):
    """QB.matmul with the result buffer in page-locked host memory: the kernel stores
    into it directly (no copy back); same values as with an ordinary array."""
    ty, k, m, n = GGUFType.Q4_K, 1024, 300, 3
    blocks = make_weights(ty, m, k, seed=8)
    w = ctx.upload(blocks)
    t = GGUFTensor("w", (k, m), ty)
    X = np.stack([lcg_fill(k, 40 + c) for c in range(n)])
    plain = QB(ctx).matmul(t, w, X, n)
    pinned = torch.full((n, m), float("nan")).pin_memory()
    got = QB(ctx).matmul(t, w, X, n, pinned.numpy())
    assert np.array_equal(got, plain)
    assert rel_err(got, oracle.matmul(ty, blocks, k, m, X, n)) <= GEMV_TIGHT


def test_gemv_reference_selftest_shape(ctx):
    """Config 1 of the benchmark: Q8_0 2048 x 2048 with the LCG activations the
    reference's self-test uses (QwenMetalSelfTest.swift:593-609)."""
    k = m = 2048
    rng = np.random.default_rng(0)
    blocks = synth.quantize_q8_0(rng.normal(0, 0.02, size=(m, k)).astype(np.float32))
    x = lcg_fill(k, 1)
    ref = oracle.matvec(GGUFType.Q8_0, blocks, k, m, x)
    got = QB(ctx).matvec(GGUFTensor("ffn_gate", (k, m), GGUFType.Q8_0), ctx.upload(blocks), x)
    assert rel_err(got, ref) <= GEMV_TIGHT


@pytest.mark.parametrize("ty", ALL_TYPES)
@pytest.mark.parametrize("n", [2, 3, 4, 5, 8])
def test_narrow_gemm_vs_gemv(ctx, ty, n):
    """The verify-batch kernel against N single matvecs
    (QwenMetalSelfTest.swift:448-495) and against the oracle."""
    k, m = SHAPES[ty][0][0], 200
    blocks = make_weights(ty, m, k, seed=n)
    w = ctx.upload(blocks)
    t = GGUFTensor("w", (k, m), ty)
    X = np.stack([lcg_fill(k, 70 + c) for c in range(n)])
    Xd = dev(X)
    enc = CudaEnc(ctx)
    out = torch.empty(n, m, dtype=torch.float32, device="cuda")
    enc.gemm(t, Xd, out, w, n)
    single = torch.empty(n, m, dtype=torch.float32, device="cuda")
    for c in range(n):
        enc.gemv(t, Xd, single, w, x_off_bytes=c * k * 4, out_off_bytes=c * m * 4)
    torch.cuda.synchronize()
    assert rel_err(out.cpu().numpy(), single.cpu().numpy()) <= 1e-5
    assert rel_err(out.cpu().numpy(), oracle.matmul(ty, blocks, k, m, X, n)) <= GEMV_TIGHT


@pytest.mark.parametrize("ty", ALL_TYPES)
@pytest.mark.parametrize("n", [1, 3])
def test_parallel_region_matches_separate_calls(ctx, ty, n):
    """Matvecs of one x inside a parallel region (the reference wraps gate || up
    and q || k || v in MetalEnc.parallel, QwenMetalEngine.swift:464-469, :691-696)
    leave as one launch and give the results of separate calls (the units of a
    tile may be dealt to other warps, so sums may differ in their last bits)."""
    k = SHAPES[ty][0][0]
    ms = [200, 96, 513]
    enc = CudaEnc(ctx)
    X = dev(np.stack([lcg_fill(k, 5 + c) for c in range(n)]))
    ws = [ctx.upload(make_weights(ty, m, k, seed=m)) for m in ms]
    ts = [GGUFTensor(f"w{m}", (k, m), ty) for m in ms]
    want = [torch.empty(n, m, dtype=torch.float32, device="cuda") for m in ms]
    got = [torch.full((n, m), float("nan"), dtype=torch.float32, device="cuda") for m in ms]
    for t, w, o in zip(ts, ws, want):
        enc.gemm(t, X, o, w, n)
    before = ctx.launches
    with enc.parallel():
        for t, w, o in zip(ts, ws, got):
            enc.gemm(t, X, o, w, n)
    assert ctx.launches - before == 1
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert rel_err(a.cpu().numpy(), b.cpu().numpy()) <= 1e-6


def test_parallel_region_mixed_calls(ctx):
    """Calls that do not fit the waiting set (another x, another type) send it off
    and still run; an unmatched end is an error."""
    enc = CudaEnc(ctx)
    k = 512
    x1 = dev(lcg_fill(k, 1)); x2 = dev(lcg_fill(k, 2))
    wa = make_weights(GGUFType.Q4_K, 64, k, seed=1); wb = make_weights(GGUFType.Q8_0, 48, k, seed=2)
    ta, tb = GGUFTensor("a", (k, 64), GGUFType.Q4_K), GGUFTensor("b", (k, 48), GGUFType.Q8_0)
    ua, ub = ctx.upload(wa), ctx.upload(wb)
    outs = [torch.empty(m, dtype=torch.float32, device="cuda") for m in (64, 64, 48)]
    with enc.parallel():
        enc.gemv(ta, x1, outs[0], ua)
        enc.gemv(ta, x2, outs[1], ua)
        enc.gemv(tb, x2, outs[2], ub)
    torch.cuda.synchronize()
    for o, (ty, blocks, m, x) in zip(outs, [(GGUFType.Q4_K, wa, 64, x1), (GGUFType.Q4_K, wa, 64, x2),
                                          (GGUFType.Q8_0, wb, 48, x2)]):
        assert rel_err(o.cpu().numpy(), oracle.matvec(ty, blocks, k, m, x.cpu().numpy())) <= GEMV_TIGHT
    with pytest.raises(OkfError):
        ctx._check(ctx.lib.okf_parallel_end(ctx.h), "okf_parallel_end")


# ---- matmul ------------------------------------------------------------------

@pytest.mark.parametrize("ty", ALL_TYPES)
@pytest.mark.parametrize("xdt,odt", [(F32, F32), (BF16, F32), (F16, F32), (BF16, BF16)])
def test_gemm_vs_oracle(ctx, ty, xdt, odt):
    """N = 33 as in the reference's tile test (QwenMetalSelfTest.swift:396-446),
    plus a ragged M and an N that is not a multiple of any tile."""
    enc = CudaEnc(ctx)
    for k, m, n in [(SHAPES[ty][0][0], 200, 33), (1024, 131, 77)]:
        blocks = make_weights(ty, m, k, seed=n)
        X = np.stack([lcg_fill(k, 10 + c) for c in range(n)])
        Xd = dev(X, TORCH_DT[xdt])
        ref = oracle.matmul(ty, blocks, k, m, Xd.float().cpu().numpy(), n)
        out = torch.full((n * m + 16,), float("nan"), dtype=TORCH_DT[odt], device="cuda")
        enc.gemm(GGUFTensor("w", (k, m), ty), Xd, out, ctx.upload(blocks), n)
        torch.cuda.synchronize()
        o = out.float().cpu().numpy()
        assert np.isnan(o[n * m:]).all()
        assert rel_err(o[:n * m].reshape(n, m), ref) <= gemm_tol(xdt, odt), (ty, k, m, n)


@pytest.mark.parametrize("m,n", [(6400, 768), (10240, 512), (9728, 500)])
def test_gemm_more_items_than_sms(ctx, m, n):
    """More (128-row slab, 256-token block) items than SMs with a few left over:
    the left-over items are cut into short runs of tokens spread over the CTAs."""
    ty, k = GGUFType.Q4_K, 256
    blocks = make_weights(ty, m, k, seed=m)
    X = np.random.default_rng(n).normal(size=(n, k)).astype(np.float32)
    Xd = dev(X, torch.bfloat16)
    ref = oracle.matmul(ty, blocks, k, m, Xd.float().cpu().numpy(), n)
    out = torch.full((n * m + 8,), float("nan"), dtype=torch.float32, device="cuda")
    CudaEnc(ctx).gemm(GGUFTensor("w", (k, m), ty), Xd, out, ctx.upload(blocks), n)
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.isnan(o[n * m:]).all()
    assert rel_err(o[:n * m].reshape(n, m), ref) <= GEMM_TOL


def test_gemm_split_k_odd_sizes(ctx):
    """A short, deep matrix makes the matmul cut K into ranges (partials in
    scratch, summed by a second kernel); M * N is odd on purpose."""
    ty, k, m, n = GGUFType.Q4_K, 8192, 131, 45
    blocks = make_weights(ty, m, k, seed=4)
    X = np.random.default_rng(5).normal(size=(n, k)).astype(np.float32)
    Xd = dev(X, torch.bfloat16)
    ref = oracle.matmul(ty, blocks, k, m, Xd.float().cpu().numpy(), n)
    for odt in (torch.float32, torch.bfloat16):
        out = torch.full((n * m + 8,), float("nan"), dtype=odt, device="cuda")
        CudaEnc(ctx).gemm(GGUFTensor("w", (k, m), ty), Xd, out, ctx.upload(blocks), n)
        torch.cuda.synchronize()
        o = out.float().cpu().numpy()
        assert np.isnan(o[n * m:]).all()
        assert rel_err(o[:n * m].reshape(n, m), ref) <= GEMM_TOL + (8e-3 if odt == torch.bfloat16 else 0)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("ty", ALL_TYPES)
def test_gemm_tile_small_n(ctx, ty):
    """gemmTile forces the tile kernel at widths the dispatcher would give to
    the narrow kernel (the reference's kernel bench does this)."""
    k, m, n = 512, 70, 3
    blocks = make_weights(ty, m, k, seed=1)
    X = np.random.default_rng(2).normal(size=(n, k)).astype(np.float32)
    out = torch.empty(n, m, dtype=torch.float32, device="cuda")
    CudaEnc(ctx).gemmTile(GGUFTensor("w", (k, m), ty), dev(X), out, ctx.upload(blocks), n)
    torch.cuda.synchronize()
    assert rel_err(out.cpu().numpy(), oracle.matmul(ty, blocks, k, m, X, n)) <= GEMM_TOL


def test_matmul_host_twin(ctx):
    ty, k, m, n = GGUFType.Q4_K, 512, 48, 12
    blocks = make_weights(ty, m, k, seed=9)
    X = np.random.default_rng(3).normal(size=(n, k)).astype(np.float32)
    got = QB(ctx).matmul(GGUFTensor("w", (k, m), ty), ctx.upload(blocks), X, n)
    assert rel_err(got, oracle.matmul(ty, blocks, k, m, X, n)) <= GEMM_TOL


# ---- linearity at full size (size-independent property) ------------------------

@pytest.mark.parametrize("ty,k,m", [(GGUFType.Q4_K, 2560, 9728), (GGUFType.Q4_K, 9728, 2560),
                                    (GGUFType.IQ2_XXS, 5120, 17408), (GGUFType.IQ2_XXS, 17408, 5120),
                                    (GGUFType.Q2_0, 2048, 6144), (GGUFType.Q8_0, 2048, 2048)])
def test_full_size_linearity_and_row_spot_checks(ctx, ty, k, m):
    """At the benchmark's full shapes: W(a*x1 + x2) == a*W x1 + W x2 within the
    tolerance, and 16 rows picked across M match the oracle run on those rows."""
    rng = np.random.default_rng(int(ty))
    blocks = synth.random_blocks(ty, m * k // block_elems(ty), rng)
    w = ctx.upload(blocks)
    t = GGUFTensor("w", (k, m), ty)
    enc = CudaEnc(ctx)
    x1 = rng.normal(size=k).astype(np.float32)
    x2 = rng.normal(size=k).astype(np.float32)
    ys = []
    for x in (x1, x2, np.float32(0.5) * x1 + x2):
        out = torch.empty(m, dtype=torch.float32, device="cuda")
        enc.gemv(t, dev(x), out, w)
        ys.append(out.cpu().numpy())
    assert rel_err(ys[2], 0.5 * ys[0] + ys[1]) <= GEMV_TOL
    rb = row_byte_count(ty, k)
    rows = np.unique(np.concatenate([[0, m - 1], rng.integers(0, m, size=14)]))
    br = blocks.reshape(m, rb)
    ref = oracle.matvec(ty, br[rows].reshape(-1), k, rows.size, x1)
    assert rel_err(ys[0][rows], ref) <= GEMV_TIGHT


# ---- offsets, errors, staged faults --------------------------------------------

def test_woff_addresses_a_tensor_inside_a_larger_buffer(ctx):
    ty, k, m = GGUFType.Q4_K, 512, 20
    a = make_weights(ty, m, k, seed=1)
    b = make_weights(ty, m, k, seed=2)
    pad = np.zeros(32, dtype=np.uint8)
    buf = np.concatenate([a, pad, b])
    w = ctx.upload(buf)
    x = np.random.default_rng(0).normal(size=k).astype(np.float32)
    got = QB(ctx).matvec(GGUFTensor("second", (k, m), ty, offset=a.size + 32), w, x)
    assert rel_err(got, oracle.matvec(ty, b, k, m, x)) <= GEMV_TIGHT


def test_fast_matvec_against_simple_kernel_on_many_shapes(ctx):
    """Seeded sweep over types, K, M, batch width and activation type: the tensor-core
    matvec against the warp-per-row kernel with exact decode (OKF_FLAG_SIMPLE_KERNELS)
    on the same device buffers.  K and M are drawn so that every shared-memory plan
    comes up: whole tiles, half tiles, row segments (aligned and not), rows that
    alias banks, several groups of tiles per CTA, one to eight columns."""
    rng = np.random.default_rng(2024)
    enc = CudaEnc(ctx)
    ks = [256, 512, 1024, 1536, 2048, 2560, 2816, 4096, 5120, 6144, 9728, 11008, 14336, 17408, 20480]
    worst = 0.0
    for case in range(48):
        ty = ALL_TYPES[case % 4]
        k = int(rng.choice(ks))
        m = int(rng.choice([1, 7, 16, 33, 250, 777, 2048, 4999, 30000 if k <= 2048 else 1500]))
        n = int(rng.choice([1, 1, 2, 3, 4, 5, 7, 8]))
        tdt = [torch.float32, torch.float16, torch.bfloat16][case % 3]
        blocks = synth.random_blocks(ty, m * k // block_elems(ty), rng)
        w = ctx.upload(blocks)
        t = GGUFTensor("w", (k, m), ty)
        X = torch.from_numpy(rng.normal(size=(n, k)).astype(np.float32)).cuda().to(tdt)
        fast = torch.full((n * m + 4,), float("nan"), dtype=torch.float32, device="cuda")
        slow = torch.empty(n * m, dtype=torch.float32, device="cuda")
        enc.gemm(t, X, fast, w, n)
        ctx.set_flags(1)
        try:
            enc.gemm(t, X, slow, w, n)
        finally:
            ctx.set_flags(0)
        torch.cuda.synchronize()
        f = fast.cpu().numpy()
        assert np.isnan(f[n * m:]).all(), (ty, k, m, n)
        err = rel_err(f[:n * m], slow.cpu().numpy())
        assert err <= GEMV_TIGHT, (int(ty), k, m, n, str(tdt), err)
        worst = max(worst, err)
    assert ctx.device_status() == 0


def test_tensor_core_matmul_against_simple_kernel_on_many_shapes(ctx):
    """Seeded sweep of the prefill matmul (N >= 9) against the fp32 register-tile kernel
    with exact decode: every work plan comes up (one or two token blocks per item,
    splits along K with the ordered reduction, token runs for left-over items),
    all activation types, fp32 and bf16 outputs, ragged M and N."""
    rng = np.random.default_rng(77)
    enc = CudaEnc(ctx)
    shapes = [(256, 19000, 300), (512, 9600, 512), (8192, 140, 64), (1024, 130, 9), (2048, 5000, 700),
              (4096, 1000, 257), (17408, 384, 96), (320, 77, 1000), (1536, 20000, 130), (6144, 2048, 512)]
    for case, (k, m, n) in enumerate(shapes * 2):
        ty = ALL_TYPES[case % 4]
        if k % block_elems(ty):
            k = k // block_elems(ty) * block_elems(ty)
        tdt = [torch.bfloat16, torch.float16, torch.float32][case % 3]
        odt = torch.bfloat16 if case % 5 == 4 else torch.float32
        blocks = synth.random_blocks(ty, m * k // block_elems(ty), rng)
        w = ctx.upload(blocks)
        t = GGUFTensor("w", (k, m), ty)
        X = torch.from_numpy(rng.normal(size=(n, k)).astype(np.float32)).cuda().to(tdt)
        fast = torch.full((n * m + 8,), float("nan"), dtype=odt, device="cuda")
        slow = torch.empty(n * m, dtype=torch.float32, device="cuda")
        enc.gemm(t, X, fast, w, n)
        ctx.set_flags(1)
        try:
            enc.gemm(t, X, slow, w, n)
        finally:
            ctx.set_flags(0)
        torch.cuda.synchronize()
        f = fast.float().cpu().numpy()
        assert np.isnan(f[n * m:]).all(), (int(ty), k, m, n)
        tol = gemm_tol(tdt, odt)
        err = rel_err(f[:n * m], slow.cpu().numpy())
        assert err <= tol, (int(ty), k, m, n, str(tdt), str(odt), err)
    assert ctx.device_status() == 0


def test_error_codes(ctx):
    ty, k, m = GGUFType.Q4_K, 512, 4
    w = ctx.upload(make_weights(ty, m, k, seed=1))
    x = torch.zeros(k, device="cuda")
    out = torch.zeros(m, device="cuda")
    enc = CudaEnc(ctx)
    with pytest.raises(OkfError) as e:
        enc.gemv(GGUFTensor("w", (k, m), 3), x, out, w)  # q4_1: no kernel
    assert e.value.status == -2
    with pytest.raises(OkfError) as e:
        enc.gemv(GGUFTensor("w", (500, m), ty), x, out, w)  # K not a multiple of 256
    assert e.value.status == -3
    with pytest.raises(OkfError) as e:
        enc.gemv(GGUFTensor("w", (k, m + 1), ty), x, out, w)  # one row too many
    assert e.value.status == -4
    with pytest.raises(OkfError) as e:
        enc.gemv(GGUFTensor("w", (k, 1), ty, offset=8), x, out, w)  # Q4_K needs 16-byte alignment
    assert e.value.status == -5
    with pytest.raises(OkfError) as e:
        enc.gemm(GGUFTensor("w", (k, m), ty), x, out, w, 0)
    assert e.value.status == -3
    enc.gemv(GGUFTensor("w", (k, m), ty), x, out, w)  # the context still works
    torch.cuda.synchronize()


def test_staged_faults_are_seeded_and_host_side(ctx):
    """GPUGate.simulate's contract (LLMTests/GPUGateTests.swift:10-43): the same
    seed fails the same calls; nothing is launched for a failed call."""
    ty, k, m = GGUFType.Q8_0, 256, 8
    w = ctx.upload(make_weights(ty, m, k, seed=1))
    t = GGUFTensor("w", (k, m), ty)
    x = torch.ones(k, device="cuda")
    out = torch.zeros(m, device="cuda")
    enc = CudaEnc(ctx)

    def run(seed):
        ctx.fault_inject(0.3, seed)
        pattern, before = [], ctx.launches
        for _ in range(40):
            try:
                enc.gemv(t, x, out, w)
                pattern.append(0)
            except OkfError as e:
                assert e.status == -8
                pattern.append(1)
        launched = ctx.launches - before
        ctx.fault_inject(0.0, 0)
        return pattern, launched

    p1, l1 = run(7)
    p2, _ = run(7)
    p3, _ = run(8)
    assert p1 == p2 and p1 != p3
    assert 0 < sum(p1) < 40 and l1 == 40 - sum(p1)
    enc.gemv(t, x, out, w)
    torch.cuda.synchronize()


# ---- activations that stress the 16-bit reduction of x ---------------------------

def _pattern_units(kind, k, rng):
    """One activation column whose 256-wide units follow an awkward pattern."""
    nu = k // 256
    x = rng.normal(size=(nu, 256)).astype(np.float32)
    if kind == "outlier_1e2":
        x[np.arange(nu), rng.integers(0, 256, nu)] *= np.float32(1e2)
    elif kind == "outlier_1e4":
        x[np.arange(nu), rng.integers(0, 256, nu)] = np.float32(1e4) * np.sign(rng.normal(size=nu)).astype(np.float32)
    elif kind == "one_hot":
        hot = rng.integers(0, 256, nu)
        x[:] = 0
        x[np.arange(nu), hot] = rng.normal(size=nu).astype(np.float32) + 3
    elif kind == "all_equal":
        x[:] = np.float32(0.7311)
    elif kind == "alternating_max":
        x[:] = np.float32(60000.0) * np.where(np.arange(256) % 2, -1, 1).astype(np.float32)
    elif kind == "f16_subnormal":
        x[:] = (rng.integers(1, 1024, size=(nu, 256)) * 2.0 ** -24).astype(np.float32) * np.sign(x)
    elif kind == "below_bit_16":
        x[:] = np.float32(1.0) + rng.integers(0, 128, size=(nu, 256)).astype(np.float32) * np.float32(2.0 ** -23)
    elif kind == "zero_unit_between_large":
        x *= np.float32(1e3)
        x[1::2] = 0
    elif kind == "f32_subnormal_unit":
        x[0] = np.float32(1e-41) * np.sign(x[0])
    elif kind == "mixed_scales":
        x *= (10.0 ** rng.integers(-6, 4, size=(nu, 1))).astype(np.float32)  # stays finite in fp16
    else:
        raise ValueError(kind)
    return x.reshape(-1)


PATTERNS = ["outlier_1e2", "outlier_1e4", "one_hot", "all_equal", "alternating_max", "f16_subnormal",
            "below_bit_16", "zero_unit_between_large", "f32_subnormal_unit", "mixed_scales"]


@pytest.mark.parametrize("ty", ALL_TYPES)
@pytest.mark.parametrize("n", [1, 4])
def test_awkward_activations_stay_within_the_stated_tolerance(ctx, ty, n):
    """The decode kernels reduce every 256-wide unit of a column of x to 16-bit integers
    with one scale.  Real residual streams are not N(0, 1): they carry outlier channels,
    one-hot and constant stretches, values near the bottom of the fp16 range.  Every such
    pattern, as fp32 / fp16 / bf16 input, must stay within the stated 1e-3 of max|y|
    against the fp32 oracle (the reference's metric, QwenMetalSelfTest.swift:575-580); the
    distance to a float64 evaluation is reported beside it."""
    k, m = 2048, 96
    blocks = make_weights(ty, m, k, seed=31)
    w = ctx.upload(blocks)
    t = GGUFTensor("w", (k, m), ty)
    enc = CudaEnc(ctx)
    rng = np.random.default_rng(1234 + int(ty) + n)
    worst, worst64 = {}, {}
    for kind in PATTERNS:
        for xdt in (F32, F16, BF16):
            if kind == "below_bit_16" and xdt != F32:
                continue  # 16-bit floats cannot hold the pattern
            if kind == "f32_subnormal_unit" and xdt == F16:
                continue
            X = np.stack([_pattern_units(kind, k, rng) for _ in range(n)])
            Xd = dev(X, TORCH_DT[xdt])
            Xr = Xd.float().cpu().numpy()
            ref = oracle.matmul(ty, blocks, k, m, Xr, n)
            ref64 = oracle.matmul_f64(ty, blocks, k, m, Xr, n)
            out = torch.full((n, m), float("nan"), dtype=torch.float32, device="cuda")
            enc.gemm(t, Xd, out, w, n)
            torch.cuda.synchronize()
            o = out.cpu().numpy()
            assert np.isfinite(o).all(), (kind, xdt)
            e, e64 = rel_err(o, ref), rel_err(o, ref64)
            worst[kind] = max(worst.get(kind, 0.0), e)
            worst64[kind] = max(worst64.get(kind, 0.0), e64)
            assert e <= GEMV_TOL, (GGUFType(ty).name, n, kind, xdt, e)
    print(f"\n{GGUFType(ty).name} n={n}: worst vs fp32 oracle / vs float64: " +
          ", ".join(f"{kd} {worst[kd]:.1e}/{worst64[kd]:.1e}" for kd in PATTERNS))
    assert ctx.device_status() == 0


# ---- the on-device yardstick itself, and the full-size prefill shapes, against the oracle ----

@pytest.mark.parametrize("ty", ALL_TYPES)
def test_simple_kernels_vs_oracle(ctx, ty):
    """The warp-per-row matvec and the fp32 register-tile matmul (OKF_FLAG_SIMPLE_KERNELS)
    are what the seeded sweeps compare the fast kernels with; here they meet the oracle
    themselves.  They decode exactly and accumulate in fp32, so the matvec bound applies."""
    enc = CudaEnc(ctx)
    ctx.set_flags(1)
    try:
        for k, m, n in [(1024, 131, 1), (1024, 131, 5), (1024, 131, 77), (2048, 200, 33)]:
            blocks = make_weights(ty, m, k, seed=k + n)
            X = np.stack([lcg_fill(k, 300 + c) for c in range(n)])
            before = ctx.launches
            out = torch.full((n * m + 4,), float("nan"), dtype=torch.float32, device="cuda")
            enc.gemm(GGUFTensor("w", (k, m), ty), dev(X), out, ctx.upload(blocks), n)
            torch.cuda.synchronize()
            assert ctx.launches == before + 1
            o = out.cpu().numpy()
            assert np.isnan(o[n * m:]).all()
            assert rel_err(o[:n * m].reshape(n, m), oracle.matmul(ty, blocks, k, m, X, n)) <= GEMV_TIGHT, (k, m, n)
    finally:
        ctx.set_flags(0)


@pytest.mark.parametrize("k,m", [(5120, 17408), (17408, 5120)])
def test_prefill_config_full_size_sampled_rows_vs_oracle(ctx, k, m):
    """The 512-token Q4_K prefill shapes at full size, bf16 activations: 32 rows picked
    across M, all 512 tokens, against the oracle run on those rows."""
    ty, n = GGUFType.Q4_K, 512
    rng = np.random.default_rng(k)
    pool = synth.quantize(ty, rng.normal(0, 0.02, size=4096 * 256).astype(np.float32)).reshape(4096, -1)
    blocks = pool[rng.integers(0, 4096, size=m * k // 256)].reshape(-1)
    X = rng.normal(size=(n, k)).astype(np.float32)
    Xd = dev(X, torch.bfloat16)
    out = torch.full((n * m + 8,), float("nan"), dtype=torch.float32, device="cuda")
    CudaEnc(ctx).gemm(GGUFTensor("w", (k, m), ty), Xd, out, ctx.upload(blocks), n)
    torch.cuda.synchronize()
    o = out.cpu().numpy()
    assert np.isnan(o[n * m:]).all()
    o = o[:n * m].reshape(n, m)
    rows = np.unique(np.concatenate([[0, 127, 128, m - 1], rng.integers(0, m, size=28)]))
    rb = row_byte_count(ty, k)
    ref = oracle.matmul(ty, blocks.reshape(m, rb)[rows].reshape(-1), k, rows.size, Xd.float().cpu().numpy(), n)
    assert rel_err(o[:, rows], ref) <= GEMM_TOL
    assert ctx.device_status() == 0


def test_host_twin_inside_a_parallel_region_returns_a_finished_result(ctx):
    """QB.matvec between okf_parallel_begin and okf_parallel_end: the narrow matvec is
    held back by the region, but the host twin promises the result on return, so it
    sends the waiting set off itself."""
    ty, k, m = GGUFType.Q4_K, 1024, 64
    blocks = make_weights(ty, m, k, seed=12)
    w = ctx.upload(blocks)
    t = GGUFTensor("w", (k, m), ty)
    x = lcg_fill(k, 3)
    enc = CudaEnc(ctx)
    fallbacks = ctx.fallbacks
    with enc.parallel():
        got = QB(ctx).matvec(t, w, x, np.full(m, np.nan, dtype=np.float32))
        assert np.isfinite(got).all()
    assert rel_err(got, oracle.matvec(ty, blocks, k, m, x)) <= GEMV_TIGHT
    assert ctx.fallbacks == fallbacks  # the tensor-core matvec took it


# ---- the rest of the decoder table (Q4_0, IQ4_NL, Q5_K, Q6_K): same entry points, plain kernels ----

@pytest.mark.parametrize("ty", MORE_TYPES)
def test_more_types_golden_matvec_and_matmul(ctx, ty):
    """The types gemma trunks and mixed K-quant files add (Blocks.decoder,
    LLM/Quantize/Blocks.swift:10-29; GQ.matvec's q4_0 / iq4_nl arms,
    LLM/Gemma/Gemma4Quant.swift:93-114): the committed fixture, then 1, 4 and 33 columns
    against the oracle.  Q4_0 has the streaming matvec and the tensor-core tile at every
    width, and so have IQ4_NL, Q5_K and Q6_K: no call here may be counted as a fallback."""
    g = golden(ty)
    k, m = int(g["k"]), int(g["m"])
    got = QB(ctx).matvec(GGUFTensor("w", (k, m), ty), ctx.upload(g["blocks"]), g["x"])
    assert rel_err(got, g["matvec"]) <= GEMV_TIGHT
    enc = CudaEnc(ctx)
    for k, m, n in [(2048, 200, 1), (1024, 131, 4), (1024, 131, 33)]:
        blocks = make_weights(ty, m, k, seed=k + n)
        X = np.stack([lcg_fill(k, 500 + c) for c in range(n)])
        for xdt in (F32, F16):
            Xd = dev(X, TORCH_DT[xdt])
            before = ctx.fallbacks
            out = torch.full((n * m + 4,), float("nan"), dtype=torch.float32, device="cuda")
            enc.gemm(GGUFTensor("w", (k, m), ty), Xd, out, ctx.upload(blocks), n)
            torch.cuda.synchronize()
            fast = True  # every type of the table has the streaming matvec and the tile
            assert ctx.fallbacks == before + (0 if fast else 1)
            o = out.cpu().numpy()
            assert np.isnan(o[n * m:]).all()
            ref = oracle.matmul(ty, blocks, k, m, Xd.float().cpu().numpy(), n)
            tol = gemm_tol(xdt, F32) if fast and n > 8 else GEMV_TIGHT
            assert rel_err(o[:n * m].reshape(n, m), ref) <= tol, (GGUFType(ty).name, k, m, n, xdt)


@pytest.mark.parametrize("ty,k", [(GGUFType.Q4_K, 9728), (GGUFType.IQ2_XXS, 17408), (GGUFType.Q8_0, 8192),
                                  (GGUFType.Q2_0, 24576)])
@pytest.mark.parametrize("n", [1, 4])
def test_long_rows_cut_into_k_chunks(ctx, ty, k, n):
    """Rows too long for a ring stage are cut into k-chunks, one stage per (tile, chunk):
    one tile, fewer tiles than SMs, more tiles than SMs; run twice; and two matrices in
    one parallel region."""
    enc = CudaEnc(ctx)
    for m in (16, 200, 1600):
        blocks = make_weights(ty, m, k, seed=m + k)
        X = np.stack([lcg_fill(k, 11 + m + c) for c in range(n)])
        ref = oracle.matmul(ty, blocks, k, m, X, n)
        w = ctx.upload(blocks)
        for rep in range(2):
            out = torch.full((n, m), float("nan"), dtype=torch.float32, device="cuda")
            enc.gemm(GGUFTensor("w", (k, m), ty), dev(X), out, w, n)
            torch.cuda.synchronize()
            assert rel_err(out.cpu().numpy(), ref) <= GEMV_TIGHT, (ty, k, m, n, rep)
    ms = [208, 1000]
    ws = [ctx.upload(make_weights(ty, m, k, seed=m)) for m in ms]
    X = np.stack([lcg_fill(k, 3 + c) for c in range(n)])
    got = [torch.full((n, m), float("nan"), dtype=torch.float32, device="cuda") for m in ms]
    with enc.parallel():
        for m, w, o in zip(ms, ws, got):
            enc.gemm(GGUFTensor(f"w{m}", (k, m), ty), dev(X), o, w, n)
    torch.cuda.synchronize()
    for m, o in zip(ms, got):
        ref = oracle.matmul(ty, make_weights(ty, m, k, seed=m), k, m, X, n)
        assert rel_err(o.cpu().numpy(), ref) <= GEMV_TIGHT, (ty, k, m, n)
    assert ctx.device_status() == 0


@pytest.mark.parametrize("xdt", [F32, F16, BF16])
def test_q4_0_streaming_matvec_and_tile(ctx, xdt):
    """Q4_0 (gemma trunks; GQ.matvec's q4_0 arm, LLM/Gemma/Gemma4Quant.swift:93-104) through the
    integer-MMA matvec at 1..8 columns and the tensor-core tile above, against the oracle;
    K short, long enough to be cut into k-chunks, and not a multiple of 256 (plain kernel)."""
    enc = CudaEnc(ctx)
    ty = GGUFType.Q4_0
    for k, m in [(256, 16), (2048, 520), (5120, 200), (9728, 333), (1056, 77)]:
        blocks = make_weights(ty, m, k, seed=k + m)
        w = ctx.upload(blocks)
        for n in (1, 2, 4, 5, 8, 40):
            X = np.stack([lcg_fill(k, 900 + k + c) for c in range(n)])
            Xd = dev(X, TORCH_DT[xdt])
            before = ctx.fallbacks
            out = torch.full((n * m + 4,), float("nan"), dtype=torch.float32, device="cuda")
            enc.gemm(GGUFTensor("w", (k, m), ty), Xd, out, w, n)
            torch.cuda.synchronize()
            o = out.cpu().numpy()
            assert np.isnan(o[n * m:]).all()
            ref = oracle.matmul(ty, blocks, k, m, Xd.float().cpu().numpy(), n)
            fast = k % 256 == 0 if n <= 8 else k % 64 == 0
            assert ctx.fallbacks == before + (0 if fast else 1), (k, m, n)
            tol = gemm_tol(xdt, F32) if n > 8 and fast else GEMV_TIGHT
            assert rel_err(o[:n * m].reshape(n, m), ref) <= tol, (k, m, n, xdt)
    assert ctx.device_status() == 0


def test_host_operator_called_again_and_again_with_the_same_buffers(ctx):
    """A decode loop calls the host-buffer operator with the same tensor and the same
    page-locked buffers for every token, only x's contents change: every call has to give
    that call's result (the copy of x and the kernel may be replayed from a recorded graph),
    the launch counter has to count every call, and more buffer sets than a cache could hold
    must still be served."""
    qb = QB(ctx)
    ty, k, m = GGUFType.Q4_K, 2048, 200
    blocks = make_weights(ty, m, k, seed=5)
    w = ctx.upload(blocks)
    t = GGUFTensor("w", (k, m), ty)
    sets = [(torch.empty(k, dtype=torch.float32).pin_memory(), torch.empty(m, dtype=torch.float32).pin_memory())
            for _ in range(11)]
    for rep in range(3):
        for i, (hx, hy) in enumerate(sets):
            x = lcg_fill(k, 40 + 7 * rep + i)
            hx.copy_(torch.from_numpy(x))
            hy.fill_(float("nan"))
            before = ctx.launches
            qb.matmul_at(t, w, hx.data_ptr(), 1, hy.data_ptr())
            assert ctx.launches == before + 1
            assert rel_err(hy.numpy(), oracle.matvec(ty, blocks, k, m, x)) <= GEMV_TIGHT, (rep, i)
    # the same buffers, other shapes and another tensor
    ty2, m2 = GGUFType.Q8_0, 64
    blocks2 = make_weights(ty2, m2, k, seed=6)
    w2 = ctx.upload(blocks2)
    hx, hy = sets[0]
    x = lcg_fill(k, 99)
    hx.copy_(torch.from_numpy(x))
    qb.matmul_at(GGUFTensor("w2", (k, m2), ty2), w2, hx.data_ptr(), 1, hy.data_ptr())
    assert rel_err(hy.numpy()[:m2], oracle.matvec(ty2, blocks2, k, m2, x)) <= GEMV_TIGHT
    assert ctx.device_status() == 0


@pytest.mark.parametrize("xdt", [F32, F16, BF16])
@pytest.mark.parametrize("ty", [GGUFType.Q6_K, GGUFType.Q5_K, GGUFType.IQ4_NL])
def test_q6_k_q5_k_iq4_nl_matvec_and_tile(ctx, ty, xdt):
    """Q6_K and Q5_K (the output projection and some FFN / attention matrices of mixed K-quant
    files; KQuant.q5K / q6K, LLM/Quantize/KQuants.swift:127-177) and IQ4_NL (gemma files;
    LLM/Gemma/Gemma4Quant.swift:5-29) through the integer-MMA matvec
    and the tensor-core tile above eight, against the oracle; Q6_K's blocks of
    210 bytes leave rows and units only 2-byte aligned; K short and long enough to be cut into
    k-chunks; one, three and forty columns."""
    enc = CudaEnc(ctx)
    for k, m in [(256, 16), (256, 37), (2560, 300), (5120, 1000), (9728, 205), (17408, 64)]:
        blocks = make_weights(ty, m, k, seed=k + m)
        w = ctx.upload(blocks)
        for n in (1, 3, 40):
            X = np.stack([lcg_fill(k, 700 + k + c) for c in range(n)])
            Xd = dev(X, TORCH_DT[xdt])
            before = ctx.fallbacks
            out = torch.full((n * m + 4,), float("nan"), dtype=torch.float32, device="cuda")
            enc.gemm(GGUFTensor("w", (k, m), ty), Xd, out, w, n)
            torch.cuda.synchronize()
            o = out.cpu().numpy()
            assert np.isnan(o[n * m:]).all()
            ref = oracle.matmul(ty, blocks, k, m, Xd.float().cpu().numpy(), n)
            assert ctx.fallbacks == before, (k, m, n)
            tol = gemm_tol(xdt, F32) if n > 8 else GEMV_TIGHT
            assert rel_err(o[:n * m].reshape(n, m), ref) <= tol, (k, m, n, xdt)
    assert ctx.device_status() == 0
