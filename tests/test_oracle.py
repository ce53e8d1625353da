"""The C oracle against the committed fixtures and against gguf-py (CPU only)."""
import numpy as np
import pytest

import oracle
from chatokf_b200 import synth
from chatokf_b200.gguf_types import GGUFType, block_bytes, block_elems, row_byte_count
from helpers import ALL_TYPES, MORE_TYPES, golden, make_weights, rel_err

ALL_TYPES = ALL_TYPES + MORE_TYPES


@pytest.mark.parametrize("ty", ALL_TYPES)
def test_geometry(ty):
    assert oracle.block_elems(ty) == block_elems(ty)
    assert oracle.block_bytes(ty) == block_bytes(ty)
    for k in (block_elems(ty), 2048, 17408 - 17408 % block_elems(ty)):
        assert oracle.row_bytes(ty, k) == row_byte_count(ty, k)


@pytest.mark.parametrize("ty", ALL_TYPES)
def test_dequant_matches_golden_bits(ty):
    g = golden(ty)
    for blocks, bits in ((g["blocks"], g["dequant_bits"]), (g["edge_blocks"], g["edge_dequant_bits"])):
        got = oracle.dequant(ty, blocks)
        assert np.array_equal(got.view(np.uint32), bits)


@pytest.mark.parametrize("ty", ALL_TYPES)
def test_matvec_matches_golden_bits(ty):
    g = golden(ty)
    k, m = int(g["k"]), int(g["m"])
    for threads in (1, 3):
        got = oracle.matvec(ty, g["blocks"], k, m, g["x"], threads=threads)
        assert np.array_equal(got.view(np.uint32), g["matvec"].view(np.uint32))
    faithful = oracle.matvec(ty, g["blocks"], k, m, g["x"], threads=2, faithful=True)
    assert np.array_equal(faithful, g["matvec"])


@pytest.mark.parametrize("ty", [GGUFType.Q8_0, GGUFType.Q4_K, GGUFType.IQ2_XXS] + MORE_TYPES)
def test_dequant_matches_gguf_py_on_random_blocks(ty):
    from gguf import GGMLQuantizationType as QT
    from gguf import quants

    qt = {GGUFType.Q8_0: QT.Q8_0, GGUFType.Q4_K: QT.Q4_K, GGUFType.IQ2_XXS: QT.IQ2_XXS, GGUFType.Q4_0: QT.Q4_0,
          GGUFType.IQ4_NL: QT.IQ4_NL, GGUFType.Q5_K: QT.Q5_K, GGUFType.Q6_K: QT.Q6_K}[ty]
    rng = np.random.default_rng(7)
    blocks = synth.random_blocks(ty, 20000, rng)
    want = quants.dequantize(blocks.reshape(1, -1), qt).reshape(-1)
    got = oracle.dequant(ty, blocks)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("ty", ALL_TYPES)
def test_matmul_is_n_matvecs(ty):
    """GQ.matmul answers most types as N matvecs (bit-equal); the Q8_0 / Q4_0
    dequant-reuse path sums in another order and only agrees closely."""
    k, m, n = 512, 9, 3
    w = make_weights(ty, m, k, seed=3)
    x = np.random.default_rng(4).normal(size=(n, k)).astype(np.float32)
    mm = oracle.matmul(ty, w, k, m, x, n)
    for c in range(n):
        mv = oracle.matvec(ty, w, k, m, x[c])
        if ty in (GGUFType.Q8_0, GGUFType.Q4_0):
            assert rel_err(mm[c], mv) < 1e-5
        else:
            assert np.array_equal(mm[c], mv)
    assert rel_err(mm, oracle.matmul_f64(ty, w, k, m, x, n)) < 1e-5


def test_ragged_and_unknown():
    with pytest.raises(ValueError):
        oracle.dequant(GGUFType.Q4_K, np.zeros(144, np.uint8), count=100)
    with pytest.raises(ValueError):
        oracle.dequant(3, np.zeros(144, np.uint8), count=256)
    assert oracle.dequant(GGUFType.Q8_0, np.zeros(0, np.uint8), count=0).size == 0


def test_neighbour_restatements_against_numpy():
    """The CPU restatements of the linears' neighbours against plain NumPy."""
    rng = np.random.default_rng(8)
    x = rng.normal(size=(3, 300)).astype(np.float32)
    r = rng.normal(size=(3, 300)).astype(np.float32)
    w = rng.normal(1, 0.1, size=300).astype(np.float32)
    xa, y = oracle.add_rmsnorm(x, r, w, 1e-6)
    assert np.array_equal(xa, x + r)
    s = x + r
    want = s / np.sqrt((s.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6) * w
    assert rel_err(y, want) < 1e-6
    a, b = x.reshape(-1), r.reshape(-1)
    assert rel_err(oracle.silu_mul(a, b), a / (1 + np.exp(-a.astype(np.float64))) * b) < 1e-6
    q = oracle.srq([0.5, 1.5, 2.5, -0.5, 300.0, -300.0, 0.26], 1.0, 0.0, 0.0)
    assert q.tolist() == [0.0, 2.0, 2.0, -0.0, 127.0, -128.0, 0.0]
    assert oracle.srq([-3.0, 0.1, 3.0], 0.0, -1.0, 2.0).tolist() == [-1.0, np.float32(0.1), 2.0]
    t = np.array([[1, 3, 3, 2], [np.nan, -1, -1, -5], [-np.inf] * 4], dtype=np.float32)
    assert oracle.argmax_rows(t).tolist() == [1, 1, 0]
