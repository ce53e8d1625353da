"""Synthetic encoders: layouts decode to what was encoded (CPU only)."""
import numpy as np
import pytest

import oracle
from chatokf_b200 import synth
from chatokf_b200.gguf_types import GGUFType, block_bytes, block_elems
from helpers import lcg_fill


def test_q8_0_follows_the_stated_recipe():
    rng = np.random.default_rng(0)
    w = rng.normal(0, 0.02, size=(8, 2048)).astype(np.float32)
    b = synth.quantize_q8_0(w).reshape(-1, 34)
    d = b[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(-1)
    want_d = (np.abs(w.reshape(-1, 32)).max(axis=1) / 127.0).astype(np.float16).astype(np.float32)
    assert np.array_equal(d, want_d)
    q = b[:, 2:].view(np.int8)
    assert np.array_equal(q, np.clip(np.rint(w.reshape(-1, 32) / d[:, None]), -128, 127).astype(np.int8))


@pytest.mark.parametrize("ty,tol", [(GGUFType.Q8_0, 0.01), (GGUFType.Q4_K, 0.12), (GGUFType.IQ2_XXS, 0.45),
                                    (GGUFType.Q4_0, 0.15), (GGUFType.IQ4_NL, 0.12), (GGUFType.Q5_K, 0.06),
                                    (GGUFType.Q6_K, 0.04)])
def test_fitted_blocks_approximate_the_weights(ty, tol):
    rng = np.random.default_rng(1)
    w = rng.normal(0, 0.02, size=(4, 1024)).astype(np.float32)
    b = synth.quantize(ty, w)
    assert b.size == w.size // block_elems(ty) * block_bytes(ty)
    deq = oracle.dequant(ty, b)
    assert np.sqrt(((deq - w.reshape(-1)) ** 2).mean()) / 0.02 < tol


def test_q4k_scale_packing_is_the_inverse_of_scale_min():
    rng = np.random.default_rng(2)
    sc = rng.integers(0, 64, size=(50, 8))
    mn = rng.integers(0, 64, size=(50, 8))
    s = synth.pack_q4k_scales(sc, mn)
    for j in range(8):
        if j < 4:
            a, m = s[:, j] & 63, s[:, j + 4] & 63
        else:
            a = (s[:, j + 4] & 0xF) | ((s[:, j - 4] >> 6) << 4)
            m = (s[:, j + 4] >> 4) | ((s[:, j] >> 6) << 4)
        assert np.array_equal(a, sc[:, j]) and np.array_equal(m, mn[:, j])


def test_ternary_blocks():
    rng = np.random.default_rng(2)
    b = synth.ternary_q2_0(rng, 6144 * 8, group=256).reshape(-1, 34)
    d = b[:, 0:2].copy().view(np.float16)
    assert np.array_equal(d[0::2], d[1::2])  # a 256-group is two blocks with one scale
    deq = oracle.dequant(GGUFType.Q2_0, b)
    sign = np.sign(deq)
    frac = [(sign == v).mean() for v in (-1, 0, 1)]
    assert abs(frac[0] - 0.25) < 0.02 and abs(frac[1] - 0.5) < 0.02 and abs(frac[2] - 0.25) < 0.02


def test_iq2_signs_have_even_parity():
    rng = np.random.default_rng(3)
    b = synth.quantize_iq2_xxs(rng.normal(0, 0.02, size=(2, 1024)).astype(np.float32))
    deq = oracle.dequant(GGUFType.IQ2_XXS, b).reshape(-1, 8)
    assert ((deq < 0).sum(axis=1) % 2 == 0).all()


def test_lcg_fill_range():
    x = lcg_fill(1000, 21)
    # s >> 33 leaves 31 bits, so the reference's generator spans [-1, 0]
    assert x.dtype == np.float32 and x.min() >= -1 and x.max() <= 0 and abs(x.mean() + 0.5) < 0.05
