"""Shared helpers for the parity tests."""
from pathlib import Path

import numpy as np

from chatokf_b200 import synth
from chatokf_b200.gguf_types import GGUFType, block_elems

GOLDEN = Path(__file__).resolve().parent / "golden"
ALL_TYPES = [GGUFType.Q8_0, GGUFType.Q4_K, GGUFType.IQ2_XXS, GGUFType.Q2_0]
# the rest of the decoder table: same entry points, plain kernels
MORE_TYPES = [GGUFType.Q4_0, GGUFType.IQ4_NL, GGUFType.Q5_K, GGUFType.Q6_K]


def golden(ty):
    return np.load(GOLDEN / f"{GGUFType(ty).name.lower()}.npz")


def make_weights(ty, m, k, seed):
    """Seeded N(0, 0.02) weights encoded as blocks of `ty` (ternary for Q2_0)."""
    rng = np.random.default_rng(seed)
    if ty == GGUFType.Q2_0:
        return synth.ternary_q2_0(rng, m * k, group=128)
    return synth.quantize(ty, rng.normal(0, 0.02, size=(m, k)).astype(np.float32))


def lcg_fill(n, seed):
    """The reference self-test's activation generator
    (LLM/Qwen/QwenMetalSelfTest.swift `fill`): a 64-bit LCG whose top 31 bits map to [-1, 0]."""
    out = np.empty(n, dtype=np.float32)
    s = (seed + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    umax = np.float32(0xFFFFFFFF)
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        bits = (s >> 33) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(bits) / umax * np.float32(2)) - np.float32(1)
    return out


def rel_err(got, ref):
    """max|got - ref| / max|ref|: the reference's own metric
    (LLM/Qwen/QwenMetalSelfTest.swift:575-580)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    mag = np.abs(ref).max()
    d = np.abs(got - ref).max()
    return d / mag if mag > 0 else d
