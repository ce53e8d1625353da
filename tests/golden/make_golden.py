#!/usr/bin/env python3
"""Generate the committed known-answer fixtures in this directory.

    python tests/golden/make_golden.py

For Q8_0, Q4_K, IQ2_XXS, Q4_0, IQ4_NL, Q5_K and Q6_K the expected dequantised values come from gguf-py's
`gguf.quants.dequantize` (ggml's arithmetic, the yardstick the reference's own
codec tests use: LLM/LLMTests/IQ1CodecTests.swift:15-102).  Q2_0 is a PrismML
type gguf-py does not know; its expectation is a NumPy restatement of
Q2_0.dequant (LLM/Base/Quant.swift:10-25) written independently of the C oracle.

Expected dot products are computed with NumPy float32 scalars in the order of
the reference's CPU engine: per block a sequential fp32 sum, block partials
added sequentially (LLM/Gemma/Gemma4Quant.swift:115-136, :250-279;
LLM/Base/Quant.swift:28-65).  They use the dequantised values above, so they do
not depend on the C oracle either.

Needs: numpy, gguf (gguf-py 0.19.0).  Output: one small .npz per type.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from gguf import GGMLQuantizationType as QT  # noqa: E402
from gguf import quants  # noqa: E402

from chatokf_b200 import synth  # noqa: E402
from chatokf_b200.gguf_types import GGUFType, block_bytes, block_elems  # noqa: E402

f32 = np.float32


def f16_bytes(v):
    return np.array([v], dtype=np.float16).view(np.uint8)


def edge_blocks(ty, rng):
    """Blocks a fitted encoder never emits: zero / subnormal / largest / negative
    scales, all-zero and all-ones payloads, extreme sub-scales."""
    bb = block_bytes(ty)
    out = []
    for d in (0.0, -0.0, 5.96e-8, -6.1e-5, 65504.0, -65504.0, 1.0, 0.0123):
        for fill in (0x00, 0xFF, 0x55, 0xAA, None):
            b = np.full(bb, 0 if fill is None else fill, dtype=np.uint8)
            if fill is None:
                b[:] = rng.integers(0, 256, size=bb, dtype=np.uint8)
            at = 208 if ty == GGUFType.Q6_K else 0
            b[at:at + 2] = f16_bytes(d)
            if ty in (GGUFType.Q4_K, GGUFType.Q5_K):
                b[2:4] = f16_bytes(abs(d) * 0.5 if fill != 0xAA else 65504.0)
            out.append(b)
    if ty == GGUFType.IQ2_XXS:  # sub-scale nibble 0 and 15 in every sub-block
        for nib in (0, 15):
            b = rng.integers(0, 256, size=bb, dtype=np.uint8)
            b[0:2] = f16_bytes(0.037)
            w = b[2:].view("<u4").copy()
            w[1::2] = (w[1::2] & 0x0FFFFFFF) | (nib << 28)
            b[2:] = w.view(np.uint8)
            out.append(b)
    if ty == GGUFType.Q6_K:  # int8 sub-scales at their extremes
        for fill in (0x00, 0x7F, 0x80, 0xFF):
            b = rng.integers(0, 256, size=bb, dtype=np.uint8)
            b[208:210] = f16_bytes(0.011)
            b[192:208] = fill
            out.append(b)
    if ty in (GGUFType.Q4_K, GGUFType.Q5_K):  # all sixteen scale bytes at their extremes
        for fill in (0x00, 0xFF, 0x3F, 0xC0):
            b = rng.integers(0, 256, size=bb, dtype=np.uint8)
            b[0:2] = f16_bytes(0.011)
            b[2:4] = f16_bytes(0.007)
            b[4:16] = fill
            out.append(b)
    return np.concatenate(out)


def q2_0_dequant_numpy(blocks):
    b = blocks.reshape(-1, 34)
    d = b[:, 0:2].copy().view(np.float16).astype(f32)  # [nb, 1]
    qs = b[:, 2:]
    j = np.arange(128)
    codes = (qs[:, j >> 2] >> ((j & 3) << 1).astype(np.uint8)) & 3
    return ((codes.astype(np.int32) - 1).astype(f32) * d).reshape(-1)


def expected_dequant(ty, blocks):
    if ty == GGUFType.Q2_0:
        return q2_0_dequant_numpy(blocks)
    qt = {GGUFType.Q8_0: QT.Q8_0, GGUFType.Q4_K: QT.Q4_K, GGUFType.IQ2_XXS: QT.IQ2_XXS, GGUFType.Q4_0: QT.Q4_0,
          GGUFType.IQ4_NL: QT.IQ4_NL, GGUFType.Q5_K: QT.Q5_K, GGUFType.Q6_K: QT.Q6_K}[ty]
    return quants.dequantize(blocks.reshape(1, -1), qt).reshape(-1).astype(f32)


def ref_matvec(ty, blocks, deq, k, m, x):
    """Reference accumulation order with float32 scalars."""
    per, bb = block_elems(ty), block_bytes(ty)
    nblk = k // per
    rows = blocks.reshape(m, nblk, bb)
    w = deq.reshape(m, nblk, per)
    y = np.zeros(m, dtype=f32)
    for r in range(m):
        acc = f32(0)
        for b in range(nblk):
            xs = x[b * per:(b + 1) * per]
            if ty == GGUFType.Q8_0:  # integer-valued dot, then * d
                d = rows[r, b, 0:2].copy().view(np.float16).astype(f32)[0]
                q = rows[r, b, 2:].view(np.int8).astype(f32)
                a = f32(0)
                for j in range(32):
                    a = f32(a + f32(q[j] * xs[j]))
                part = f32(a * d)
            elif ty in (GGUFType.Q4_0, GGUFType.IQ4_NL):  # low / high nibble products in turn, then * d
                d = rows[r, b, 0:2].copy().view(np.float16).astype(f32)[0]
                qs = rows[r, b, 2:]
                val = (lambda n: f32(float(n) - 8.0)) if ty == GGUFType.Q4_0 else (lambda n: synth.IQ4_NL_VALUES[n])
                a = f32(0)
                for j in range(16):
                    a = f32(a + f32(val(int(qs[j]) & 15) * xs[j]))
                    a = f32(a + f32(val(int(qs[j]) >> 4) * xs[j + 16]))
                part = f32(a * d)
            elif ty == GGUFType.Q2_0:  # d * (lo + 2*hi - sum)
                d = rows[r, b, 0:2].copy().view(np.float16).astype(f32)[0]
                qs = rows[r, b, 2:]
                lo = hi = sy = f32(0)
                for j in range(128):
                    code = (int(qs[j >> 2]) >> ((j & 3) << 1)) & 3
                    sy = f32(sy + xs[j])
                    if code & 1:
                        lo = f32(lo + xs[j])
                    if code & 2:
                        hi = f32(hi + xs[j])
                part = f32(d * f32(f32(lo + f32(f32(2) * hi)) - sy))
            else:  # decode, then a sequential 256-long dot
                a = f32(0)
                for j in range(256):
                    a = f32(a + f32(w[r, b, j] * xs[j]))
                part = a
            acc = f32(acc + part)
        y[r] = acc
    return y


def main():
    for ty in (GGUFType.Q8_0, GGUFType.Q4_K, GGUFType.IQ2_XXS, GGUFType.Q2_0, GGUFType.Q4_0, GGUFType.IQ4_NL,
               GGUFType.Q5_K, GGUFType.Q6_K):
        rng = np.random.default_rng(1000 + int(ty))
        per = block_elems(ty)
        k, m = 4 * 256, 6
        if ty == GGUFType.Q2_0:
            fitted = synth.ternary_q2_0(rng, k * m)
        else:
            fitted = synth.quantize(ty, rng.normal(0, 0.02, size=(m, k)).astype(f32))
        x = rng.normal(0, 1, size=k).astype(f32)
        deq = expected_dequant(ty, fitted)
        y = ref_matvec(ty, fitted, deq, k, m, x)
        edge = np.concatenate([edge_blocks(ty, rng), synth.random_blocks(ty, 24, rng)])
        edge_deq = expected_dequant(ty, edge)
        assert np.isfinite(edge_deq).all()
        name = HERE / f"{ty.name.lower()}.npz"
        np.savez_compressed(
            name, type=np.int32(ty), k=np.int32(k), m=np.int32(m), blocks=fitted,
            dequant_bits=deq.view(np.uint32), x=x, matvec=y,
            edge_blocks=edge, edge_dequant_bits=edge_deq.view(np.uint32))
        print(f"{name.name}: {fitted.size} + {edge.size} block bytes, per={per}")


if __name__ == "__main__":
    main()
