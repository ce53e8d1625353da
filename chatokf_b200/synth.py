"""Synthetic block encoders for the four weight types (NumPy, host side).

The reference only decodes GGUF blocks; it has no quantizer for any type, and
its benchmarks read tensors out of downloaded model files.  Tests and the bench
here need valid blocks built from seeded Gaussian weights instead, so this
module encodes them.  The encoders do not have to match ggml's choices: parity
is defined on decode and dot products of whatever bytes are produced.

Block layouts follow the reference decoders:
  Q8_0     34 B / 32 w   {f16 d; i8 q[32]}              LLM/Gemma/Gemma4Quant.swift:51-69
  Q4_K    144 B / 256 w  {f16 d; f16 dmin; u8 sc[12]; u8 qs[128]}
                                                         LLM/Quantize/KQuants.swift:86-125
  IQ2_XXS  66 B / 256 w  {f16 d; u16 qs[32]}             LLM/Quantize/IQ2XXS.swift:34-53
  Q2_0     34 B / 128 w  {f16 d; u8 qs[32]}, (code-1)*d  LLM/Base/Quant.swift:2-25
"""
from __future__ import annotations

import numpy as np

from .gguf_types import GGUFType, block_bytes, block_elems


def _f16(a) -> np.ndarray:
    return np.asarray(a, dtype=np.float32).astype(np.float16)


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """d = fp16(max|w| / 127) per 32 weights, q = round(w / d) as int8."""
    w = np.asarray(w, dtype=np.float32).reshape(-1, 32)
    d16 = _f16(np.abs(w).max(axis=1) / 127.0)
    d = d16.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d[:, None] > 0, np.rint(w / d[:, None]), 0.0)
    q = np.clip(q, -128, 127).astype(np.int8)
    out = np.empty((w.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def pack_q4k_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of KQuant.scaleMin: eight 6-bit (scale, min) pairs -> 12 bytes."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    s = np.empty(sc.shape[:-1] + (12,), dtype=np.uint8)
    s[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    s[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    s[..., 8:12] = (sc[..., 4:8] & 0xF) | ((mn[..., 4:8] & 0xF) << 4)
    return s


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """Min/max affine fit per 32-weight sub-block, 6-bit scales per super-block."""
    w = np.asarray(w, dtype=np.float32).reshape(-1, 8, 32)
    lo = np.minimum(w.min(axis=2), 0.0)
    hi = w.max(axis=2)
    scale = (hi - lo) / 15.0
    neg = -lo
    d16 = _f16(scale.max(axis=1) / 63.0)
    m16 = _f16(neg.max(axis=1) / 63.0)
    d = d16.astype(np.float32)[:, None]
    dm = m16.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d > 0, np.rint(scale / d), 0.0)
        mn = np.where(dm > 0, np.rint(neg / dm), 0.0)
    sc = np.clip(sc, 0, 63)
    mn = np.clip(mn, 0, 63)
    eff = (d * sc)[:, :, None]
    off = (dm * mn)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(eff > 0, np.rint((w + off) / eff), 0.0)
    q = np.clip(q, 0, 15).astype(np.uint8)
    nb = w.shape[0]
    out = np.empty((nb, 144), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = m16.view(np.uint8).reshape(-1, 2)
    out[:, 4:16] = pack_q4k_scales(sc, mn)
    q = q.reshape(nb, 4, 2, 32)  # group g: sub-block 2g in low nibbles, 2g+1 in high
    out[:, 16:] = (q[:, :, 0, :] | (q[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(-1)


_GRID = None


def iq2xxs_grid() -> np.ndarray:
    """The 256 x 8 magnitude grid as uint8 (values 8, 25, 43)."""
    global _GRID
    if _GRID is None:
        from gguf import quants

        quants.IQ2_XXS.init_grid()
        _GRID = np.asarray(quants.IQ2_XXS.grid, dtype=np.float32).reshape(256, 8).astype(np.uint8)
    return _GRID


def quantize_iq2_xxs(w: np.ndarray, chunk: int = 1 << 16) -> np.ndarray:
    """Nearest grid entry per group of eight, even-parity signs, 4-bit sub-scale."""
    w = np.asarray(w, dtype=np.float32).reshape(-1, 8, 4, 8)  # block, sub, group, elem
    nb = w.shape[0]
    grid = iq2xxs_grid().astype(np.float32)
    g2 = (grid * grid).sum(axis=1)
    amax = np.abs(w).reshape(nb, 8, 32).max(axis=2)
    # 0.8: let the largest magnitudes clip to 43 so typical ones land near 8..25
    want = 0.8 * amax / 43.0  # desired db per sub-block
    d16 = _f16(want.max(axis=1) / (15.5 * 0.25))
    d = d16.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        s = np.where(d > 0, np.rint(want / (d * 0.25) - 0.5), 0.0)
    s = np.clip(s, 0, 15).astype(np.uint32)
    db = d * (0.5 + s.astype(np.float32)) * 0.25
    with np.errstate(divide="ignore", invalid="ignore"):
        t = np.where(db[:, :, None, None] > 0, np.abs(w) / db[:, :, None, None], 0.0)
    t = t.reshape(-1, 8)
    idx = np.empty(t.shape[0], dtype=np.uint8)
    for a in range(0, t.shape[0], chunk):
        tt = t[a:a + chunk]
        dist = g2[None, :] - 2.0 * (tt @ grid.T)
        idx[a:a + chunk] = dist.argmin(axis=1).astype(np.uint8)
    negs = (w.reshape(-1, 8) < 0)
    odd = (negs.sum(axis=1) & 1).astype(bool)
    flip = t.argmin(axis=1)
    rows = np.nonzero(odd)[0]
    negs[rows, flip[rows]] ^= True
    bits = (negs.astype(np.uint32) << np.arange(8, dtype=np.uint32)[None, :]).sum(axis=1)
    sign7 = (bits & 127).astype(np.uint32).reshape(nb, 8, 4)
    idx = idx.astype(np.uint32).reshape(nb, 8, 4)
    a0 = idx[:, :, 0] | (idx[:, :, 1] << 8) | (idx[:, :, 2] << 16) | (idx[:, :, 3] << 24)
    a1 = sign7[:, :, 0] | (sign7[:, :, 1] << 7) | (sign7[:, :, 2] << 14) | (sign7[:, :, 3] << 21) | (s << 28)
    words = np.stack([a0, a1], axis=2).astype("<u4").reshape(nb, 16)
    out = np.empty((nb, 66), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = words.view(np.uint8).reshape(nb, 64)
    return out.reshape(-1)


def pack_q2_0(codes: np.ndarray, d: np.ndarray) -> np.ndarray:
    """codes in 0..3 (weight = code - 1), one fp16 scale per 128 weights."""
    codes = np.asarray(codes, dtype=np.uint8).reshape(-1, 32, 4)
    nb = codes.shape[0]
    d16 = _f16(d).reshape(nb)
    qs = codes[:, :, 0] | (codes[:, :, 1] << 2) | (codes[:, :, 2] << 4) | (codes[:, :, 3] << 6)
    out = np.empty((nb, 34), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = qs
    return out.reshape(-1)


def ternary_q2_0(rng: np.random.Generator, n_weights: int, group: int = 256,
                 scale_sigma: float = 0.05) -> np.ndarray:
    """Ternary weights with P(-1, 0, +1) = (1/4, 1/2, 1/4) and one |N(0, sigma)|
    scale per `group` weights, laid out as Q2_0 blocks (128 weights each).  A
    group of 256 becomes two consecutive blocks that carry the same scale."""
    assert n_weights % group == 0 and group % 128 == 0
    tern = rng.choice(np.array([0, 1, 1, 2], dtype=np.uint8), size=n_weights)
    scales = np.abs(rng.normal(0.0, scale_sigma, size=n_weights // group)).astype(np.float32)
    d = np.repeat(scales, group // 128)
    return pack_q2_0(tern, d)


IQ4_NL_VALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], dtype=np.float32)


def _pack_nibbles_16(q: np.ndarray) -> np.ndarray:
    """32 four-bit codes per block -> 16 bytes: byte j = code j | code (j + 16) << 4."""
    q = q.astype(np.uint8).reshape(-1, 2, 16)
    return q[:, 0, :] | (q[:, 1, :] << 4)


def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    """d = max|w| / 7 per 32 weights, q = round(w / d) + 8 in 0..15."""
    w = np.asarray(w, dtype=np.float32).reshape(-1, 32)
    d16 = _f16(np.abs(w).max(axis=1) / 7.0)
    d = d16.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(d > 0, np.rint(w / d), 0.0)
    q = np.clip(q + 8, 0, 15)
    out = np.empty((w.shape[0], 18), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = _pack_nibbles_16(q)
    return out.reshape(-1)


def quantize_iq4_nl(w: np.ndarray) -> np.ndarray:
    """d = max|w| / 127 per 32 weights, each weight to the nearest of the 16 codebook values."""
    w = np.asarray(w, dtype=np.float32).reshape(-1, 32)
    d16 = _f16(np.abs(w).max(axis=1) / 127.0)
    d = d16.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        t = np.where(d > 0, w / d, 0.0)
    q = np.abs(t[:, :, None] - IQ4_NL_VALUES[None, None, :]).argmin(axis=2)
    out = np.empty((w.shape[0], 18), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = _pack_nibbles_16(q)
    return out.reshape(-1)


def quantize_q5_k(w: np.ndarray) -> np.ndarray:
    """Min/max affine fit per 32-weight sub-block with five-bit codes, 6-bit scales per super-block."""
    w = np.asarray(w, dtype=np.float32).reshape(-1, 8, 32)
    lo = np.minimum(w.min(axis=2), 0.0)
    hi = w.max(axis=2)
    scale = (hi - lo) / 31.0
    neg = -lo
    d16 = _f16(scale.max(axis=1) / 63.0)
    m16 = _f16(neg.max(axis=1) / 63.0)
    d = d16.astype(np.float32)[:, None]
    dm = m16.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d > 0, np.rint(scale / d), 0.0)
        mn = np.where(dm > 0, np.rint(neg / dm), 0.0)
    sc = np.clip(sc, 0, 63)
    mn = np.clip(mn, 0, 63)
    eff = (d * sc)[:, :, None]
    off = (dm * mn)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(eff > 0, np.rint((w + off) / eff), 0.0)
    q = np.clip(q, 0, 31).astype(np.uint8)
    nb = w.shape[0]
    out = np.empty((nb, 176), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = m16.view(np.uint8).reshape(-1, 2)
    out[:, 4:16] = pack_q4k_scales(sc, mn)
    # fifth bit of sub-block j is bit j of qh[l]
    out[:, 16:48] = ((q >> 4) << np.arange(8, dtype=np.uint8)[None, :, None]).sum(axis=1).astype(np.uint8)
    nib = (q & 15).reshape(nb, 4, 2, 32)  # group g: sub-block 2g in low nibbles, 2g+1 in high
    out[:, 48:] = (nib[:, :, 0, :] | (nib[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(-1)


def quantize_q6_k(w: np.ndarray) -> np.ndarray:
    """Six-bit codes q in 0..63 (weight = d * s * (q - 32)), one int8 scale s per 16 weights."""
    w = np.asarray(w, dtype=np.float32).reshape(-1, 16, 16)  # block, scale group, element
    nb = w.shape[0]
    want = np.abs(w).max(axis=2) / 31.0  # d * s per group
    d16 = _f16(want.max(axis=1) / 127.0)
    d = d16.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        s = np.where(d > 0, np.rint(want / d), 0.0)
    s = np.clip(s, 0, 127)
    eff = (d * s)[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(eff > 0, np.rint(w / eff), 0.0)
    q = (np.clip(q, -32, 31) + 32).astype(np.uint8).reshape(nb, 2, 4, 32)  # half n, quarter r, l
    out = np.empty((nb, 210), dtype=np.uint8)
    lo = q & 15
    # ql[n*64 + l] = r0 | r2 << 4, ql[n*64 + 32 + l] = r1 | r3 << 4
    ql = np.empty((nb, 2, 64), dtype=np.uint8)
    ql[:, :, 0:32] = lo[:, :, 0, :] | (lo[:, :, 2, :] << 4)
    ql[:, :, 32:64] = lo[:, :, 1, :] | (lo[:, :, 3, :] << 4)
    out[:, 0:128] = ql.reshape(nb, 128)
    h = q >> 4
    out[:, 128:192] = (h[:, :, 0, :] | (h[:, :, 1, :] << 2) | (h[:, :, 2, :] << 4) | (h[:, :, 3, :] << 6)).reshape(nb, 64)
    # scale index n*8 + 2r + l/16 = the groups in k order
    out[:, 192:208] = s.astype(np.int8).view(np.uint8)
    out[:, 208:210] = d16.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def quantize(ty: int, w: np.ndarray) -> np.ndarray:
    """Encode fp32 weights (any shape, K fastest) as blocks of type `ty`."""
    ty = int(ty)
    w = np.asarray(w, dtype=np.float32)
    assert w.size % block_elems(ty) == 0
    if ty == GGUFType.Q8_0:
        return quantize_q8_0(w)
    if ty == GGUFType.Q4_K:
        return quantize_q4_k(w)
    if ty == GGUFType.IQ2_XXS:
        return quantize_iq2_xxs(w)
    if ty == GGUFType.Q2_0:
        # nearest ternary code at a per-block scale of mean |w| * 1.5
        ww = w.reshape(-1, 128)
        d = np.abs(ww).mean(axis=1) * 1.5
        with np.errstate(divide="ignore", invalid="ignore"):
            c = np.where(d[:, None] > 0, np.rint(ww / d[:, None]), 0.0)
        return pack_q2_0(np.clip(c, -1, 1).astype(np.int8) + 1, d)
    if ty == GGUFType.Q4_0:
        return quantize_q4_0(w)
    if ty == GGUFType.IQ4_NL:
        return quantize_iq4_nl(w)
    if ty == GGUFType.Q5_K:
        return quantize_q5_k(w)
    if ty == GGUFType.Q6_K:
        return quantize_q6_k(w)
    raise ValueError(f"no encoder for type {ty}")


def random_blocks(ty: int, n_blocks: int, rng: np.random.Generator) -> np.ndarray:
    """Uniformly random payload bytes with a finite, modest fp16 scale: every
    bit pattern of the payload is a valid block for every type here, so this
    reaches codes a fitted encoder never emits (e.g. ternary code 3)."""
    bb = block_bytes(ty)
    out = rng.integers(0, 256, size=(n_blocks, bb), dtype=np.uint8)
    d = _f16(rng.normal(0, 0.01, size=n_blocks))
    at = 208 if int(ty) == GGUFType.Q6_K else 0  # Q6_K keeps its scale at the end of the block
    out[:, at:at + 2] = d.view(np.uint8).reshape(-1, 2)
    if int(ty) in (GGUFType.Q4_K, GGUFType.Q5_K):
        out[:, 2:4] = _f16(np.abs(rng.normal(0, 0.01, size=n_blocks))).view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)
