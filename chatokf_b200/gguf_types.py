"""ggml tensor type ids and block geometry for the types this library handles.

Mirrors GGUFType and GGUF.rowByteCount of the reference
(LLM/Base/GGUF.swift:3-14, :160-188) and GQ.blockElems
(LLM/Gemma/Gemma4Quant.swift:77-87).
"""
from __future__ import annotations

import enum


class GGUFType(enum.IntEnum):
    Q4_0 = 2
    Q8_0 = 8
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    IQ2_XXS = 16
    IQ4_NL = 20
    Q2_0 = 42  # PrismML ternary, 128 weights / 34 bytes


_GEOM = {
    GGUFType.Q8_0: (32, 34),
    GGUFType.Q4_K: (256, 144),
    GGUFType.IQ2_XXS: (256, 66),
    GGUFType.Q2_0: (128, 34),
    GGUFType.Q4_0: (32, 18),
    GGUFType.IQ4_NL: (32, 18),
    GGUFType.Q5_K: (256, 176),
    GGUFType.Q6_K: (256, 210),
}


def _geom(ty: int):
    try:
        return _GEOM[GGUFType(int(ty))]
    except (ValueError, KeyError):
        raise ValueError(f"unsupported ggml type {ty}") from None


def block_elems(ty: int) -> int:
    return _geom(ty)[0]


def block_bytes(ty: int) -> int:
    return _geom(ty)[1]


def row_byte_count(ty: int, n: int) -> int:
    per, bb = _geom(ty)
    return n // per * bb
