"""ctypes binding of the C oracle in okf_oracle.c (test infrastructure).

Each call cites the reference routine its C twin restates; see okf_oracle.c.
"""
import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libokf_oracle.so"

# ggml type ids, LLM/Base/GGUF.swift:3-14
Q8_0, Q4_K, IQ2_XXS, Q2_0 = 8, 12, 16, 42
Q4_0, Q5_K, Q6_K, IQ4_NL = 2, 13, 14, 20
TYPES = {"q8_0": Q8_0, "q4_k": Q4_K, "iq2_xxs": IQ2_XXS, "q2_0": Q2_0,
         "q4_0": Q4_0, "q5_k": Q5_K, "q6_k": Q6_K, "iq4_nl": IQ4_NL}

_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "okf_oracle.c"
    tab = HERE.parent / "chatokf_b200" / "csrc" / "iq2xxs_tables.h"
    stale = (not LIB.exists()) or LIB.stat().st_mtime < max(src.stat().st_mtime, tab.stat().st_mtime)
    if force or stale:
        subprocess.check_call(["make", "-s", "-B", "-C", str(HERE), "libokf_oracle.so"])
    return LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(LIB))
        sz, vp, ci = ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int
        L.okf_ref_block_elems.argtypes = [ci]
        L.okf_ref_block_bytes.argtypes = [ci]
        L.okf_ref_row_bytes.argtypes = [ci, sz]
        L.okf_ref_row_bytes.restype = sz
        L.okf_ref_dequant.argtypes = [ci, vp, sz, vp]
        L.okf_ref_matvec.argtypes = [ci, vp, sz, sz, vp, vp, ci, ci]
        L.okf_ref_matmul.argtypes = [ci, vp, sz, sz, vp, sz, vp, ci]
        L.okf_ref_matmul_f64.argtypes = [ci, vp, sz, sz, vp, sz, vp, ci]
        cf = ctypes.c_float
        L.okf_ref_add_rmsnorm.argtypes = [vp, vp, vp, vp, sz, sz, cf, sz, sz]
        L.okf_ref_add_rmsnorm.restype = None
        L.okf_ref_silu_mul.argtypes = [vp, vp, sz]
        L.okf_ref_silu_mul.restype = None
        L.okf_ref_srq.argtypes = [vp, vp, sz, cf, cf, cf]
        L.okf_ref_srq.restype = None
        L.okf_ref_argmax_rows.argtypes = [vp, sz, sz, vp]
        L.okf_ref_argmax_rows.restype = None
        _lib = L
    return _lib


def block_elems(ty: int) -> int:
    return lib().okf_ref_block_elems(ty)


def block_bytes(ty: int) -> int:
    return lib().okf_ref_block_bytes(ty)


def row_bytes(ty: int, k: int) -> int:
    return lib().okf_ref_row_bytes(ty, k)


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def dequant(ty: int, blocks, count: int | None = None) -> np.ndarray:
    """GQ.gather / QB.dequant: `count` weights from a block boundary."""
    b = _u8(blocks)
    if count is None:
        count = b.size // block_bytes(ty) * block_elems(ty)
    out = np.empty(count, dtype=np.float32)
    if lib().okf_ref_dequant(ty, _ptr(b), count, _ptr(out)) != 0:
        raise ValueError("okf_ref_dequant: unsupported type or ragged count")
    return out


def _threads(threads):
    return threads if threads else (os.cpu_count() or 1)


def matvec(ty: int, w, k: int, m: int, x, threads: int = 0, faithful: bool = False) -> np.ndarray:
    """GQ.matvec: fp32 x[K] -> fp32 out[M]."""
    b = _u8(w)
    assert b.size >= row_bytes(ty, k) * m
    xx = np.ascontiguousarray(x, dtype=np.float32)
    assert xx.size == k
    out = np.empty(m, dtype=np.float32)
    if lib().okf_ref_matvec(ty, _ptr(b), k, m, _ptr(xx), _ptr(out), _threads(threads), int(faithful)) != 0:
        raise ValueError("okf_ref_matvec failed")
    return out


def matmul(ty: int, w, k: int, m: int, x, n: int, threads: int = 0) -> np.ndarray:
    """GQ.matmul: fp32 X[N][K] -> fp32 out[N][M]."""
    b = _u8(w)
    assert b.size >= row_bytes(ty, k) * m
    xx = np.ascontiguousarray(x, dtype=np.float32)
    assert xx.size == n * k
    out = np.empty((n, m), dtype=np.float32)
    if lib().okf_ref_matmul(ty, _ptr(b), k, m, _ptr(xx), n, _ptr(out), _threads(threads)) != 0:
        raise ValueError("okf_ref_matmul failed")
    return out


def matmul_f64(ty: int, w, k: int, m: int, x, n: int = 1, threads: int = 0) -> np.ndarray:
    """Float64 accumulation of the same products (accuracy yardstick)."""
    b = _u8(w)
    xx = np.ascontiguousarray(x, dtype=np.float32)
    assert xx.size == n * k
    out = np.empty((n, m), dtype=np.float64)
    if lib().okf_ref_matmul_f64(ty, _ptr(b), k, m, _ptr(xx), n, _ptr(out), _threads(threads)) != 0:
        raise ValueError("okf_ref_matmul_f64 failed")
    return out


def add_rmsnorm(x, r, w, eps: float):
    """x += r (r may be None), y = rmsnorm(x) * w per row; returns (x after the add, y)."""
    x = np.array(x, dtype=np.float32, copy=True, ndmin=2)
    rows, n = x.shape
    y = np.empty_like(x)
    rr = None if r is None else np.ascontiguousarray(np.asarray(r, dtype=np.float32).reshape(rows, n))
    ww = np.ascontiguousarray(w, dtype=np.float32)
    lib().okf_ref_add_rmsnorm(_ptr(x), None if rr is None else _ptr(rr), _ptr(ww), _ptr(y), n, rows, float(eps), n, n)
    return x, y


def silu_mul(a, b) -> np.ndarray:
    a = np.array(a, dtype=np.float32, copy=True).reshape(-1)
    bb = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
    lib().okf_ref_silu_mul(_ptr(a), _ptr(bb), a.size)
    return a


def srq(x, scale: float, lo: float, hi: float) -> np.ndarray:
    src = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    dst = np.empty_like(src)
    lib().okf_ref_srq(_ptr(src), _ptr(dst), src.size, float(scale), float(lo), float(hi))
    return dst


def argmax_rows(x) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, n = x.shape
    out = np.empty(rows, dtype=np.int32)
    lib().okf_ref_argmax_rows(_ptr(x), n, rows, _ptr(out))
    return out
