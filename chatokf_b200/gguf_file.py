"""GGUF files through the C ABI: the host-side mirror of the reference's GGUF class.

`GGUFFile(path)` maps and parses a model file (LLM/Base/GGUF.swift:92-158): `.tensors`
maps names to GGUFTensor records whose `offset` counts from the start of the data
region, `.meta` reads metadata keys (GGUF.int / .double / .string and the array
accessors, LLM/Base/GGUF.swift:190-230), and `.upload(ctx)` copies the data region to
the GPU in one piece so that the offsets are the `woff` the operator calls take.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib
from ._lib import OkfError
from .enc import GGUFTensor, Weights


class GGUFFile:
    def __init__(self, path: str):
        self.lib = _lib.load()
        h = ctypes.c_void_p()
        rc = self.lib.okf_gguf_open(str(path).encode(), ctypes.byref(h))
        if rc:
            raise OkfError(rc, f"okf_gguf_open({path})")
        self.h = h
        self.version = int(self.lib.okf_gguf_version(h))
        self.data_offset = int(self.lib.okf_gguf_data_offset(h))
        self.data_bytes = int(self.lib.okf_gguf_data_bytes(h))
        self.tensors: dict[str, GGUFTensor] = {}
        self._bytes: dict[str, int] = {}
        self._host: dict[str, int] = {}
        info = _lib.GGUFTensorInfo()
        for i in range(int(self.lib.okf_gguf_tensor_count(h))):
            rc = self.lib.okf_gguf_tensor_at(h, i, ctypes.byref(info))
            if rc:
                raise OkfError(rc, "okf_gguf_tensor_at")
            name = info.name.decode()
            dims = tuple(int(info.dims[d]) for d in range(info.n_dims))
            self.tensors[name] = GGUFTensor(name, dims, int(info.type), int(info.offset))
            self._bytes[name] = int(info.bytes)
            self._host[name] = int(info.host)

    def close(self):
        if getattr(self, "h", None):
            self.lib.okf_gguf_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def byte_count(self, name: str) -> int:
        return self._bytes[name]

    def host_bytes(self, name: str) -> np.ndarray:
        """The tensor's bytes as stored in the file (a copy)."""
        n = self._bytes[name]
        return np.ctypeslib.as_array((ctypes.c_ubyte * n).from_address(self._host[name])).copy()

    def keys(self) -> list[str]:
        return [self.lib.okf_gguf_meta_key(self.h, i).decode() for i in range(int(self.lib.okf_gguf_meta_count(self.h)))]

    def meta(self, key: str, default=None):
        """The value of a metadata key: int, float, bool, str, or a list of them."""
        k = key.encode()
        kind = self.lib.okf_gguf_meta_kind(self.h, k)
        if kind == 0:
            return default
        if kind in (1, 4):
            v = ctypes.c_int64()
            self._check(self.lib.okf_gguf_meta_int(self.h, k, ctypes.byref(v)), key)
            return bool(v.value) if kind == 4 else int(v.value)
        if kind == 2:
            d = ctypes.c_double()
            self._check(self.lib.okf_gguf_meta_double(self.h, k, ctypes.byref(d)), key)
            return float(d.value)
        if kind == 3:
            p, n = ctypes.c_void_p(), ctypes.c_uint64()
            self._check(self.lib.okf_gguf_meta_string(self.h, k, ctypes.byref(p), ctypes.byref(n)), key)
            return ctypes.string_at(p.value, n.value).decode("utf-8", "replace") if n.value else ""
        cnt, pi, pd = ctypes.c_uint64(), ctypes.c_void_p(), ctypes.c_void_p()
        self._check(self.lib.okf_gguf_meta_array(self.h, k, ctypes.byref(cnt), ctypes.byref(pi), ctypes.byref(pd)), key)
        if kind == 5:
            return list((ctypes.c_int64 * cnt.value).from_address(pi.value)) if cnt.value else []
        if kind == 6:
            return list((ctypes.c_double * cnt.value).from_address(pd.value)) if cnt.value else []
        out = []
        for i in range(cnt.value):
            p, n = ctypes.c_void_p(), ctypes.c_uint64()
            self._check(self.lib.okf_gguf_meta_string_at(self.h, k, i, ctypes.byref(p), ctypes.byref(n)), key)
            out.append(ctypes.string_at(p.value, n.value).decode("utf-8", "replace") if n.value else "")
        return out

    def _check(self, rc, what):
        if rc:
            raise OkfError(rc, f"gguf metadata {what}")

    def upload(self, ctx) -> Weights:
        """okf_gguf_upload: the data region as one weights buffer on ctx's device."""
        h = ctypes.c_void_p()
        ctx._check(self.lib.okf_gguf_upload(ctx.h, self.h, ctypes.byref(h)), "okf_gguf_upload")
        return Weights(ctx, h, self.data_bytes, None)
