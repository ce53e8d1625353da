"""Host-side mirror of the reference's operator layer over the C ABI.

`CudaEnc` carries the method names and argument meaning of `MetalEnc`
(LLM/Base/MetalEnc.swift:84-93 gemv, :241-289 gemm, :326-352 gemmTile, :402-459
dequantRow); `QB` / `GQ` are the host-buffer twins of the CPU operator
(LLM/Base/Quant.swift:68-77, LLM/Gemma/Gemma4Quant.swift:89-170).  PyTorch is
used for device buffers and streams only; every computation is a call into
libokfcuda.so.
"""
from __future__ import annotations

import contextlib

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import OkfError
from .gguf_types import GGUFType, block_elems, row_byte_count

F32, F16, BF16 = 0, 1, 2
_DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}


@dataclass(frozen=True)
class GGUFTensor:
    """GGUFTensor of the reference (LLM/Base/GGUF.swift:49-57): dims[0] = K is the
    fastest axis, dims[1] = M rows; `offset` is the byte offset of the tensor in
    the weights buffer it was uploaded with (WeightRef.local)."""
    name: str
    dims: tuple
    type: int
    offset: int = 0

    @property
    def K(self) -> int:
        return int(self.dims[0])

    @property
    def M(self) -> int:
        return int(self.dims[1]) if len(self.dims) > 1 else 1

    @property
    def byte_count(self) -> int:
        return row_byte_count(self.type, self.K) * self.M


class Context:
    """okf_ctx: one per engine thread and device (MetalContext's role)."""

    def __init__(self, device: int = 0):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("chatokf_b200 needs a CUDA device; there is no CPU path")
        h = ctypes.c_void_p()
        rc = self.lib.okf_init(int(device), ctypes.byref(h))
        if rc:
            raise OkfError(rc, "okf_init")
        self.h = h
        self.device = int(device)

    def _check(self, rc: int, what: str):
        if rc:
            raise OkfError(rc, what, self.lib.okf_last_cuda_error(self.h))

    def close(self):
        if getattr(self, "h", None):
            self.lib.okf_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        self._check(self.lib.okf_sync(self.h), "okf_sync")

    @property
    def launches(self) -> int:
        return int(self.lib.okf_launch_count(self.h))

    @property
    def fallbacks(self) -> int:
        """Calls that ran on the simple kernels because a fast one declined the shape."""
        return int(self.lib.okf_fallback_count(self.h))

    def device_status(self) -> int:
        """0 unless a bounded wait inside a kernel gave up (okf_device_status)."""
        v = ctypes.c_int(0)
        self._check(self.lib.okf_device_status(self.h, ctypes.byref(v)), "okf_device_status")
        return v.value

    def set_flags(self, flags: int):
        """okf_set_flags: 1 = simple kernels only (device-side yardstick)."""
        self._check(self.lib.okf_set_flags(self.h, int(flags)), "okf_set_flags")

    def fault_inject(self, rate: float, seed: int = 0):
        """GPUGate.simulate(faultRate:seed:), LLM/Base/MetalGates.swift:101-108."""
        self._check(self.lib.okf_fault_inject(self.h, float(rate), int(seed)), "okf_fault_inject")

    def upload(self, blocks) -> "Weights":
        """Copy host GGUF bytes into one device allocation."""
        a = np.ascontiguousarray(blocks).view(np.uint8).reshape(-1)
        h = ctypes.c_void_p()
        self._check(self.lib.okf_weights_upload(self.h, a.ctypes.data, a.size, ctypes.byref(h)),
                    "okf_weights_upload")
        return Weights(self, h, a.size, None)

    def wrap(self, t: torch.Tensor, nbytes: int | None = None) -> "Weights":
        """Adopt a uint8 device tensor as a weights buffer (no copy).  The tensor
        should be at least 256 bytes longer than `nbytes`."""
        assert t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous()
        n = t.numel() if nbytes is None else int(nbytes)
        h = ctypes.c_void_p()
        self._check(self.lib.okf_weights_wrap(self.h, t.data_ptr(), n, ctypes.byref(h)), "okf_weights_wrap")
        return Weights(self, h, n, t)


class Weights:
    """okf_weights: device copy of a GGUF data region (or of one row shard)."""

    def __init__(self, ctx: Context, h, nbytes: int, keep):
        self.ctx, self.h, self.nbytes, self._keep = ctx, h, nbytes, keep

    def free(self):
        if self.h and self.ctx.h:
            self.ctx.lib.okf_weights_free(self.ctx.h, self.h)
        self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _stream_ptr(stream) -> int:
    s = torch.cuda.current_stream() if stream is None else stream
    return int(s.cuda_stream)


class CudaEnc:
    """Drop-in for MetalEnc's quantized linear operators on one stream."""

    NARROW_MAX = 8  # MetalEnc.narrowMax is 5 (MetalEnc.swift:172); widened to the verify batch of 8

    def __init__(self, ctx: Context, stream: torch.cuda.Stream | None = None):
        self.ctx, self.stream = ctx, stream

    def gemv(self, w: GGUFTensor, x: torch.Tensor, out: torch.Tensor, off: Weights,
             x_off_bytes: int = 0, out_off_bytes: int = 0):
        """MetalEnc.gemv(w, x:, out:, off:, xOffBytes:, outOffBytes:)."""
        assert out.dtype == torch.float32
        c = self.ctx
        c._check(c.lib.okf_gemv(c.h, int(w.type), off.h, w.offset, w.K, w.M,
                                x.data_ptr() + x_off_bytes, _DT[x.dtype],
                                out.data_ptr() + out_off_bytes, _stream_ptr(self.stream)), "okf_gemv")

    def _gemm(self, fn, name, w, X, out, off, N):
        c = self.ctx
        c._check(fn(c.h, int(w.type), off.h, w.offset, w.K, w.M, X.data_ptr(), _DT[X.dtype], int(N),
                    out.data_ptr(), _DT[out.dtype], _stream_ptr(self.stream)), name)

    def gemm(self, w: GGUFTensor, X: torch.Tensor, out: torch.Tensor, off: Weights, N: int):
        """MetalEnc.gemm(w, X:, out:, off:, N:): out[n*M + m]."""
        self._gemm(self.ctx.lib.okf_gemm, "okf_gemm", w, X, out, off, N)

    @contextlib.contextmanager
    def parallel(self):
        """MetalEnc.parallel { ... } (LLM/Base/MetalEnc.swift:42-47): the calls inside
        have no order among themselves; narrow matvecs of the same x leave as one launch."""
        c = self.ctx
        c._check(c.lib.okf_parallel_begin(c.h), "okf_parallel_begin")
        try:
            yield self
        finally:
            c._check(c.lib.okf_parallel_end(c.h), "okf_parallel_end")

    def gemm_gather(self, w: GGUFTensor, X: torch.Tensor, gather, off: Weights, N: int = 1):
        """okf_gemm_gather: this rank's rows of a row-sharded matrix, stored straight into
        every rank's output (`gather`: a tp.PeerOutputs slot); N <= 8.  The next gathered
        call waits for this exchange before it reads x; end a chain with gather_wait()."""
        c = self.ctx
        c._check(c.lib.okf_gemm_gather(c.h, int(w.type), off.h, w.offset, w.K, w.M, X.data_ptr(), _DT[X.dtype], int(N),
                                       ctypes.byref(gather), _stream_ptr(self.stream)), "okf_gemm_gather")

    def gather_wait(self):
        """okf_gather_wait: what follows on the stream sees the last gathered output whole."""
        c = self.ctx
        c._check(c.lib.okf_gather_wait(c.h, _stream_ptr(self.stream)), "okf_gather_wait")

    def gemmTile(self, w: GGUFTensor, X: torch.Tensor, out: torch.Tensor, off: Weights, N: int):
        """MetalEnc.gemmTile: the tensor-core tile at any N (kernel bench)."""
        self._gemm(self.ctx.lib.okf_gemm_tile, "okf_gemm_tile", w, X, out, off, N)

    def gemm_noalloc(self, w: GGUFTensor, X: torch.Tensor, out: torch.Tensor, off: Weights, N: int):
        """okf_gemm_noalloc: the matmul with its scratch in a fixed array of the library,
        for callers that may not allocate device memory (N * M <= 2 Mi outputs)."""
        self._gemm(self.ctx.lib.okf_gemm_noalloc, "okf_gemm_noalloc", w, X, out, off, N)

    def dequantRow(self, off: Weights, out: torch.Tensor, n: int, type: int,
                   weight_off: int = 0, out_off_bytes: int = 0):
        """MetalEnc.dequantRow(weightOff:, out:, n:, type:, outOffBytes:)."""
        assert out.dtype == torch.float32
        c = self.ctx
        c._check(c.lib.okf_dequant(c.h, int(type), off.h, int(weight_off), int(n),
                                   out.data_ptr() + out_off_bytes, _stream_ptr(self.stream)), "okf_dequant")


    # ---- the linears' neighbours ----------------------------------------------------

    def embedBatch(self, ids: torch.Tensor, off: Weights, out: torch.Tensor, nEmbd: int, N: int, type: int,
                   rows: int, weight_off: int = 0):
        """MetalEnc.embedBatch(ids:, weightOff:, out:, nEmbd:, N:, type:): out[n] = row ids[n],
        unpacked exactly.  `rows` is the height of the embedding matrix (ids are checked against it)."""
        assert ids.dtype == torch.int32 and out.dtype == torch.float32
        c = self.ctx
        c._check(c.lib.okf_embed_batch(c.h, int(type), off.h, int(weight_off), int(nEmbd), int(rows), ids.data_ptr(),
                                       int(N), out.data_ptr(), _stream_ptr(self.stream)), "okf_embed_batch")

    def argmaxRows(self, x: torch.Tensor, out: torch.Tensor, n: int, rows: int):
        """MetalEnc.argmaxRows(x:, out:, n:, rows:): ties to the lower index."""
        assert x.dtype == torch.float32 and out.dtype == torch.int32
        c = self.ctx
        c._check(c.lib.okf_argmax_rows(c.h, x.data_ptr(), int(n), int(rows), out.data_ptr(),
                                       _stream_ptr(self.stream)), "okf_argmax_rows")

    def addRmsnormBatch(self, x: torch.Tensor, r, weight: torch.Tensor, y: torch.Tensor, n: int, rows: int,
                        eps: float, x_stride: int | None = None, y_stride: int | None = None):
        """MetalEnc.addRmsnormBatch / rmsnormBatch (r = None): x += r; y = rmsnorm(x) * weight."""
        c = self.ctx
        c._check(c.lib.okf_add_rmsnorm(c.h, x.data_ptr(), r.data_ptr() if r is not None else None, weight.data_ptr(),
                                       y.data_ptr(), int(n), int(rows), float(eps), int(x_stride or n),
                                       int(y_stride or n), _stream_ptr(self.stream)), "okf_add_rmsnorm")

    def siluMul(self, a: torch.Tensor, b: torch.Tensor, n: int):
        """MetalEnc.siluMul: a = silu(a) * b."""
        c = self.ctx
        c._check(c.lib.okf_silu_mul(c.h, a.data_ptr(), b.data_ptr(), int(n), _stream_ptr(self.stream)), "okf_silu_mul")

    def srq(self, src: torch.Tensor, dst: torch.Tensor, n: int, side):
        """srqTo / srqInPlace: side = (scale, lo, hi) as SRQ.Side."""
        c = self.ctx
        s = _lib.SrqSide(*side)
        c._check(c.lib.okf_srq(c.h, src.data_ptr(), dst.data_ptr(), int(n), ctypes.byref(s), _stream_ptr(self.stream)),
                 "okf_srq")

    def linear(self, w: GGUFTensor, X: torch.Tensor, out: torch.Tensor, off: Weights, N: int, srq_in, srq_out,
               scratch: torch.Tensor | None):
        """MetalEnc.linear(w, X:, out:, off:, N:, srq:, scratch:): clamp -> gemm -> clamp."""
        c = self.ctx
        a, b = _lib.SrqSide(*srq_in), _lib.SrqSide(*srq_out)
        c._check(c.lib.okf_linear(c.h, int(w.type), off.h, w.offset, w.K, w.M, X.data_ptr(), int(N), out.data_ptr(),
                                  ctypes.byref(a), ctypes.byref(b), scratch.data_ptr() if scratch is not None else None,
                                  _stream_ptr(self.stream)), "okf_linear")


class QB:
    """Host-buffer operator: QB.matvec / QB.dequant (LLM/Base/Quant.swift:68-77)
    and GQ.matmul (LLM/Gemma/Gemma4Quant.swift:150-170) with numpy fp32 arrays.
    Each call moves x to the device, runs the kernel and brings the result back."""

    def __init__(self, ctx: Context):
        self.ctx = ctx

    def matvec(self, w: GGUFTensor, off: Weights, x: np.ndarray, out: np.ndarray | None = None) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        assert x.size == w.K
        if out is None:
            out = np.empty(w.M, dtype=np.float32)
        assert out.dtype == np.float32 and out.size == w.M and out.flags.c_contiguous
        c = self.ctx
        c._check(c.lib.okf_matvec_host(c.h, int(w.type), off.h, w.offset, w.K, w.M,
                                       x.ctypes.data, out.ctypes.data), "okf_matvec_host")
        return out

    def matmul(self, w: GGUFTensor, off: Weights, X: np.ndarray, N: int, out: np.ndarray | None = None) -> np.ndarray:
        X = np.ascontiguousarray(X, dtype=np.float32)
        assert X.size == N * w.K
        if out is None:
            out = np.empty((N, w.M), dtype=np.float32)
        assert out.dtype == np.float32 and out.size == N * w.M and out.flags.c_contiguous
        c = self.ctx
        c._check(c.lib.okf_matmul_host(c.h, int(w.type), off.h, w.offset, w.K, w.M,
                                       X.ctypes.data, int(N), out.ctypes.data), "okf_matmul_host")
        return out

    def matmul_at(self, w: GGUFTensor, off: Weights, x_addr: int, N: int, out_addr: int) -> None:
        """okf_matmul_host on raw host addresses (N x K floats in, N x M floats out), as a host
        that keeps its own buffers calls it: nothing is checked, converted or allocated here."""
        c = self.ctx
        rc = c.lib.okf_matmul_host(c.h, int(w.type), off.h, w.offset, w.K, w.M, x_addr, N, out_addr)
        if rc:
            c._check(rc, "okf_matmul_host")

    def dequant(self, w: GGUFTensor, off: Weights, row: int, count: int) -> np.ndarray:
        """QB.dequant(w, row:, count:, into:): `count` weights from the row start."""
        out = np.empty(count, dtype=np.float32)
        c = self.ctx
        c._check(c.lib.okf_dequant_host(c.h, int(w.type), off.h,
                                        w.offset + row * row_byte_count(w.type, w.K), int(count),
                                        out.ctypes.data), "okf_dequant_host")
        return out


GQ = QB  # both lineages route to the same engine (LLM/Base/Quant.swift:68-71)
