"""ctypes binding of libokfcuda.so (the C ABI in include/okf_cuda.h).

There is no other compute path: if the shared library is missing or does not
load, importing anything that needs it raises.  The library is looked for
beside this file only, so a stale copy elsewhere is never picked up.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libokfcuda.so"

OKF_OK = 0
STATUS = {
    0: "OKF_OK", -1: "OKF_E_ARG", -2: "OKF_E_TYPE", -3: "OKF_E_SHAPE", -4: "OKF_E_RANGE",
    -5: "OKF_E_ALIGN", -6: "OKF_E_CUDA", -7: "OKF_E_NOMEM", -8: "OKF_E_INJECTED", -9: "OKF_E_LIMIT",
    -10: "OKF_E_FORMAT", -11: "OKF_E_IO",
}

# every symbol include/okf_cuda.h declares: name -> (restype, argtypes)
_vp, _sz, _u64, _u32, _ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int
_pp = ctypes.POINTER(ctypes.c_void_p)
SIGNATURES = {
    "okf_strerror": (ctypes.c_char_p, [_ci]),
    "okf_init": (_ci, [_ci, _pp]),
    "okf_destroy": (None, [_vp]),
    "okf_last_cuda_error": (_ci, [_vp]),
    "okf_ctx_stream": (_vp, [_vp]),
    "okf_sync": (_ci, [_vp]),
    "okf_weights_upload": (_ci, [_vp, _vp, _sz, _pp]),
    "okf_weights_wrap": (_ci, [_vp, _vp, _sz, _pp]),
    "okf_weights_free": (None, [_vp, _vp]),
    "okf_weights_device_ptr": (_vp, [_vp]),
    "okf_weights_bytes": (_sz, [_vp]),
    "okf_row_bytes": (_sz, [_ci, _sz]),
    "okf_gemv": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _ci, _vp, _vp]),
    "okf_gemm": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _ci, _u32, _vp, _ci, _vp]),
    "okf_parallel_begin": (_ci, [_vp]),
    "okf_parallel_end": (_ci, [_vp]),
    "okf_gemm_tile": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _ci, _u32, _vp, _ci, _vp]),
    "okf_gemm_noalloc": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _ci, _u32, _vp, _ci, _vp]),
    "okf_dequant": (_ci, [_vp, _ci, _vp, _u64, _u64, _vp, _vp]),
    "okf_matvec_host": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _vp]),
    "okf_matmul_host": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _u32, _vp]),
    "okf_dequant_host": (_ci, [_vp, _ci, _vp, _u64, _u64, _vp]),
    "okf_fault_inject": (_ci, [_vp, ctypes.c_double, _u64]),
    "okf_device_status": (_ci, [_vp, ctypes.POINTER(ctypes.c_int)]),
    "okf_set_flags": (_ci, [_vp, _u32]),
    "okf_launch_count": (_u64, [_vp]),
    "okf_fallback_count": (_u64, [_vp]),
}



class IpcHandle(ctypes.Structure):
    """okf_ipc_handle"""
    _fields_ = [("bytes", ctypes.c_ubyte * 64)]


class Gather(ctypes.Structure):
    """okf_gather"""
    _fields_ = [("nranks", _u32), ("rank", _u32), ("m_total", _u32), ("row_first", _u32),
                ("out", _vp * 8), ("arrivals", _vp * 8), ("epoch", _vp), ("flags", _u32)]


SIGNATURES.update({
    "okf_shared_alloc": (_ci, [_vp, _sz, _pp, ctypes.POINTER(IpcHandle)]),
    "okf_shared_open": (_ci, [_vp, ctypes.POINTER(IpcHandle), _pp]),
    "okf_shared_close": (_ci, [_vp, _vp]),
    "okf_shared_free": (_ci, [_vp, _vp]),
    "okf_copy_to_host": (_ci, [_vp, _vp, _vp, _sz]),
    "okf_gemm_gather": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _ci, _u32, ctypes.POINTER(Gather), _vp]),
    "okf_gather_wait": (_ci, [_vp, _vp]),
})

class SrqSide(ctypes.Structure):
    """okf_srq_side"""
    _fields_ = [("scale", ctypes.c_float), ("lo", ctypes.c_float), ("hi", ctypes.c_float)]


class GGUFTensorInfo(ctypes.Structure):
    """okf_gguf_tensor"""
    _fields_ = [("name", ctypes.c_char_p), ("n_dims", _u32), ("dims", _u64 * 4), ("type", ctypes.c_int32),
                ("offset", _u64), ("bytes", _u64), ("host", _vp)]


_cs, _pu64 = ctypes.c_char_p, ctypes.POINTER(_u64)
SIGNATURES.update({
    "okf_gguf_open": (_ci, [_cs, _pp]),
    "okf_gguf_close": (None, [_vp]),
    "okf_gguf_version": (_u32, [_vp]),
    "okf_gguf_tensor_count": (_u64, [_vp]),
    "okf_gguf_tensor_at": (_ci, [_vp, _u64, ctypes.POINTER(GGUFTensorInfo)]),
    "okf_gguf_find": (_ci, [_vp, _cs, ctypes.POINTER(GGUFTensorInfo)]),
    "okf_gguf_data_offset": (_u64, [_vp]),
    "okf_gguf_data_bytes": (_u64, [_vp]),
    "okf_gguf_meta_count": (_u64, [_vp]),
    "okf_gguf_meta_key": (_cs, [_vp, _u64]),
    "okf_gguf_meta_kind": (_ci, [_vp, _cs]),
    "okf_gguf_meta_int": (_ci, [_vp, _cs, ctypes.POINTER(ctypes.c_int64)]),
    "okf_gguf_meta_double": (_ci, [_vp, _cs, ctypes.POINTER(ctypes.c_double)]),
    "okf_gguf_meta_string": (_ci, [_vp, _cs, _pp, _pu64]),
    "okf_gguf_meta_array": (_ci, [_vp, _cs, _pu64, _pp, _pp]),
    "okf_gguf_meta_string_at": (_ci, [_vp, _cs, _u64, _pp, _pu64]),
    "okf_gguf_upload": (_ci, [_vp, _vp, _pp]),
})

_f = ctypes.c_float
SIGNATURES.update({
    "okf_embed_batch": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _u32, _vp, _vp]),
    "okf_argmax_rows": (_ci, [_vp, _vp, _u32, _u32, _vp, _vp]),
    "okf_add_rmsnorm": (_ci, [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _f, _u32, _u32, _vp]),
    "okf_silu_mul": (_ci, [_vp, _vp, _vp, _sz, _vp]),
    "okf_srq": (_ci, [_vp, _vp, _vp, _sz, ctypes.POINTER(SrqSide), _vp]),
    "okf_linear": (_ci, [_vp, _ci, _vp, _u64, _u32, _u32, _vp, _u32, _vp, ctypes.POINTER(SrqSide),
                         ctypes.POINTER(SrqSide), _vp, _vp]),
})

_lib = None


class OkfError(RuntimeError):
    """A C-ABI call returned a negative okf_status."""

    def __init__(self, status: int, what: str, cuda_error: int = 0):
        self.status = status
        self.cuda_error = cuda_error
        msg = f"{what}: {STATUS.get(status, status)}"
        try:
            msg += f" ({load().okf_strerror(status).decode()})"
        except Exception:
            pass
        if cuda_error:
            msg += f" [cudaError {cuda_error}]"
        super().__init__(msg)


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m chatokf_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError here = header and library out of step
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib
