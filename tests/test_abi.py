"""The C-ABI library loads and exports what include/okf_cuda.h declares (CPU only:
nothing here launches a kernel)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "okf_cuda.h"


def declared():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"OKF_API[^;]*?\b(okf_\w+)\s*\(", text)))


def test_header_declares_the_operator_entry_points():
    names = declared()
    for need in ("okf_init", "okf_destroy", "okf_weights_upload", "okf_gemv", "okf_gemm",
                 "okf_gemm_tile", "okf_dequant", "okf_matvec_host", "okf_matmul_host", "okf_strerror"):
        assert need in names


def test_library_exports_every_declared_symbol(lib_built):
    from chatokf_b200 import _lib

    L = ctypes.CDLL(str(lib_built))
    for name in declared():
        assert hasattr(L, name), f"{name} declared in okf_cuda.h but not exported"
    assert sorted(_lib.SIGNATURES) == declared()


def test_header_compiles_as_c11(tmp_path):
    import subprocess

    src = tmp_path / "t.c"
    src.write_text('#include "okf_cuda.h"\nint main(void){return okf_row_bytes(OKF_Q4_K, 256) == 144 ? 0 : 1;}\n')
    subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Werror", "-I", str(HEADER.parent), "-c", str(src),
                           "-o", str(tmp_path / "t.o")])


def test_pure_host_entry_points(lib_built):
    from chatokf_b200 import _lib
    from chatokf_b200.gguf_types import GGUFType, row_byte_count

    L = _lib.load()
    for ty in GGUFType:
        for k in (256, 2048, 5120, 17408):
            assert L.okf_row_bytes(int(ty), k) == row_byte_count(ty, k)
    assert L.okf_row_bytes(3, 256) == 0
    assert b"block size" in L.okf_strerror(-3)
    assert L.okf_launch_count(None) == 0


def test_missing_library_is_loud(monkeypatch, tmp_path):
    from chatokf_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libokfcuda.so")
    with pytest.raises(ImportError):
        _lib.load()
