"""The IQ2_XXS codebook header against its sources (CPU only)."""
import os
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "chatokf_b200" / "csrc" / "iq2xxs_tables.h"
# where a checkout of the reference lives, if there is one on this machine
REF = Path(os.environ.get("CHATOKF_REFERENCE", "/root/reference")) / "LLM" / "Quantize" / "IQ2Grid.swift"


def header_tables():
    text = HEADER.read_text()
    grid_txt = text[text.index("OKF_IQ2XXS_GRID_VALUES"):text.index("OKF_IQ2XXS_KSIGNS_VALUES")]
    grid = np.array([int(v, 16) for v in re.findall(r"0x([0-9a-f]{16})ULL", grid_txt)], dtype=np.uint64)
    ks_txt = text[text.index("OKF_IQ2XXS_KSIGNS_VALUES"):text.index("#ifndef __CUDACC__")]
    ks = np.array([int(v) for v in re.findall(r"\b\d+\b", ks_txt.split("\\", 1)[1])], dtype=np.uint8)
    return grid, ks


def test_header_is_what_the_generator_emits(tmp_path):
    import importlib.util

    spec = importlib.util.spec_from_file_location("gen", HEADER.with_name("gen_iq2_tables.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    out = tmp_path / "t.h"
    gen.emit(out)
    assert out.read_text() == HEADER.read_text()


def test_shapes_and_sign_rule():
    grid, ks = header_tables()
    assert grid.shape == (256,) and ks.shape == (128,)
    assert set(np.unique(grid.view(np.uint8))) == {0x08, 0x19, 0x2B}
    # the kernels compute the sign byte as i | parity(i) << 7 instead of a lookup
    for i in range(128):
        assert ks[i] == i | ((bin(i).count("1") & 1) << 7)


@pytest.mark.skipif(not REF.exists(), reason="reference tree not present")
def test_header_equals_reference_swift_tables():
    """IQ2Grid.xxs / ksigns / kmask, LLM/Quantize/IQ2Grid.swift:6-87."""
    src = REF.read_text()
    m = re.search(r"static let xxs: \[UInt64\] = \[(.*?)\]", src, re.S)
    ref_grid = np.array([int(v, 16) for v in re.findall(r"0x[0-9a-fA-F]+", m.group(1))], dtype=np.uint64)
    m = re.search(r"static let ksigns: \[UInt8\] = \[(.*?)\]", src, re.S)
    ref_ks = np.array([int(v) for v in re.findall(r"\d+", m.group(1))], dtype=np.uint8)
    m = re.search(r"static let kmask: \[UInt8\] = \[(.*?)\]", src, re.S)
    assert [int(v) for v in re.findall(r"\d+", m.group(1))] == [1 << j for j in range(8)]
    grid, ks = header_tables()
    assert np.array_equal(grid, ref_grid)
    assert np.array_equal(ks, ref_ks)
