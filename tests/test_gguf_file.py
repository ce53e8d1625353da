"""The GGUF reader (C ABI, host side) against files written by gguf-py and by hand."""
import struct

import numpy as np
import pytest

import oracle
from chatokf_b200._lib import OkfError
from chatokf_b200.gguf_types import GGUFType, row_byte_count
from helpers import make_weights, rel_err


def write_with_gguf_py(path):
    from gguf import GGMLQuantizationType as QT
    from gguf import GGUFWriter

    w = GGUFWriter(str(path), "qwen35")
    w.add_uint32("qwen35.block_count", 3)
    w.add_float32("qwen35.attention.layer_norm_rms_epsilon", 1e-6)
    w.add_string("general.name", "synthetic")
    w.add_bool("tokenizer.ggml.add_bos_token", True)
    w.add_array("tokenizer.ggml.tokens", ["<s>", "hello", "", "wörld"])
    w.add_array("qwen35.rope.dimension_sections", [11, 11, 10, 0])
    w.add_array("tokenizer.ggml.scores", [0.5, -1.25])
    tensors = {}
    for name, ty, qt, k, m in [("token_embd.weight", GGUFType.Q8_0, QT.Q8_0, 512, 20),
                               ("blk.0.ffn_gate.weight", GGUFType.Q4_K, QT.Q4_K, 512, 48),
                               ("blk.0.attn_q.weight", GGUFType.IQ2_XXS, QT.IQ2_XXS, 512, 32),
                               ("blk.0.ffn_down.weight", GGUFType.Q6_K, QT.Q6_K, 768, 16),
                               ("blk.0.attn_v.weight", GGUFType.Q4_0, QT.Q4_0, 512, 8)]:
        blocks = make_weights(ty, m, k, seed=len(name))
        tensors[name] = (ty, k, m, blocks)
        w.add_tensor(name, blocks.reshape(m, row_byte_count(ty, k)), raw_dtype=qt)
    norm = np.linspace(0.5, 1.5, 512, dtype=np.float32)
    w.add_tensor("blk.0.attn_norm.weight", norm)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return tensors, norm


def test_reads_what_gguf_py_wrote(lib_built, tmp_path):
    from gguf import GGUFReader

    from chatokf_b200.gguf_file import GGUFFile

    path = tmp_path / "m.gguf"
    tensors, norm = write_with_gguf_py(path)
    with GGUFFile(path) as g:
        assert g.version == 3
        assert g.meta("qwen35.block_count") == 3
        assert abs(g.meta("qwen35.attention.layer_norm_rms_epsilon") - 1e-6) < 1e-12
        assert g.meta("general.name") == "synthetic"
        assert g.meta("tokenizer.ggml.add_bos_token") is True
        assert g.meta("tokenizer.ggml.tokens") == ["<s>", "hello", "", "wörld"]
        assert g.meta("qwen35.rope.dimension_sections") == [11, 11, 10, 0]
        assert g.meta("tokenizer.ggml.scores") == [0.5, -1.25]
        assert g.meta("no.such.key") is None and g.meta("no.such.key", 7) == 7
        assert "general.architecture" in g.keys()
        ref = GGUFReader(str(path))
        assert g.data_offset == ref.data_offset
        assert list(g.tensors) == [t.name for t in ref.tensors]
        for t in ref.tensors:
            mine = g.tensors[t.name]
            assert mine.offset == t.data_offset - ref.data_offset
            assert g.byte_count(t.name) == t.n_bytes
            assert int(mine.type) == int(t.tensor_type)
            assert list(mine.dims) == [int(d) for d in t.shape]
        for name, (ty, k, m, blocks) in tensors.items():
            t = g.tensors[name]
            assert (t.K, t.M, t.type) == (k, m, int(ty))
            assert np.array_equal(g.host_bytes(name), blocks)
        assert np.array_equal(g.host_bytes("blk.0.attn_norm.weight").view(np.float32), norm)


def hand_written(path, ty=42, alignment=64, magic=b"GGUF", truncate=None, bad_offset=False):
    """A version-3 file with one PrismML ternary tensor and general.alignment set."""
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    k, m = 256, 6
    blocks = make_weights(GGUFType.Q2_0, m, k, seed=4)
    head = magic + struct.pack("<IQQ", 3, 1, 2)
    head += s("general.alignment") + struct.pack("<II", 4, alignment)
    head += s("qwen35.some.i8") + struct.pack("<Ib", 1, -5)
    head += s("blk.0.ffn_up.weight") + struct.pack("<IQQIQ", 2, k, m, ty, 1 << 40 if bad_offset else 0)
    pad = (-len(head)) % alignment
    data = head + b"\0" * pad + blocks.tobytes()
    path.write_bytes(data if truncate is None else data[:truncate])
    return blocks, k, m, len(head) + pad


def test_prismml_type_alignment_and_errors(lib_built, tmp_path):
    from chatokf_b200.gguf_file import GGUFFile

    path = tmp_path / "t.gguf"
    blocks, k, m, start = hand_written(path)
    with GGUFFile(path) as g:
        assert g.data_offset == start and start % 64 == 0
        assert g.meta("qwen35.some.i8") == -5
        t = g.tensors["blk.0.ffn_up.weight"]
        assert (t.type, t.K, t.M, t.offset) == (42, k, m, 0)
        assert np.array_equal(g.host_bytes(t.name), blocks)
    for kwargs, status in [(dict(magic=b"GGML"), -10), (dict(truncate=40), -10), (dict(truncate=start + 10), -4),
                           (dict(ty=99), -2), (dict(bad_offset=True), -4)]:
        hand_written(path, **kwargs)
        with pytest.raises(OkfError) as e:
            GGUFFile(path)
        assert e.value.status == status, kwargs
    with pytest.raises(OkfError) as e:
        GGUFFile(tmp_path / "missing.gguf")
    assert e.value.status == -11


@pytest.mark.gpu
def test_matvec_straight_from_a_file(ctx, tmp_path):
    """Open, upload the data region once, and run the operators with the tensors' offsets,
    as the engines do with WeightRef.local: a matvec per quantized tensor, an embedding row,
    and the norm weights read as fp32 from the same buffer."""
    import torch

    from chatokf_b200.enc import CudaEnc
    from chatokf_b200.gguf_file import GGUFFile

    path = tmp_path / "m.gguf"
    tensors, norm = write_with_gguf_py(path)
    enc = CudaEnc(ctx)
    with GGUFFile(path) as g:
        w = g.upload(ctx)
        for name, (ty, k, m, blocks) in tensors.items():
            t = g.tensors[name]
            x = np.random.default_rng(k + m).normal(size=k).astype(np.float32)
            out = torch.empty(m, dtype=torch.float32, device="cuda")
            enc.gemv(t, torch.from_numpy(x).cuda(), out, w)
            torch.cuda.synchronize()
            assert rel_err(out.cpu().numpy(), oracle.matvec(ty, blocks, k, m, x)) <= 1e-4, name
        emb = g.tensors["token_embd.weight"]
        ids = torch.tensor([19, 0, 7], dtype=torch.int32, device="cuda")
        rows = torch.empty(3, emb.K, dtype=torch.float32, device="cuda")
        enc.embedBatch(ids, w, rows, emb.K, 3, emb.type, emb.M, weight_off=emb.offset)
        torch.cuda.synchronize()
        full = oracle.dequant(emb.type, tensors[emb.name][3]).reshape(emb.M, emb.K)
        assert np.array_equal(rows.cpu().numpy(), full[[19, 0, 7]])
        w.free()
