"""chatokf_b200: ChatOKF's block-quantized matvec / matmul operator on B200.

Only the hot path lives here: the CUDA kernels and C ABI (csrc/, built into
libokfcuda.so), the host-side mirror of the reference's operator interface
(enc.py), the row-sharded multi-GPU wrapper (tp.py) and synthetic block
encoders for tests and the bench (synth.py).
"""
from .gguf_types import GGUFType, block_bytes, block_elems, row_byte_count  # noqa: F401

__all__ = ["GGUFType", "block_bytes", "block_elems", "row_byte_count"]
