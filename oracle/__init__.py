"""CPU oracle (test infrastructure): ctypes wrapper over okf_oracle.c.

Only the tests, the smoke check and the bench's CPU-baseline leg import this
package.  The shipped library never does.
"""
from .oracle import (  # noqa: F401
    Q8_0, Q4_K, IQ2_XXS, Q2_0, Q4_0, Q5_K, Q6_K, IQ4_NL, TYPES, block_bytes, block_elems, build, dequant,
    matmul, matmul_f64, matvec, row_bytes, add_rmsnorm, silu_mul, srq, argmax_rows,
)
