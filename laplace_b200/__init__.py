"""laplace_b200 - B200 (sm_100a) back-end for Laplace's block-quantized weight matmul.

The product is the C-ABI shared library built from ``csrc/`` (header:
``include/laplace_cuda.h``). This package is the thin host-side mirror of the
reference's matmul front-end (Laplace ``src/matmul.h``) used by tests and the
benchmark; it loads the library through ctypes and fails loudly when the
library is missing. Nothing here computes a matmul on the CPU.
"""
from .ggml import GGMLType, block_bytes, block_elems, row_bytes  # noqa: F401
from .matmul import (  # noqa: F401
    LaplaceCudaError,
    Tensor,
    fused_moe_gemm_idx,
    fused_moe_gemm_multi,
    matmul_register_weights,
    matmul_row,
    matmul_rows,
    matmul_unregister_weights,
)
