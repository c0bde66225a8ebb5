"""Host-side mirror of Laplace's matmul front-end (``src/matmul.h:18-54``).

Same names and argument meaning as the reference: ``matmul_rows(x, w, y, M, K, N)``
overwrites ``y[M, N]`` with ``x[M, K] @ W^T`` for a weight tensor of N rows of K
block-quantized elements; ``fused_moe_gemm_idx`` / ``fused_moe_gemm_multi`` are the
expert-indexed GEMVs of ``src/matmul.cpp:456-500``. Arrays are numpy arrays in
host memory, exactly like the reference's raw pointers; every call goes through
the C ABI to the GPU. Where the reference would fall back to its scalar CPU
code (an unsupported type), this mirror raises instead: the library has no CPU
path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import _lib
from .ggml import GGMLType, row_bytes


class LaplaceCudaError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"laplace_cuda error {code}: {msg}")
        self.code = code


@dataclass
class Tensor:
    """The fields of the reference's ``Tensor`` view that this path reads (src/tensor.h:130-163)."""

    type: int
    data: np.ndarray          # uint8, the GGUF bytes: N rows (x n_experts) of row_bytes(type, K)
    dims: tuple = ()


_initialised = False


def _ensure_init(device: int = 0) -> C.CDLL:
    global _initialised
    lib = _lib.load()
    if not _initialised:
        _check(lib, lib.laplace_cuda_init(device))
        _initialised = True
    return lib


def _check(lib, rc: int) -> None:
    if rc == 0:
        return
    if rc == 1:
        raise LaplaceCudaError(1, "weight type not handled by the CUDA back-end (the reference would fall back to scalar)")
    raise LaplaceCudaError(rc, lib.laplace_cuda_last_error().decode())


def _f32(a: np.ndarray, n: int, what: str) -> np.ndarray:
    if a.dtype != np.float32 or not a.flags.c_contiguous:
        raise TypeError(f"{what} must be a C-contiguous float32 array")
    if a.size < n:
        raise ValueError(f"{what} holds {a.size} floats, need {n}")
    return a


def _u8(w: Tensor, nbytes: int) -> np.ndarray:
    d = w.data
    if d.dtype != np.uint8 or not d.flags.c_contiguous:
        raise TypeError("Tensor.data must be a C-contiguous uint8 array")
    if d.size < nbytes:
        raise ValueError(f"Tensor.data holds {d.size} bytes, need {nbytes}")
    return d


def matmul_register_weights(base: np.ndarray) -> None:
    """``matmul_register_weights(base, size)`` (src/matmul.h:26): uploads the region to HBM once."""
    lib = _ensure_init()
    _check(lib, lib.laplace_cuda_register_weights(base.ctypes.data, base.nbytes))


def matmul_unregister_weights(base: np.ndarray) -> None:
    lib = _ensure_init()
    _check(lib, lib.laplace_cuda_unregister_weights(base.ctypes.data))


def matmul_rows(x: np.ndarray, w: Tensor, y: np.ndarray, M: int, K: int, N: int) -> None:
    """``matmul_rows`` (src/matmul.cpp:408-433): y[m*N+j] = dot(x[m], row j of w)."""
    lib = _ensure_init()
    x = np.ascontiguousarray(x, dtype=np.float32) if not (isinstance(x, np.ndarray) and x.flags.c_contiguous) else x
    _f32(x, M * K, "x")
    _f32(y, M * N, "y")
    d = _u8(w, N * row_bytes(w.type, K)) if int(w.type) in (2, 6, 8, 12, 14) else w.data
    _check(lib, lib.laplace_cuda_gemm(x.ctypes.data, d.ctypes.data, int(w.type), y.ctypes.data, M, K, N))


def matmul_row(x: np.ndarray, w: Tensor, y: np.ndarray, K: int, N: int) -> None:
    """``matmul_row`` (src/matmul.cpp:435-437)."""
    matmul_rows(x, w, y, 1, K, N)


def _moe(fn_name: str, x, w: Tensor, y, expert_idx, n_experts: int, K: int, N: int, x_rows: int) -> None:
    lib = _ensure_init()
    idx = np.ascontiguousarray(expert_idx, dtype=np.int32)
    if idx.size < n_experts:
        raise ValueError("expert_idx shorter than n_experts")
    _f32(x, x_rows * K, "x")
    _f32(y, n_experts * N, "y")
    need = (int(idx[:n_experts].max()) + 1) * N * row_bytes(w.type, K) if n_experts > 0 else 0
    d = _u8(w, need)
    fn = getattr(lib, fn_name)
    _check(lib, fn(x.ctypes.data, d.ctypes.data, int(w.type), idx.ctypes.data, n_experts, y.ctypes.data, K, N))


def fused_moe_gemm_idx(x, w: Tensor, y, expert_idx, n_experts: int, K: int, N: int) -> None:
    """``fused_moe_gemm_idx`` (src/matmul.cpp:456-477): one shared x for all selected experts."""
    _moe("laplace_cuda_moe_gemv", x, w, y, expert_idx, n_experts, K, N, 1)


def fused_moe_gemm_multi(x, w: Tensor, y, expert_idx, n_experts: int, K: int, N: int) -> None:
    """``fused_moe_gemm_multi`` (src/matmul.cpp:479-500): x[k*K..] per selected expert."""
    _moe("laplace_cuda_moe_gemv_multi", x, w, y, expert_idx, n_experts, K, N, n_experts)
