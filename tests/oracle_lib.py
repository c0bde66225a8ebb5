"""ctypes access to the CPU checkers under oracle/ - for tests, smoke and the CPU-baseline timer only.

``Oracle`` wraps liboracle_q8.so (the C restatement of the reference's int8
path). ``Reference`` wraps oracle/_ref/libref_matmul.so when it exists (the
reference's own scalar code compiled from its sources; it is built only where
the reference checkout is present).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent.parent / "oracle"

ACTQ8 = np.dtype([("d", "<f4"), ("sum", "<f4"), ("sum_lo", "<i2"), ("sum_hi", "<i2"), ("qs", "i1", (32,))])
assert ACTQ8.itemsize == 44

MODE_F32, MODE_F64, MODE_MASS = 0, 1, 2
_vp, _i, _u32 = C.c_void_p, C.c_int, C.c_uint32


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def build_oracle() -> Path:
    lib = ORACLE_DIR / "liboracle_q8.so"
    src = [ORACLE_DIR / "oracle_q8.c", ORACLE_DIR / "oracle_q8.h"]
    if not lib.exists() or any(s.stat().st_mtime > lib.stat().st_mtime for s in src):
        subprocess.run(["make", "-s", "-C", str(ORACLE_DIR), "all"], check=True)
    return lib


class Oracle:
    def __init__(self):
        self.lib = L = C.CDLL(str(build_oracle()))
        L.lpo_fp16_to_fp32.restype = C.c_float
        L.lpo_fp16_to_fp32.argtypes = [C.c_uint16]
        L.lpo_fp32_to_fp16.restype = C.c_uint16
        L.lpo_fp32_to_fp16.argtypes = [C.c_float]
        L.lpo_row_bytes.restype = C.c_size_t
        L.lpo_row_bytes.argtypes = [_u32, _i]
        L.lpo_quantize_rows.argtypes = [_vp, _i, _i, _vp]
        L.lpo_gemm.argtypes = [_vp, _vp, _u32, _vp, _i, _i, _i, _i, _i]
        L.lpo_moe_gemv.argtypes = [_vp, _vp, _u32, _vp, _i, _vp, _i, _i, _i, _i]
        L.lpo_moe_gemv_multi.argtypes = [_vp, _vp, _u32, _vp, _i, _vp, _i, _i, _i, _i]
        L.lpo_gemm_blocksums.argtypes = [_vp, _vp, _u32, _vp, _i, _i, _i]
        L.lpo_gemm_scalar.argtypes = [_vp, _vp, _u32, _vp, _i, _i, _i, _i]
        L.lpo_dequantize.argtypes = [_u32, _vp, _vp, C.c_size_t]
        L.lpo_testgen_x.argtypes = [_u32, _i, _vp]
        L.lpo_testgen_weights.argtypes = [_u32, _i, _i, _vp]

    def fp16_to_fp32(self, h: int) -> float:
        return self.lib.lpo_fp16_to_fp32(h)

    def fp32_to_fp16(self, f: float) -> int:
        return self.lib.lpo_fp32_to_fp16(f)

    def row_bytes(self, t: int, K: int) -> int:
        return self.lib.lpo_row_bytes(t, K)

    def quantize(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
        M, K = x.shape
        out = np.zeros((M, K // 32), dtype=ACTQ8)
        self.lib.lpo_quantize_rows(_ptr(x), M, K, _ptr(out))
        return out

    def gemm(self, x, w, t, M, K, N, mode=MODE_F32, threads=1) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        y = np.zeros((M, N), dtype=np.float32)
        rc = self.lib.lpo_gemm(_ptr(x), _ptr(w), int(t), _ptr(y), M, K, N, mode, threads)
        if rc:
            raise ValueError(f"oracle does not handle type {t}")
        return y

    def moe_gemv(self, x, w, t, idx, K, N, multi=False, mode=MODE_F32, threads=1) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        y = np.zeros((idx.size, N), dtype=np.float32)
        fn = self.lib.lpo_moe_gemv_multi if multi else self.lib.lpo_moe_gemv
        rc = fn(_ptr(x), _ptr(w), int(t), _ptr(idx), idx.size, _ptr(y), K, N, mode, threads)
        if rc:
            raise ValueError(f"oracle does not handle type {t}")
        return y

    def blocksums(self, x, w, t, M, K, N) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        per = K // 16 if int(t) == 14 else K // 32
        out = np.zeros((M, N, per), dtype=np.int32)
        rc = self.lib.lpo_gemm_blocksums(_ptr(x), _ptr(w), int(t), _ptr(out), M, K, N)
        if rc:
            raise ValueError(f"oracle does not handle type {t}")
        return out

    def gemm_scalar(self, x, w, t, M, K, N, threads=1) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        y = np.zeros((M, N), dtype=np.float32)
        self.lib.lpo_gemm_scalar(_ptr(x), _ptr(w), int(t), _ptr(y), M, K, N, threads)
        return y

    def dequantize(self, w, t, n) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.uint8)
        out = np.zeros(n, dtype=np.float32)
        self.lib.lpo_dequantize(int(t), _ptr(w), _ptr(out), n)
        return out

    def testgen(self, t: int, K: int, N: int):
        """x and weight bytes exactly as the reference's tests/test_matmul.cpp builds them."""
        x = np.zeros(K, dtype=np.float32)
        self.lib.lpo_testgen_x(int(t), K, _ptr(x))
        w = np.zeros((N, self.row_bytes(t, K)), dtype=np.uint8)
        self.lib.lpo_testgen_weights(int(t), K, N, _ptr(w))
        return x, w


def rmsnorm_rows_np(x, w, eps):
    """Restatement of the reference's scalar rmsnorm (src/ops.cpp:69-73): ms summed in index order in fp32,
    inv = 1 / sqrt(ms / n + eps), y = x * inv * w (two fp32 multiplies in that order)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    y = np.zeros_like(x)
    n = x.shape[1]
    for r in range(x.shape[0]):
        ms = np.float32(0.0)
        for v in x[r]:
            ms = np.float32(ms + np.float32(v * v))
        inv = np.float32(1.0) / np.sqrt(np.float32(ms / np.float32(n)) + np.float32(eps), dtype=np.float32)
        y[r] = (x[r] * inv).astype(np.float32) * w
    return y


class Reference:
    """The reference's own scalar matmul, when oracle/_ref was built (needs the reference checkout)."""

    PATH = ORACLE_DIR / "_ref" / "libref_matmul.so"

    @classmethod
    def available(cls) -> bool:
        return cls.PATH.exists()

    def __init__(self):
        self.lib = L = C.CDLL(str(self.PATH))
        L.ref_set_threads.argtypes = [_i]
        L.ref_threads.restype = _i
        L.ref_matmul_rows.argtypes = [_vp, _vp, _u32, _vp, _i, _i, _i]
        L.ref_fused_moe_gemm_idx.argtypes = [_vp, _vp, _u32, _vp, _i, _i, _vp, _i, _i]
        L.ref_fused_moe_gemm_multi.argtypes = [_vp, _vp, _u32, _vp, _i, _i, _vp, _i, _i]
        L.ref_dequantize.argtypes = [_vp, _u32, _vp, _i]
        L.ref_fp16_to_fp32.restype = C.c_float
        L.ref_fp16_to_fp32.argtypes = [C.c_uint16]
        L.ref_fp32_to_fp16.restype = C.c_uint16
        L.ref_fp32_to_fp16.argtypes = [C.c_float]
        if hasattr(L, "ref_rmsnorm_rows"):
            L.ref_rmsnorm_rows.argtypes = [_vp, _vp, _vp, _i, _i, C.c_float]

    def rmsnorm_rows(self, x, w, eps) -> np.ndarray:
        """ops::rmsnorm_rows of the reference build (src/ops.cpp:34-80)."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        y = np.zeros_like(x)
        self.lib.ref_rmsnorm_rows(_ptr(x), _ptr(w), _ptr(y), x.shape[0], x.shape[1], float(eps))
        return y

    def set_threads(self, t: int) -> int:
        self.lib.ref_set_threads(t)
        return self.lib.ref_threads()

    def matmul_rows(self, x, w, t, M, K, N) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        y = np.zeros((M, N), dtype=np.float32)
        self.lib.ref_matmul_rows(_ptr(x), _ptr(w), int(t), _ptr(y), M, K, N)
        return y

    def moe(self, x, w, t, idx, n_total, K, N, multi=False) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.uint8)
        idx = np.ascontiguousarray(idx, dtype=np.int32)
        y = np.zeros((idx.size, N), dtype=np.float32)
        fn = self.lib.ref_fused_moe_gemm_multi if multi else self.lib.ref_fused_moe_gemm_idx
        fn(_ptr(x), _ptr(w), int(t), _ptr(idx), idx.size, n_total, _ptr(y), K, N)
        return y

    def dequantize(self, w, t, n) -> np.ndarray:
        w = np.ascontiguousarray(w, dtype=np.uint8)
        out = np.zeros(n, dtype=np.float32)
        self.lib.ref_dequantize(_ptr(w), int(t), _ptr(out), n)
        return out
