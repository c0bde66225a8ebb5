"""ctypes binding of liblaplace_cuda.so (declarations: include/laplace_cuda.h)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "liblaplace_cuda.so"

# every symbol include/laplace_cuda.h declares: name -> (restype, argtypes)
_vp, _i, _u32, _sz = C.c_void_p, C.c_int, C.c_uint32, C.c_size_t
SYMBOLS = {
    "laplace_cuda_init": (_i, [_i]),
    "laplace_cuda_shutdown": (None, []),
    "laplace_cuda_sync": (_i, []),
    "laplace_cuda_sync_stream": (_i, [_vp]),
    "laplace_cuda_last_error": (C.c_char_p, []),
    "laplace_cuda_sm_count": (_i, []),
    "laplace_cuda_register_weights": (_i, [_vp, _sz]),
    "laplace_cuda_unregister_weights": (_i, [_vp]),
    "laplace_cuda_nsplit": (None, [_i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    "laplace_cuda_gemm": (_i, [_vp, _vp, _u32, _vp, _i, _i, _i]),
    "laplace_cuda_moe_gemv": (_i, [_vp, _vp, _u32, _vp, _i, _vp, _i, _i]),
    "laplace_cuda_moe_gemv_multi": (_i, [_vp, _vp, _u32, _vp, _i, _vp, _i, _i]),
    "laplace_cuda_gemm_dev": (_i, [_vp, _vp, _u32, _vp, _i, _i, _i, _vp]),
    "laplace_cuda_gemm_multi_dev": (_i, [_vp, _vp, C.c_float, _vp, _vp, _i, _u32, _i, _i, _vp]),
    "laplace_cuda_gemm_noalloc_dev": (_i, [_vp, _vp, _u32, _vp, _i, _i, _i, _vp]),
    "laplace_cuda_moe_gemv_dev": (_i, [_vp, _vp, _u32, _vp, _i, _vp, _i, _i, _i, _vp]),
    "laplace_cuda_moe_grouped_dev": (_i, [_vp, _vp, _u32, _vp, _vp, _i, _i, _vp, _i, _i, _vp]),
    "laplace_cuda_moe_ffn_dev": (_i, [_vp, _vp, _vp, _u32, _u32, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp]),
    "laplace_cuda_moe_route_dev": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp]),
    "laplace_cuda_peer_alloc": (_i, [_sz, C.POINTER(_vp), _vp]),
    "laplace_cuda_peer_open": (_i, [_vp, C.POINTER(_vp)]),
    "laplace_cuda_peer_close": (_i, [_vp]),
    "laplace_cuda_peer_free": (_i, [_vp]),
    "laplace_cuda_gemm_allgather_dev": (_i, [_vp, _vp, _u32, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp]),
    "laplace_cuda_allgather_wait_dev": (_i, [_vp, _vp, _i, _i, _vp]),
    "laplace_cuda_gemm_peers_dev": (_i, [_vp, _vp, _u32, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "laplace_cuda_allgather_step_wait_dev": (_i, [_vp, _vp, _i, _i, _vp]),
    "laplace_cuda_moe_pack_dev": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "laplace_cuda_moe_unpack_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "laplace_cuda_quantize_act_dev": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "laplace_cuda_debug_blocksums_dev": (_i, [_vp, _vp, _u32, _vp, _i, _i, _i, _vp]),
    "laplace_cuda_debug_tensor_peak": (_i, [_i, C.POINTER(C.c_double)]),
    "laplace_cuda_dequantize_dev": (_i, [_vp, _u32, _vp, C.c_longlong, _vp]),
    "laplace_cuda_embed_rows_dev": (_i, [_vp, _u32, _vp, _i, _i, C.c_longlong, C.c_float, _vp, _vp]),
    "laplace_cuda_lm_head_dev": (_i, [_vp, _vp, _u32, _vp, _i, _i, _i, C.c_float, _vp]),
    "laplace_cuda_gguf_open": (_i, [C.c_char_p, _i, _i, C.POINTER(C.c_char_p), _i, C.POINTER(_vp)]),
    "laplace_cuda_gguf_upload": (_i, [_vp]),
    "laplace_cuda_gguf_tensor_count": (_i, [_vp]),
    "laplace_cuda_gguf_tensor": (_i, [_vp, _i, C.c_char_p, _vp]),
    "laplace_cuda_gguf_meta_u64": (_i, [_vp, C.c_char_p, C.POINTER(C.c_ulonglong)]),
    "laplace_cuda_gguf_meta_f64": (_i, [_vp, C.c_char_p, C.POINTER(C.c_double)]),
    "laplace_cuda_gguf_meta_str": (C.c_char_p, [_vp, C.c_char_p]),
    "laplace_cuda_gguf_close": (None, [_vp]),
    "laplace_cuda_last_path": (_i, []),
    "laplace_cuda_launch_count": (C.c_longlong, [_i]),
}



class GgufTensorInfo(C.Structure):
    """laplace_cuda_gguf_tensor_info."""
    _fields_ = [("name", C.c_char_p), ("type", C.c_uint32), ("n_dims", C.c_uint32), ("dims", C.c_ulonglong * 4),
                ("kind", C.c_int), ("row_begin", C.c_ulonglong), ("row_end", C.c_ulonglong),
                ("expert_begin", C.c_ulonglong), ("expert_end", C.c_ulonglong), ("file_offset", C.c_ulonglong),
                ("bytes", C.c_ulonglong), ("host", C.c_void_p), ("dev", C.c_void_p)]


class Matrix(C.Structure):
    """laplace_cuda_matrix: one weight matrix of a multi-matrix call (device pointers)."""
    _fields_ = [("w", C.c_void_p), ("y", C.c_void_p), ("N", C.c_int)]


_lib = None


def load() -> C.CDLL:
    """Loads the shared library and types every entry point. No CUDA call is made."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m laplace_b200.build` "
            "(there is no CPU fallback for this path)"
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
