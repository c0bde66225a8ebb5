"""GGML type ids and block geometry of the weight formats on this path.

Values follow Laplace ``src/tensor.h:11-34`` (ids) and ``src/tensor.h:41-100`` /
``src/kernels.h:21-54`` (bytes and elements per block).
"""
from __future__ import annotations

import enum


class GGMLType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q5_0 = 6
    Q8_0 = 8
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    BF16 = 30


_GEOM = {
    GGMLType.Q4_0: (32, 18),
    GGMLType.Q5_0: (32, 22),
    GGMLType.Q8_0: (32, 34),
    GGMLType.Q4_K: (256, 144),
    GGMLType.Q6_K: (256, 210),
}

SUPPORTED = tuple(_GEOM)          # the types with an int8 path (Q8 activations)

# every type the library takes: those above, and those served with fp32 activations / dequantized only
# (elements and bytes per block, Laplace src/tensor.h:41-100)
ALL_GEOM = dict(_GEOM)
ALL_GEOM.update({GGMLType.F32: (1, 4), GGMLType.F16: (1, 2), GGMLType.BF16: (1, 2),
                 GGMLType.Q2_K: (256, 84), GGMLType.Q3_K: (256, 110), GGMLType.Q5_K: (256, 176)})
F32_ACTIVATION_TYPES = (GGMLType.F32, GGMLType.F16, GGMLType.BF16, GGMLType.Q2_K, GGMLType.Q3_K, GGMLType.Q5_K)


def any_row_bytes(t: int, K: int) -> int:
    e, b = ALL_GEOM[GGMLType(t)]
    return K // e * b


def block_elems(t: int) -> int:
    return _GEOM[GGMLType(t)][0]


def block_bytes(t: int) -> int:
    return _GEOM[GGMLType(t)][1]


def row_bytes(t: int, K: int) -> int:
    """Bytes of one weight row of K elements (``rb`` in src/matmul_simd.cpp:482)."""
    e, b = _GEOM[GGMLType(t)]
    if K % e:
        raise ValueError(f"K={K} is not a multiple of the {e}-element block of {GGMLType(t).name}")
    return K // e * b


def blocksums_per_row(t: int, K: int) -> int:
    """Integer block sums per (activation row, weight row): per 16 values for Q6_K, per 32 otherwise."""
    return K // 16 if GGMLType(t) == GGMLType.Q6_K else K // 32
