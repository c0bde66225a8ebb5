"""Seeded synthetic inputs for tests and the benchmark (numpy, host side only).

No model file or public dataset is involved: weights are fp32 ~ N(0, 0.02^2)
and activations fp32 ~ N(0, 1), drawn from a counter-based Philox generator so
that any process regenerates the same tensor from (seed, shape).

Three ways of turning fp32 weights into GGUF blocks:

* ``pack_ref_*``  - restatements of the only fp32->block packers the reference
  owns, the test helpers of Laplace ``tests/test_metal.cpp:23-96`` (they are
  crude on purpose: Q4_K / Q6_K sub-block scales are LCG bytes);
* ``pack_affine_*`` - straightforward min/max (Q4_K) and absmax (others)
  quantizers written for this repository, whose dequantized values do resemble
  the fp32 input;
* ``random_blocks`` - random payload bytes with sane fp16 scales, the style of
  Laplace ``tests/test_matmul.cpp:51-55,142-212``.

The dot kernels do not care how the bytes were made; the variety is there to
exercise every bit pattern of the layouts.
"""
from __future__ import annotations

import numpy as np

from laplace_b200.ggml import GGMLType, row_bytes

# ------------------------------------------------------------------ RNG


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def normal_f32(seed: int, shape, std: float = 1.0) -> np.ndarray:
    a = rng(seed).standard_normal(shape, dtype=np.float32)
    if std != 1.0:
        a *= np.float32(std)
    return a


# ------------------------------------------------------------------ fp16


def f32_to_f16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> binary16 bits the way Laplace ``src/fp16.h:40-69`` narrows (half-up on the dropped bits)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.int64)
    sign = (bits >> 16) & 0x8000
    e = ((bits >> 23) & 0xFF) - 112
    man = bits & 0x7FFFFF
    out = np.zeros(bits.shape, dtype=np.int64)

    sub = e <= 0
    sh = np.clip(1 - e, 0, 40)
    m_sub = (man | 0x800000) >> sh
    m_sub = np.where(m_sub & 0x1000, m_sub + 0x2000, m_sub)
    out = np.where(sub, np.where(e < -10, sign, sign | (m_sub >> 13)), out)

    infnan = e == (0xFF - 112)
    out = np.where(infnan, sign | 0x7C00 | np.where(man != 0, man >> 13, 0), out)

    big = (~sub) & (~infnan) & (e > 30)
    out = np.where(big, sign | 0x7C00, out)

    norm = (~sub) & (~infnan) & (e <= 30)
    m2 = np.where(man & 0x1000, man + 0x2000, man)
    carry = (m2 & 0x800000) != 0
    e2 = np.where(carry, e + 1, e)
    m2 = np.where(carry, 0, m2)
    val = np.where(e2 > 30, sign | 0x7C00, sign | (e2 << 10) | (m2 >> 13))
    out = np.where(norm, val, out)
    return out.astype(np.uint16)


def f16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(h, dtype=np.uint16).view(np.float16).astype(np.float32)


def _roundf(v: np.ndarray) -> np.ndarray:
    """C roundf: nearest, halves away from zero."""
    t = np.trunc(v)
    return t + np.where(np.abs(v - t) >= 0.5, np.sign(v), 0).astype(v.dtype)


def _lcg_bytes(seed: int, n: int) -> np.ndarray:
    """(uint8)(s >> 16) of s <- s*1103515245 + 12345 (mod 2^32), n values after the seed."""
    a = np.full(n, 1103515245, dtype=np.uint64)
    apow = np.cumprod(a, dtype=np.uint64) & 0xFFFFFFFF              # a^1 .. a^n  (wraps mod 2^64, then mask)
    # cumprod in uint64 wraps mod 2^64, and (x mod 2^64) mod 2^32 == x mod 2^32
    geo = np.concatenate(([1], apow[:-1])).astype(np.uint64)        # a^0 .. a^(n-1)
    gsum = np.cumsum(geo, dtype=np.uint64) & 0xFFFFFFFF             # 1 + a + ... + a^(k-1)
    s = (apow * np.uint64(seed) + np.uint64(12345) * gsum) & 0xFFFFFFFF
    return (s >> 16).astype(np.uint32)                              # caller narrows


# ------------------------------------------------- reference test packers


def _blocks(w: np.ndarray, n: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32)
    N, K = w.shape
    if K % n:
        raise ValueError(f"K={K} not a multiple of {n}")
    return w.reshape(N, K // n, n)


def _amax_d(b: np.ndarray, div: float):
    amax = np.abs(b).max(axis=-1)
    d = (amax / np.float32(div)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    return amax, d, inv


def pack_ref_q4_0(w: np.ndarray) -> np.ndarray:
    """tests/test_metal.cpp:23-35."""
    b = _blocks(w, 32)
    _, d, inv = _amax_d(b, 8)
    q = _roundf(b * inv[..., None] + np.float32(8)).astype(np.int32)
    out = np.zeros(b.shape[:2] + (18,), dtype=np.uint8)
    out[..., 0:2] = f32_to_f16_bits(d)[..., None].view(np.uint8).reshape(b.shape[:2] + (2,))
    out[..., 2:] = ((q[..., :16] & 0xF) | ((q[..., 16:] & 0xF) << 4)).astype(np.uint8)
    return out.reshape(b.shape[0], -1)


def pack_ref_q5_0(w: np.ndarray) -> np.ndarray:
    """tests/test_metal.cpp:36-50: d = amax / 16, q = roundf(x / d + 16); low four bits in the nibbles, bit 4 in qh."""
    b = _blocks(w, 32)
    _, d, inv = _amax_d(b, 16)
    q = _roundf(b * inv[..., None] + np.float32(16)).astype(np.int64)
    out = np.zeros(b.shape[:2] + (22,), dtype=np.uint8)
    out[..., 0:2] = f32_to_f16_bits(d)[..., None].view(np.uint8).reshape(b.shape[:2] + (2,))
    qh = (((q >> 4) & 1) << np.arange(32, dtype=np.int64)).sum(axis=-1).astype(np.uint32)
    out[..., 2:6] = qh[..., None].view(np.uint8).reshape(b.shape[:2] + (4,))
    out[..., 6:] = ((q[..., :16] & 0xF) | ((q[..., 16:] & 0xF) << 4)).astype(np.uint8)
    return out.reshape(b.shape[0], -1)


def pack_ref_q8_0(w: np.ndarray) -> np.ndarray:
    """tests/test_metal.cpp:51-60."""
    b = _blocks(w, 32)
    _, d, inv = _amax_d(b, 127)
    q = np.clip(_roundf(b * inv[..., None]), -127, 127).astype(np.int8)
    out = np.zeros(b.shape[:2] + (34,), dtype=np.uint8)
    out[..., 0:2] = f32_to_f16_bits(d)[..., None].view(np.uint8).reshape(b.shape[:2] + (2,))
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(b.shape[0], -1)


def pack_ref_q4_K(w: np.ndarray) -> np.ndarray:
    """tests/test_metal.cpp:61-75 (scale bytes from the LCG seeded 999, in block order)."""
    b = _blocks(w, 256)
    amax, d, inv = _amax_d(b, 15)
    nb = b.shape[0] * b.shape[1]
    out = np.zeros(b.shape[:2] + (144,), dtype=np.uint8)
    out[..., 0:2] = f32_to_f16_bits(d)[..., None].view(np.uint8).reshape(b.shape[:2] + (2,))
    dmin = (amax / np.float32(240)).astype(np.float32)
    out[..., 2:4] = f32_to_f16_bits(dmin)[..., None].view(np.uint8).reshape(b.shape[:2] + (2,))
    out[..., 4:16] = _lcg_bytes(999, nb * 12).astype(np.uint8).reshape(b.shape[:2] + (12,))
    q = _roundf(b * inv[..., None]).astype(np.int32)
    out[..., 16:] = ((q[..., :128] & 0xF) | ((q[..., 128:] & 0xF) << 4)).astype(np.uint8)
    return out.reshape(b.shape[0], -1)


def pack_ref_q6_K(w: np.ndarray) -> np.ndarray:
    """tests/test_metal.cpp:76-96 (scales from the LCG seeded 777; its qh shifts are kept as written)."""
    b = _blocks(w, 256)
    _, d, inv = _amax_d(b, 31)
    nb = b.shape[0] * b.shape[1]
    out = np.zeros(b.shape[:2] + (210,), dtype=np.uint8)
    val = np.clip(_roundf(b * inv[..., None] + np.float32(32)), 0, 63).astype(np.int32)
    lo, hi = val & 0xF, (val >> 4) & 3
    v4 = lo.reshape(b.shape[:2] + (2, 2, 64))             # [half][l >= 64][l % 64]
    ql = (v4[..., 0, :] | (v4[..., 1, :] << 4)).astype(np.uint8)
    out[..., 0:128] = ql.reshape(b.shape[:2] + (128,))
    h4 = hi.reshape(b.shape[:2] + (2, 4, 32))             # [half][l // 32][l % 32]
    shift = np.where(np.arange(32) < 16, 0, 2)            # (l // 16) * 2 for l < 32
    qh = ((h4[..., 0, :] << shift) | (h4[..., 1, :] << (shift + 4))) & 0xFF   # l >= 64 shifts past the byte
    out[..., 128:192] = qh.astype(np.uint8).reshape(b.shape[:2] + (64,))
    sc = (_lcg_bytes(777, nb * 16) % 64).astype(np.int32) - 32
    out[..., 192:208] = sc.astype(np.int8).view(np.uint8).reshape(b.shape[:2] + (16,))
    out[..., 208:210] = f32_to_f16_bits(d)[..., None].view(np.uint8).reshape(b.shape[:2] + (2,))
    return out.reshape(b.shape[0], -1)


# ------------------------------------------------------- affine packers


def _h(d: np.ndarray):
    """Rounds scales to fp16 and returns (bits, value actually stored)."""
    bits = np.ascontiguousarray(d, dtype=np.float32).astype(np.float16).view(np.uint16)
    return bits, bits.view(np.float16).astype(np.float32)


def _put16(out: np.ndarray, lo: int, bits: np.ndarray) -> None:
    out[..., lo] = (bits & 0xFF).astype(np.uint8)
    out[..., lo + 1] = (bits >> 8).astype(np.uint8)


def _safe_div(a, b):
    with np.errstate(divide="ignore", invalid="ignore"):
        return np.where(b != 0, a / np.where(b != 0, b, 1), 0).astype(np.float32)


def pack_affine_q4_0(w: np.ndarray) -> np.ndarray:
    b = _blocks(w, 32)
    bits, d = _h(np.abs(b).max(axis=-1) / np.float32(7))
    q = np.clip(np.rint(_safe_div(b, d[..., None])) + 8, 0, 15).astype(np.uint8)
    out = np.zeros(b.shape[:2] + (18,), dtype=np.uint8)
    _put16(out, 0, bits)
    out[..., 2:] = q[..., :16] | (q[..., 16:] << 4)
    return out.reshape(b.shape[0], -1)


def pack_affine_q5_0(w: np.ndarray) -> np.ndarray:
    b = _blocks(w, 32)
    bits, d = _h(np.abs(b).max(axis=-1) / np.float32(15))
    q = np.clip(np.rint(_safe_div(b, d[..., None])) + 16, 0, 31).astype(np.int64)
    out = np.zeros(b.shape[:2] + (22,), dtype=np.uint8)
    _put16(out, 0, bits)
    qh = ((q >> 4) << np.arange(32, dtype=np.int64)).sum(axis=-1).astype(np.uint32)
    out[..., 2:6] = qh[..., None].view(np.uint8).reshape(b.shape[:2] + (4,))
    out[..., 6:] = ((q[..., :16] & 0xF) | ((q[..., 16:] & 0xF) << 4)).astype(np.uint8)
    return out.reshape(b.shape[0], -1)


def pack_affine_q8_0(w: np.ndarray) -> np.ndarray:
    b = _blocks(w, 32)
    bits, d = _h(np.abs(b).max(axis=-1) / np.float32(127))
    q = np.clip(np.rint(_safe_div(b, d[..., None])), -127, 127).astype(np.int8)
    out = np.zeros(b.shape[:2] + (34,), dtype=np.uint8)
    _put16(out, 0, bits)
    out[..., 2:] = q.view(np.uint8)
    return out.reshape(b.shape[0], -1)


def pack_affine_q4_K(w: np.ndarray) -> np.ndarray:
    b = _blocks(w, 256)
    s = b.reshape(b.shape[:2] + (8, 32))
    mn = np.minimum(s.min(axis=-1), 0)
    mx = np.maximum(s.max(axis=-1), 0)
    scale = (mx - mn) / np.float32(15)                     # per sub-block step
    offs = -mn                                             # per sub-block offset, >= 0
    dbits, d = _h(scale.max(axis=-1) / np.float32(63))
    mbits, dmin = _h(offs.max(axis=-1) / np.float32(63))
    sc = np.clip(np.rint(_safe_div(scale, d[..., None])), 0, 63).astype(np.int32)
    mm = np.clip(np.rint(_safe_div(offs, dmin[..., None])), 0, 63).astype(np.int32)
    step = d[..., None] * sc
    q = np.clip(np.rint(_safe_div(s + (dmin[..., None] * mm)[..., None], step[..., None])), 0, 15).astype(np.uint8)
    out = np.zeros(b.shape[:2] + (144,), dtype=np.uint8)
    _put16(out, 0, dbits)
    _put16(out, 2, mbits)
    # 12 bytes holding eight 6-bit (scale, min) pairs; inverse of get_scale_min_k4 (src/kernels.h:82-90)
    for j in range(4):
        out[..., 4 + j] = (sc[..., j] | ((sc[..., j + 4] >> 4) << 6)).astype(np.uint8)
        out[..., 8 + j] = (mm[..., j] | ((mm[..., j + 4] >> 4) << 6)).astype(np.uint8)
        out[..., 12 + j] = ((sc[..., j + 4] & 0xF) | ((mm[..., j + 4] & 0xF) << 4)).astype(np.uint8)
    q = q.reshape(b.shape[:2] + (4, 2, 32))                # [chunk][low/high nibble][l]
    out[..., 16:] = (q[..., 0, :] | (q[..., 1, :] << 4)).reshape(b.shape[:2] + (128,))
    return out.reshape(b.shape[0], -1)


def pack_affine_q6_K(w: np.ndarray) -> np.ndarray:
    b = _blocks(w, 256)
    g = b.reshape(b.shape[:2] + (16, 16))
    a = np.abs(g).max(axis=-1)                             # per 16 values
    dbits, d = _h(a.max(axis=-1) / np.float32(31 * 127))
    sc = np.clip(np.rint(_safe_div(a, (np.float32(31) * d)[..., None])), 1, 127).astype(np.int32)
    q = np.clip(np.rint(_safe_div(g, (d[..., None] * sc)[..., None])) + 32, 0, 63).astype(np.int32)
    q = q.reshape(b.shape[:2] + (2, 4, 32))                # [half][g][l]
    lo, hi = q & 0xF, q >> 4
    out = np.zeros(b.shape[:2] + (210,), dtype=np.uint8)
    ql = np.stack([lo[..., 0, :] | (lo[..., 2, :] << 4), lo[..., 1, :] | (lo[..., 3, :] << 4)], axis=-2)
    out[..., 0:128] = ql.astype(np.uint8).reshape(b.shape[:2] + (128,))
    qh = hi[..., 0, :] | (hi[..., 1, :] << 2) | (hi[..., 2, :] << 4) | (hi[..., 3, :] << 6)
    out[..., 128:192] = qh.astype(np.uint8).reshape(b.shape[:2] + (64,))
    out[..., 192:208] = sc.astype(np.int8).view(np.uint8)
    _put16(out, 208, dbits)
    return out.reshape(b.shape[0], -1)


PACK_REF = {GGMLType.Q4_0: pack_ref_q4_0, GGMLType.Q5_0: pack_ref_q5_0, GGMLType.Q8_0: pack_ref_q8_0,
            GGMLType.Q4_K: pack_ref_q4_K, GGMLType.Q6_K: pack_ref_q6_K}
PACK_AFFINE = {GGMLType.Q4_0: pack_affine_q4_0, GGMLType.Q5_0: pack_affine_q5_0, GGMLType.Q8_0: pack_affine_q8_0,
               GGMLType.Q4_K: pack_affine_q4_K, GGMLType.Q6_K: pack_affine_q6_K}


# ---------------------------------------------------------- random blocks


def random_blocks(t: int, K: int, N: int, seed: int) -> np.ndarray:
    """Random payload bytes, fp16 scales in [0.005, 0.07], Q6_K sub-scales in -8..8."""
    t = GGMLType(t)
    g = rng(seed)
    rb = row_bytes(t, K)
    raw = g.integers(0, 256, size=(N, rb), dtype=np.uint8)
    bb = {GGMLType.Q4_0: 18, GGMLType.Q5_0: 22, GGMLType.Q8_0: 34, GGMLType.Q4_K: 144, GGMLType.Q6_K: 210}[t]
    blk = raw.reshape(N, rb // bb, bb)

    def scale():
        return (0.005 + 0.065 * g.random(blk.shape[:2], dtype=np.float32)).astype(np.float16).view(np.uint16)

    if t in (GGMLType.Q4_0, GGMLType.Q5_0, GGMLType.Q8_0):
        _put16(blk, 0, scale())
    elif t == GGMLType.Q4_K:
        _put16(blk, 0, scale())
        _put16(blk, 2, scale())
    else:
        blk[..., 192:208] = g.integers(-8, 9, size=blk.shape[:2] + (16,), dtype=np.int8).view(np.uint8)
        _put16(blk, 208, scale())
    return blk.reshape(N, rb)


def weights(t: int, K: int, N: int, seed: int, how: str = "ref") -> np.ndarray:
    """[N, row_bytes] uint8 weights: fp32 N(0, 0.02^2) packed by ``how`` in {"ref", "affine"}, or "random" blocks."""
    if how == "random":
        return random_blocks(t, K, N, seed)
    w = normal_f32(seed, (N, K), 0.02)
    return (PACK_REF if how == "ref" else PACK_AFFINE)[GGMLType(t)](w)


def lossless_q8_activations(seed: int, M: int, K: int) -> np.ndarray:
    """fp32 activations that the per-32 Q8 quantizer represents exactly: every block is d * q with q integers in
    [-127, 127], one of them +-127, and d a power of two. The quantizer then recovers exactly (d, q), so the
    reference's fp32-activation scalar path and its int8 path compute the same dot products up to fp32 summation
    order - which lets code that follows the int8 path be compared with the compiled scalar path at 1e-5."""
    g = rng(seed)
    q = g.integers(-127, 128, size=(M, K // 32, 32)).astype(np.int32)
    pos = g.integers(0, 32, size=(M, K // 32))
    sign = g.integers(0, 2, size=(M, K // 32)) * 2 - 1
    np.put_along_axis(q, pos[..., None], (127 * sign)[..., None], axis=2)
    e = g.integers(-9, -5, size=(M, K // 32, 1))
    return (q.astype(np.float32) * np.exp2(e).astype(np.float32)).reshape(M, K)


def single_live_block(t: int, K: int, N: int, seed: int, live: int):
    """Weights with random payload in which every scale is zero except the ones that cover 32-value block `live`
    of each row (for Q6_K: the two 16-value groups of that block), plus one activation row whose only non-zero
    block is `live`, holding integers q in [-127, 127] (one of them 127) times 2^-3. Every other term of the dot
    is exactly zero, so y[j] = (weight scale product) * 2^-3 * (integer block sum), bit for bit, on any correct
    implementation of the int8 path; returns (w, x, scale[N] or scale[N, 2] for Q6_K)."""
    t = GGMLType(t)
    g = rng(seed)
    w = random_blocks(t, K, N, seed + 1)
    rb = row_bytes(t, K)
    x = np.zeros((1, K), dtype=np.float32)
    q = g.integers(-127, 128, size=32).astype(np.float32)
    q[int(g.integers(0, 32))] = 127.0
    x[0, live * 32:(live + 1) * 32] = q * np.float32(0.125)
    one = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
    if t in (GGMLType.Q4_0, GGMLType.Q5_0, GGMLType.Q8_0):
        bb = {GGMLType.Q4_0: 18, GGMLType.Q5_0: 22, GGMLType.Q8_0: 34}[t]
        blk = w.reshape(N, rb // bb, bb)
        blk[:, :, 0:2] = 0
        blk[:, live, 0:2] = one
        return w, x, np.ones(N, dtype=np.float32)
    sb, j = live // 8, live % 8
    if t == GGMLType.Q4_K:
        blk = w.reshape(N, rb // 144, 144)
        blk[:, :, 0:4] = 0                       # d = dmin = 0 everywhere ...
        blk[:, sb, 0:2] = one                    # ... except d of the live super-block (dmin stays 0)
        sc = np.zeros((N, 8), dtype=np.int64)
        live_sc = g.integers(1, 64, size=N)
        sc[:, j] = live_sc
        packed = np.zeros((N, 12), dtype=np.uint8)   # 6-bit packing of Laplace src/kernels.h:82-90, mins all zero
        for i in range(4):
            packed[:, i] = (sc[:, i] & 63) | ((sc[:, i + 4] >> 4) << 6)
            packed[:, 8 + i] = sc[:, i + 4] & 15
        blk[:, sb, 4:16] = packed
        return w, x, live_sc.astype(np.float32)
    blk = w.reshape(N, rb // 210, 210)
    blk[:, :, 208:210] = 0
    blk[:, sb, 208:210] = one
    scales = np.zeros((N, 16), dtype=np.int8)
    live_sc = g.integers(-128, 128, size=(N, 2)).astype(np.int8)
    half, gq = j // 4, j % 4
    scales[:, 8 * half + 2 * gq] = live_sc[:, 0]
    scales[:, 8 * half + 2 * gq + 1] = live_sc[:, 1]
    blk[:, sb, 192:208] = scales.view(np.uint8)
    return w, x, live_sc.astype(np.float32)


# ---- weight types that are served with fp32 activations / only dequantized (F32, F16, BF16, Q5_0, Q2_K, Q3_K, Q5_K)
_OTHER_GEOM = {0: (1, 4), 1: (1, 2), 30: (1, 2), 6: (32, 22), 10: (256, 84), 11: (256, 110), 13: (256, 176)}
_OTHER_SCALE_FIELDS = {6: (0,), 10: (80, 82), 11: (108,), 13: (0, 2)}        # byte offsets of the fp16 scales in a block


def other_type_weights(t: int, K: int, N: int, seed: int) -> np.ndarray:
    """[N, row_bytes] uint8: random blocks of a type outside the int8 path, fp16 scale fields set to small positive
    values (random bytes there would be NaNs and infinities), plain types filled with N(0, 0.02^2) values."""
    t = int(t)
    g = rng(seed)
    if t in (0, 1, 30):
        v = (g.standard_normal((N, K)) * 0.02).astype(np.float32)
        if t == 0:
            return v.view(np.uint8).reshape(N, K * 4)
        if t == 1:
            return v.astype(np.float16).view(np.uint8).reshape(N, K * 2)
        return (v.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8).reshape(N, K * 2)
    e, b = _OTHER_GEOM[t]
    nb = K // e
    w = g.integers(0, 256, size=(N, nb, b), dtype=np.uint8)
    for off in _OTHER_SCALE_FIELDS[t]:
        d = (g.uniform(0.001, 0.05, size=(N, nb))).astype(np.float16).view(np.uint16)
        w[:, :, off] = (d & 0xFF).astype(np.uint8)
        w[:, :, off + 1] = (d >> 8).astype(np.uint8)
    return w.reshape(N, nb * b)
