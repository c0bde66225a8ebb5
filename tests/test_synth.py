"""The seeded input generators: sizes, determinism, and the restated reference packers against a
literal scalar transcription of what those helpers do on a tiny case."""
import numpy as np
import pytest

from tests import synth
from laplace_b200.ggml import GGMLType, row_bytes

TYPES = [GGMLType.Q4_0, GGMLType.Q5_0, GGMLType.Q8_0, GGMLType.Q4_K, GGMLType.Q6_K]


def test_lcg_matches_a_plain_loop():
    s, want = 999, []
    for _ in range(50):
        s = (s * 1103515245 + 12345) & 0xFFFFFFFF
        want.append(s >> 16)
    assert list(synth._lcg_bytes(999, 50)) == want


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("how", ["ref", "affine", "random"])
def test_shapes_and_determinism(t, how):
    K, N = 768 if t in (GGMLType.Q4_K, GGMLType.Q6_K) else 96, 7
    a = synth.weights(t, K, N, seed=3, how=how)
    b = synth.weights(t, K, N, seed=3, how=how)
    assert a.shape == (N, row_bytes(t, K)) and a.dtype == np.uint8
    assert np.array_equal(a, b)
    assert not np.array_equal(a, synth.weights(t, K, N, seed=4, how=how))


def test_affine_packers_approximate_their_input(oracle):
    w = synth.normal_f32(8, (6, 1024), 0.02)
    for t, tol in ((GGMLType.Q4_0, 0.15), (GGMLType.Q5_0, 0.08), (GGMLType.Q8_0, 0.01), (GGMLType.Q4_K, 0.12), (GGMLType.Q6_K, 0.04)):
        deq = oracle.dequantize(synth.PACK_AFFINE[t](w), t, w.size).reshape(w.shape)
        assert np.linalg.norm(deq - w) / np.linalg.norm(w) < tol, t


def test_ref_q4_k_packer_scalar_transcription():
    """pack_q4_K of the reference's tests/test_metal.cpp:61-75, loop for loop, on two blocks."""
    w = synth.normal_f32(5, (1, 512), 0.02)
    got = synth.pack_ref_q4_K(w)[0]
    rs = 999
    for b in range(2):
        x = w[0, b * 256:(b + 1) * 256]
        amax = np.float32(np.abs(x).max())
        d = np.float32(amax / np.float32(15))
        blk = got[b * 144:(b + 1) * 144]
        assert int(blk[0]) | (int(blk[1]) << 8) == int(synth.f32_to_f16_bits(np.array([d]))[0])
        assert int(blk[2]) | (int(blk[3]) << 8) == int(synth.f32_to_f16_bits(np.array([amax / np.float32(240)], dtype=np.float32))[0])
        for s in range(12):
            rs = (rs * 1103515245 + 12345) & 0xFFFFFFFF
            assert blk[4 + s] == (rs >> 16) & 0xFF
        inv = np.float32(1) / d
        for i in range(128):
            q0 = int(np.floor(abs(x[i] * inv) + np.float32(0.5)) * np.sign(x[i]))
            q1 = int(np.floor(abs(x[i + 128] * inv) + np.float32(0.5)) * np.sign(x[i + 128]))
            assert blk[16 + i] == (q0 & 0xF) | ((q1 & 0xF) << 4)


def test_ref_q6_k_packer_scalar_transcription():
    """pack_q6_K of tests/test_metal.cpp:76-96 on one block, including its byte-truncated qh shifts."""
    w = synth.normal_f32(6, (1, 256), 0.02)
    got = synth.pack_ref_q6_K(w)[0]
    x = w[0]
    d = np.float32(np.abs(x).max() / np.float32(31))
    inv = np.float32(1) / d
    ql, qh = [0] * 128, [0] * 64
    for n in range(256):
        v = x[n] * inv + np.float32(32)
        val = int(max(0, min(63, np.floor(abs(v) + np.float32(0.5)) * np.sign(v))))
        lo, hi = val & 0xF, (val >> 4) & 3
        half, l = n // 128, n % 128
        if l < 64:
            ql[half * 64 + l] = (ql[half * 64 + l] & 0xF0) | lo
        else:
            ql[half * 64 + l - 64] = (ql[half * 64 + l - 64] & 0x0F) | (lo << 4)
        qh[half * 32 + l % 32] = (qh[half * 32 + l % 32] | (hi << ((l // 16) * 2))) & 0xFF
    assert list(got[:128]) == ql and list(got[128:192]) == qh
    rs, sc = 777, []
    for _ in range(16):
        rs = (rs * 1103515245 + 12345) & 0xFFFFFFFF
        sc.append(((rs >> 16) % 64 - 32) & 0xFF)
    assert list(got[192:208]) == sc
    assert int(got[208]) | (int(got[209]) << 8) == int(synth.f32_to_f16_bits(np.array([d]))[0])
