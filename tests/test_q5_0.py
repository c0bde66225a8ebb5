"""Q5_0 on the int8 path. The reference's SIMD back-end serves Q5_0 with Q8 activations
(dot_row_q5_0_int_neon, src/matmul_simd.cpp:184-224; dispatched at :486, :586, :604) - plain matmuls and both
expert-indexed forms. Its own test_matmul.cpp has no Q5_0 case, so the restatement is pinned here against the
reference's compiled scalar code: dequantize() bit for bit, one-hot activations (Q8 lossless, so the int8 dot
reproduces single dequantized weights), the stored scalar outputs within activation rounding, and - in
test_oracle - the stored reference outputs on lossless activations at 1e-5."""
import numpy as np
import pytest

from tests import synth
from tests.parity import check_close
from laplace_b200.ggml import GGMLType, row_bytes

T = GGMLType.Q5_0


def test_geometry_and_packer():
    """22-byte blocks; the restated packer of tests/test_metal.cpp:36-50 against a literal loop on two blocks."""
    assert row_bytes(T, 4096) == 128 * 22
    w = synth.normal_f32(21, (1, 64), 0.02)
    got = synth.pack_ref_q5_0(w)[0]
    for b in range(2):
        x = w[0, b * 32:(b + 1) * 32]
        d = np.float32(np.abs(x).max() / np.float32(16))
        inv = np.float32(1) / d
        blk = got[b * 22:(b + 1) * 22]
        assert int(blk[0]) | (int(blk[1]) << 8) == int(synth.f32_to_f16_bits(np.array([d]))[0])
        qh = 0
        for i in range(16):
            v0, v1 = np.float32(x[i] * inv + np.float32(16)), np.float32(x[i + 16] * inv + np.float32(16))
            q0 = int(np.floor(abs(v0) + np.float32(0.5)) * np.sign(v0))
            q1 = int(np.floor(abs(v1) + np.float32(0.5)) * np.sign(v1))
            assert blk[6 + i] == (q0 & 0xF) | ((q1 & 0xF) << 4)
            qh |= ((q0 >> 4) & 1) << i
            qh |= ((q1 >> 4) & 1) << (i + 16)
        assert int.from_bytes(bytes(blk[2:6]), "little") == qh & 0xFFFFFFFF


def test_oracle_against_stored_reference_outputs(oracle, golden_dir):
    """dequantize() equals the reference build's stored values bit for bit; the restated scalar dot equals its
    stored matmul_rows; the int8 path is apart from that only by activation rounding."""
    z = np.load(golden_dir / "other_types_golden.npz")
    w, x, K = z["w_6"], z["x"], int(z["K"])
    M, N = x.shape[0], w.shape[0]
    assert np.array_equal(oracle.dequantize(w, T, N * K).view(np.uint32), z["deq_6"].view(np.uint32))
    ys = oracle.gemm_scalar(x, w, T, M, K, N)
    assert np.allclose(ys, z["y_6"], rtol=1e-5, atol=1e-6)
    y8 = oracle.gemm(x, w, T, M, K, N, mode=1).astype(np.float64)
    assert np.linalg.norm(y8 - z["y_6"]) / np.linalg.norm(z["y_6"]) < 3e-2


def test_one_hot_activations_select_single_weights(oracle, golden_dir):
    """x = 127 e_k quantizes to d = 1, q = 127 exactly, so y[j] = 127 * dequantized weight (j, k)."""
    z = np.load(golden_dir / "other_types_golden.npz")
    w, K = z["w_6"], int(z["K"])
    N = w.shape[0]
    deq = z["deq_6"].reshape(N, K).astype(np.float64)
    for k in (0, 15, 16, 31, 32, 47, 255, 300, 511):
        x = np.zeros((1, K), dtype=np.float32)
        x[0, k] = 127.0
        for mode in (0, 1):
            y = oracle.gemm(x, w, T, 1, K, N, mode=mode)[0]
            assert np.allclose(y, 127.0 * deq[:, k], rtol=2e-6, atol=1e-9), (k, mode)


def test_every_fifth_bit_is_read_from_its_own_position(oracle):
    """One block whose nibbles are all zero: value l is (bit l of qh) * 16 - 16, so a one-hot activation at l
    returns -16 d or 0 depending on that bit alone."""
    K = 32
    for qh in (0x00000001, 0x80000000, 0x00010000, 0x00008000, 0xA5A55A5A):
        blk = np.zeros(22, dtype=np.uint8)
        blk[0:2] = np.frombuffer(np.float16(1.0).tobytes(), dtype=np.uint8)
        blk[2:6] = np.frombuffer(int(qh).to_bytes(4, "little"), dtype=np.uint8)
        for l in range(32):
            x = np.zeros((1, K), dtype=np.float32)
            x[0, l] = 127.0
            y = oracle.gemm(x, blk[None], T, 1, K, 1, mode=0)[0, 0]
            assert y == 127.0 * (16.0 * ((qh >> l) & 1) - 16.0), (hex(qh), l)
            assert oracle.blocksums(x, blk[None], T, 1, K, 1)[0, 0, 0] == 127 * (16 * ((qh >> l) & 1) - 16)


# ------------------------------------------------------------------ GPU


@pytest.mark.gpu
def test_goes_through_the_int8_kernel_not_the_fp32_activation_one(oracle):
    import torch
    from laplace_b200 import device
    K, N = 4096, 320
    w = synth.weights(T, K, N, seed=6001, how="ref")
    x = synth.normal_f32(6002, (1, K))
    y = device.gemm(torch.from_numpy(x).cuda(), device.upload_weights(w), T, 1, K, N)
    device.sync()
    assert device.lib().laplace_cuda_last_path() == 1
    check_close(y.cpu().numpy(), oracle.gemm(x, w, T, 1, K, N, mode=1), "Q5_0 4096x320")
    # and is apart from the fp32-activation result by activation rounding, as in the reference
    ys = oracle.gemm_scalar(x, w, T, 1, K, N).astype(np.float64)
    rel = np.linalg.norm(y.cpu().numpy() - ys) / np.linalg.norm(ys)
    assert 1e-5 < rel < 3e-2


@pytest.mark.gpu
def test_fifth_bits_on_the_device(oracle):
    """Random payload with all 32 fifth-bit positions exercised, bit-exact block sums and one-hot activations."""
    import torch
    from laplace_b200 import device
    K, N = 256, 9
    w = synth.random_blocks(T, K, N, seed=6010)
    wd = device.upload_weights(w)
    deq = oracle.dequantize(w, T, N * K).reshape(N, K).astype(np.float64)
    x = np.zeros((8, K), dtype=np.float32)
    ks = (0, 15, 16, 31, 100, 143, 200, 255)
    for m, k in enumerate(ks):
        x[m, k] = 127.0
    y = device.gemm(torch.from_numpy(x).cuda(), wd, T, 8, K, N)
    device.sync()
    for m, k in enumerate(ks):
        assert np.allclose(y.cpu().numpy()[m], 127.0 * deq[:, k], rtol=2e-6, atol=1e-9), k
    xr = synth.normal_f32(6011, (2, K))
    bs = device.debug_blocksums(torch.from_numpy(xr).cuda(), wd, T, 2, K, N)
    device.sync()
    assert np.array_equal(bs.cpu().numpy(), oracle.blocksums(xr, w, T, 2, K, N))


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (1, 14336, 512), (8, 4096, 1024), (40, 1024, 128), (130, 512, 96)])
def test_shapes_up_to_prefill(oracle, M, K, N):
    """Any row count: more than eight rows are walked in passes of eight through the streaming kernel."""
    import torch
    from laplace_b200 import device
    w = synth.weights(T, K, N, seed=6020 + M, how="ref")
    x = synth.normal_f32(6021 + M, (M, K))
    y = device.gemm(torch.from_numpy(x).cuda(), device.upload_weights(w), T, M, K, N)
    device.sync()
    check_close(y.cpu().numpy(), oracle.gemm(x, w, T, M, K, N, mode=1, threads=8), f"Q5_0 {M}x{K}x{N}")


@pytest.mark.gpu
def test_multi_matrix_call_and_norm_prologue(oracle):
    """Q5_0 through the several-matrices-one-launch entry with the RMSNorm prologue."""
    import torch
    from laplace_b200 import device
    from tests.oracle_lib import rmsnorm_rows_np
    K, ns = 1024, (96, 40)
    ws = [synth.weights(T, K, n, seed=6030 + i, how="ref") for i, n in enumerate(ns)]
    x = synth.normal_f32(6033, (2, K))
    g = (1.0 + 0.1 * synth.normal_f32(6034, (K,))).astype(np.float32)
    ys, xn = device.gemm_multi(torch.from_numpy(x).cuda(), [device.upload_weights(w) for w in ws], T, 2, K, list(ns),
                               norm_weight=torch.from_numpy(g).cuda(), eps=1e-6, want_x_norm=True)
    device.sync()
    xr = rmsnorm_rows_np(x, g, 1e-6)
    assert np.allclose(xn.cpu().numpy(), xr, rtol=2e-6, atol=1e-7)
    for y, w, n in zip(ys, ws, ns):
        check_close(y.cpu().numpy(), oracle.gemm(xn.cpu().numpy(), w, T, 2, K, n, mode=1), f"Q5_0 multi N={n}")
