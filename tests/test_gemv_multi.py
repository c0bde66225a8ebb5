"""Several matrices against one (optionally RMS-normalised) activation in one launch (laplace_cuda_gemm_multi_dev):
the reference's  ops::rmsnorm + one matmul_rows per matrix  (src/ops.cpp:34-74, src/arch_llama.cpp:475-501)."""
import numpy as np
import pytest

from laplace_b200.ggml import GGMLType
from tests import synth
from tests.oracle_lib import Reference, rmsnorm_rows_np
from tests.parity import check_close


def test_rmsnorm_restatement_matches_the_reference_build():
    if not Reference.available() or not hasattr(Reference().lib, "ref_rmsnorm_rows"):
        pytest.skip("oracle/_ref (with src/ops.cpp) is not present")
    x = synth.normal_f32(71, (3, 1024)) * np.float32(3.0)
    w = (1.0 + 0.1 * synth.normal_f32(72, (1024,))).astype(np.float32)
    assert np.array_equal(Reference().rmsnorm_rows(x, w, 1e-5), rmsnorm_rows_np(x, w, 1e-5))


@pytest.mark.gpu
@pytest.mark.parametrize("t,M,K,Ns", [(GGMLType.Q4_K, 1, 4096, (4096, 1024, 1024)), (GGMLType.Q4_K, 1, 4096, (14336, 14336)),
                                      (GGMLType.Q6_K, 2, 1024, (96, 40)), (GGMLType.Q8_0, 5, 512, (33, 64, 8)),
                                      (GGMLType.Q4_0, 8, 256, (24,)), (GGMLType.Q4_K, 4, 2048, (200, 136)),
                                      (GGMLType.Q6_K, 1, 14336, (64, 32)),
                                      # one row of a 32-value-block type: activations held in registers
                                      (GGMLType.Q8_0, 1, 1024, (40, 24)), (GGMLType.Q4_0, 1, 4096, (33,)), (GGMLType.Q5_0, 1, 2048, (96, 40, 8))])
@pytest.mark.parametrize("norm", [False, True])
def test_multi_matrix_gemv(oracle, t, M, K, Ns, norm):
    import torch
    from laplace_b200 import device
    ws = [synth.weights(t, K, n, seed=80 + i, how="affine") for i, n in enumerate(Ns)]
    x = synth.normal_f32(90, (M, K)) * np.float32(2.5)
    nw = (1.0 + 0.1 * synth.normal_f32(91, (K,))).astype(np.float32)
    wd = [device.upload_weights(w) for w in ws]
    if norm:
        ys, xn = device.gemm_multi(torch.from_numpy(x).cuda(), wd, t, M, K, Ns, norm_weight=torch.from_numpy(nw).cuda(), eps=1e-5, want_x_norm=True)
        device.sync()
        xn = xn.cpu().numpy()
        ref_norm = Reference().rmsnorm_rows(x, nw, 1e-5) if Reference.available() and hasattr(Reference().lib, "ref_rmsnorm_rows") else rmsnorm_rows_np(x, nw, 1e-5)
        # the sum of squares is added in another order on the device: last-bit differences
        assert np.allclose(xn, ref_norm, rtol=2e-6, atol=0.0)
        x_in = xn                                  # the matmuls are checked on the device's own normalised rows
    else:
        ys = device.gemm_multi(torch.from_numpy(x).cuda(), wd, t, M, K, Ns)
        device.sync()
        x_in = x
    for y, w, n in zip(ys, ws, Ns):
        mass = oracle.gemm(x_in, w, t, M, K, n, mode=2)
        check_close(y.cpu().numpy(), oracle.gemm(x_in, w, t, M, K, n, mode=1), f"multi {t.name} M={M} K={K} N={n} norm={norm}", mass)
        # and bit-identical to a single-matrix call on the same activations (the same kernel), except where the single
        # call takes another kernel (Q4_K with 3..8 rows runs on mma.sync tiles: another fp32 summation order)
        single = device.gemm(torch.from_numpy(np.ascontiguousarray(x_in)).cuda(), device.upload_weights(w), t, M, K, n)
        device.sync()
        if t == GGMLType.Q4_K and 3 <= M <= 8 and K % 256 == 0:
            check_close(single.cpu().numpy(), y.cpu().numpy().astype(np.float64), "single (mma kernel) vs multi (dp4a kernel)", mass)
        else:
            assert np.array_equal(single.cpu().numpy(), y.cpu().numpy())


@pytest.mark.gpu
@pytest.mark.parametrize("t,M,K,Ns", [(GGMLType.Q4_K, 64, 1024, (256, 136, 128)), (GGMLType.Q6_K, 40, 2048, (200, 128)),
                                      (GGMLType.Q4_K, 512, 4096, (1024, 1024))])
@pytest.mark.parametrize("norm", [False, True])
def test_multi_matrix_prefill(oracle, t, M, K, Ns, norm):
    """More than 8 rows: one (normalising) quantizer launch, then one tensor-core GEMM per matrix on the shared operand."""
    import os
    import torch
    from laplace_b200 import device
    ws = [synth.weights(t, K, n, seed=180 + i, how="affine") for i, n in enumerate(Ns)]
    x = synth.normal_f32(190, (M, K)) * np.float32(2.5)
    nw = (1.0 + 0.1 * synth.normal_f32(191, (K,))).astype(np.float32)
    wd = [device.upload_weights(w) for w in ws]
    if norm:
        ys, xn = device.gemm_multi(torch.from_numpy(x).cuda(), wd, t, M, K, Ns, norm_weight=torch.from_numpy(nw).cuda(), eps=1e-5, want_x_norm=True)
        device.sync()
        xn = xn.cpu().numpy()
        assert np.allclose(xn, rmsnorm_rows_np(x, nw, 1e-5), rtol=2e-6, atol=0.0)
        x_in = xn
    else:
        ys = device.gemm_multi(torch.from_numpy(x).cuda(), wd, t, M, K, Ns)
        device.sync()
        x_in = x
    assert device.lib().laplace_cuda_last_path() == 2
    for y, w, n in zip(ys, ws, Ns):
        check_close(y.cpu().numpy(), oracle.gemm(x_in, w, t, M, K, n, mode=1, threads=os.cpu_count() or 1), f"multi prefill {t.name} M={M} K={K} N={n} norm={norm}")
        single = device.gemm(torch.from_numpy(np.ascontiguousarray(x_in)).cuda(), device.upload_weights(w), t, M, K, n)
        device.sync()
        assert np.array_equal(single.cpu().numpy(), y.cpu().numpy())
