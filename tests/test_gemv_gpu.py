"""GPU parity of the decode GEMV (M = 1..8) against the CPU oracle, through the C ABI.

Bars: integer block sums bit-exact; fp32 outputs within 1e-5 relative L2 and
1e-3 max-abs over the output RMS of the oracle (accumulation order differs).
"""
import numpy as np
import pytest

from tests import synth
from laplace_b200.ggml import GGMLType

pytestmark = pytest.mark.gpu

TYPES = [GGMLType.Q4_0, GGMLType.Q5_0, GGMLType.Q8_0, GGMLType.Q4_K, GGMLType.Q6_K]


from tests.parity import check_close  # noqa: E402


def run_dev(t, x, w, M, K, N):
    import torch
    from laplace_b200 import device
    xd = torch.from_numpy(x).cuda()
    wd = device.upload_weights(w)
    y = device.gemm(xd, wd, t, M, K, N)
    device.sync()
    return y.cpu().numpy()


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("how", ["random", "ref", "affine"])
@pytest.mark.parametrize("K,N", [(512, 1), (512, 8), (512, 33), (512, 256), (2816, 8), (2816, 256)])
def test_gemv_m1_reference_test_shapes(oracle, t, how, K, N):
    """Shapes of the reference's tests/test_matmul.cpp:278-291 (K=2816 there only for the K-quants)."""
    if K % 256 and t in (GGMLType.Q4_K, GGMLType.Q6_K):
        pytest.skip("K-quants need K % 256 == 0")
    w = synth.weights(t, K, N, seed=100 + int(t), how=how)
    x = synth.normal_f32(200 + int(t), (1, K))
    y = run_dev(t, x, w, 1, K, N)
    mass = oracle.gemm(x, w, t, 1, K, N, mode=2)
    check_close(y, oracle.gemm(x, w, t, 1, K, N, mode=1), f"{t.name} {how} K={K} N={N} vs f64", mass)
    check_close(y, oracle.gemm(x, w, t, 1, K, N, mode=0), f"{t.name} {how} K={K} N={N} vs f32-lanes", 2 * mass)


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("M", [2, 3, 4, 7, 8])
def test_gemv_small_batch(oracle, t, M):
    K, N = 1024, 77
    w = synth.weights(t, K, N, seed=300 + int(t), how="affine")
    x = synth.normal_f32(400 + M, (M, K))
    y = run_dev(t, x, w, M, K, N)
    check_close(y, oracle.gemm(x, w, t, M, K, N, mode=1), f"{t.name} M={M}")


@pytest.mark.parametrize("t", TYPES)
def test_long_rows_are_sliced(oracle, t):
    """K = 14336 rows exceed one stage slot, so the kernel walks K-slices."""
    K, N = 14336, 40
    w = synth.weights(t, K, N, seed=500 + int(t), how="random")
    for M in (1, 4):
        x = synth.normal_f32(600 + M, (M, K))
        y = run_dev(t, x, w, M, K, N)
        check_close(y, oracle.gemm(x, w, t, M, K, N, mode=1), f"{t.name} K=14336 M={M}")


@pytest.mark.parametrize("t", TYPES)
def test_blocksums_bit_exact(oracle, t):
    import torch
    from laplace_b200 import device
    M, K, N = 3, 1024 if t in (GGMLType.Q4_K, GGMLType.Q6_K) else 768, 19
    w = synth.weights(t, K, N, seed=700 + int(t), how="random")
    x = synth.normal_f32(800, (M, K))
    out = device.debug_blocksums(torch.from_numpy(x).cuda(), device.upload_weights(w), t, M, K, N)
    device.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.blocksums(x, w, t, M, K, N))


def test_quantizer_bit_exact(oracle):
    import torch
    from laplace_b200 import device
    M, K = 5, 4096
    x = synth.normal_f32(900, (M, K))
    x[0, :32] = 0.0                      # all-zero block: d = 0, id = 0
    x[1, 40] = 1e30                      # huge outlier
    x[2, 64:96] = 0.5                    # ties: every value equals amax
    x[3, 100] = np.float32(1e-40)        # subnormal input
    q, d, s, isum = device.quantize_act(torch.from_numpy(x).cuda(), M, K)
    device.sync()
    ref = oracle.quantize(x)
    assert np.array_equal(q.cpu().numpy().reshape(M, K // 32, 32), ref["qs"])
    assert np.array_equal(d.cpu().numpy().view(np.uint32), ref["d"].view(np.uint32))
    assert np.array_equal(s.cpu().numpy().view(np.uint32), ref["sum"].view(np.uint32))
    assert np.array_equal(isum.cpu().numpy()[..., 0], ref["sum_lo"])
    assert np.array_equal(isum.cpu().numpy()[..., 1], ref["sum_hi"])


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("multi", [False, True])
def test_moe_gemv(oracle, t, multi):
    import torch
    from laplace_b200 import device
    n_total, K, N = 6, 512, 48
    w = synth.weights(t, K, N * n_total, seed=1000 + int(t), how="affine")
    idx = np.array([4, 0, 5, 2], dtype=np.int32)
    x = synth.normal_f32(1100, (len(idx) if multi else 1, K))
    y = device.moe_gemv(torch.from_numpy(x).cuda(), device.upload_weights(w), t,
                        torch.from_numpy(idx).cuda(), K, N, per_expert_x=multi)
    device.sync()
    ref = oracle.moe_gemv(x, w, t, idx, K, N, multi=multi, mode=1)
    check_close(y.cpu().numpy(), ref, f"moe {t.name} multi={multi}")


@pytest.mark.parametrize("t", TYPES)
def test_host_pointer_entry_points(oracle, t):
    """The three reference-facing calls with host buffers (kernels.h:97,103,110)."""
    import laplace_b200 as lb
    K, N, M = 512, 64, 7
    w = synth.weights(t, K, N * 3, seed=1200 + int(t), how="random")
    x = synth.normal_f32(1300, (M, K))
    y = np.zeros((M, N), dtype=np.float32)
    lb.matmul_rows(x, lb.Tensor(t, w[:N]), y, M, K, N)
    check_close(y, oracle.gemm(x, w[:N], t, M, K, N, mode=1), "matmul_rows")
    # registered region: pointer resolved by offset
    lb.matmul_register_weights(w)
    try:
        y1 = np.zeros((1, N), dtype=np.float32)
        lb.matmul_row(x[2], lb.Tensor(t, w[N:2 * N]), y1, K, N)
        check_close(y1, oracle.gemm(x[2:3], w[N:2 * N], t, 1, K, N, mode=1), "matmul_row registered")
        idx = np.array([2, 0], dtype=np.int32)
        ym = np.zeros((2, N), dtype=np.float32)
        lb.fused_moe_gemm_idx(x[0], lb.Tensor(t, w), ym, idx, 2, K, N)
        check_close(ym, oracle.moe_gemv(x[0], w, t, idx, K, N, multi=False, mode=1), "fused_moe_gemm_idx")
        lb.fused_moe_gemm_multi(x[:2], lb.Tensor(t, w), ym, idx, 2, K, N)
        check_close(ym, oracle.moe_gemv(x[:2], w, t, idx, K, N, multi=True, mode=1), "fused_moe_gemm_multi")
    finally:
        lb.matmul_unregister_weights(w)


def test_unsupported_type_and_bad_args():
    import laplace_b200 as lb
    x = np.zeros((1, 512), dtype=np.float32)
    y = np.zeros((1, 4), dtype=np.float32)
    w = np.zeros((4, 2048), dtype=np.uint8)
    with pytest.raises(lb.LaplaceCudaError) as e:
        lb.matmul_rows(x, lb.Tensor(3, w), y, 1, 512, 4)          # Q4_1: no kernel in the reference either
    assert e.value.code == 1                   # "not handled": the reference would fall back to scalar
    with pytest.raises(lb.LaplaceCudaError) as e:
        lb.matmul_rows(x[:, :500], lb.Tensor(GGMLType.F32, w), y, 1, 500, 4)      # plain rows are walked 16 values at a time
    assert e.value.code == 1
    # K not a multiple of the block: rejected by the library itself (device-pointer call)
    import torch
    from laplace_b200 import device
    L = device.lib()
    xd = torch.zeros(512, device="cuda")
    wd = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    yd = torch.zeros(4, device="cuda")
    rc = L.laplace_cuda_gemm_dev(xd.data_ptr(), wd.data_ptr(), int(GGMLType.Q4_0), yd.data_ptr(), 1, 500, 4, None)
    assert rc == -1 and b"multiple" in L.laplace_cuda_last_error()
    rc = L.laplace_cuda_gemm_dev(None, wd.data_ptr(), int(GGMLType.Q4_0), yd.data_ptr(), 1, 512, 4, None)
    assert rc == -1


def test_nan_block_propagates(oracle):
    """A NaN activation makes its block's scale NaN in the reference (NEON FMAX), hence the whole row."""
    t, K, N = GGMLType.Q8_0, 512, 8
    w = synth.weights(t, K, N, seed=1400, how="affine")
    x = synth.normal_f32(1401, (1, K))
    x[0, 70] = np.nan
    y = run_dev(t, x, w, 1, K, N)
    ref = oracle.gemm(x, w, t, 1, K, N, mode=0)
    assert np.isnan(ref).all() and np.isnan(y).all()


@pytest.mark.parametrize("t", [GGMLType.Q6_K, GGMLType.Q8_0])
def test_long_rows_many_activation_rows(oracle, t):
    """M = 8 at K = 14336 does not fit one pass (the quantized activations would fill shared memory):
    the dispatcher splits the rows into smaller passes."""
    M, K, N = 8, 14336, 24
    w = synth.weights(t, K, N, seed=1500 + int(t), how="random")
    x = synth.normal_f32(1501, (M, K))
    y = run_dev(t, x, w, M, K, N)
    check_close(y, oracle.gemm(x, w, t, M, K, N, mode=1), f"{t.name} M=8 K=14336")


@pytest.mark.parametrize("t,M,K,N", [(GGMLType.Q4_K, 1, 4096, 512), (GGMLType.Q6_K, 4, 512, 96), (GGMLType.Q4_0, 8, 256, 40)])
def test_fused_allgather_on_one_gpu(oracle, t, M, K, N):
    """The fused all-gather path with a world of one: results go through the peer-store epilogue into the
    step's slot of the rank's own buffer, the step flag is raised and the wait kernel sees it."""
    import torch
    from laplace_b200 import device
    from laplace_b200.shard import PeerGather, RowShards
    L = device.lib()
    w = synth.weights(t, K, N, seed=700 + M, how="random")
    wd = device.upload_weights(w)
    pg = PeerGather(L, RowShards(L, N, 0, 1), M)
    try:
        for step in range(1, 4):
            x = synth.normal_f32(710 + step, (M, K))
            xd = torch.from_numpy(x).cuda()
            pg.gemm(xd, wd, t, K, device._stream())
            pg.wait(device._stream())
            device.sync()
            got = pg.slot(step).cpu().numpy()
            want = device.gemm(xd, wd, t, M, K, N)
            device.sync()
            assert np.array_equal(got, want.cpu().numpy()), f"step {step}"
            check_close(got, oracle.gemm(x, w, t, M, K, N, mode=1), f"fused all-gather {t.name} step {step}")
    finally:
        pg.close()
