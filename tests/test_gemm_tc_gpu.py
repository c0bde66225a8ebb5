"""GPU parity of the tensor-core prefill GEMM (M > 8) against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest

from tests import synth
from laplace_b200.ggml import GGMLType
from tests.parity import check_close

pytestmark = pytest.mark.gpu
THREADS = os.cpu_count() or 1


def run_dev(t, x, w, M, K, N):
    import torch
    from laplace_b200 import device
    y = device.gemm(torch.from_numpy(x).cuda(), device.upload_weights(w), t, M, K, N)
    device.sync()
    return y.cpu().numpy(), device.lib().laplace_cuda_last_path()


@pytest.mark.parametrize("how", ["random", "ref", "affine"])
@pytest.mark.parametrize("M,K,N", [(128, 512, 128), (9, 256, 8), (64, 1024, 256), (200, 2816, 200), (512, 4096, 384), (130, 768, 129),
                                   (512, 4096, 1024), (100, 2048, 130), (33, 4608, 100)])
def test_q4k_prefill(oracle, how, M, K, N):
    t = GGMLType.Q4_K
    w = synth.weights(t, K, N, seed=40 + M, how=how)
    x = synth.normal_f32(41 + N, (M, K))
    y, path = run_dev(t, x, w, M, K, N)
    assert path == 2, "the tensor-core kernel did not run"
    ref = oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS)
    check_close(y, ref, f"Q4_K prefill {how} M={M} K={K} N={N}")


def test_prefill_rows_equal_decode_rows(oracle):
    """Row m of a prefill call and a decode call on row m alone agree to fp32 rounding
    (the reference's test_batched_rows, tests/test_matmul.cpp:217-250, allows 1e-4)."""
    t, M, K, N = GGMLType.Q4_K, 64, 512, 64
    w = synth.weights(t, K, N, seed=77, how="affine")
    x = synth.normal_f32(78, (M, K))
    yb, path = run_dev(t, x, w, M, K, N)
    assert path == 2
    for m in (0, 17, 63):
        ys, p1 = run_dev(t, x[m:m + 1], w, 1, K, N)
        assert p1 == 1
        assert np.allclose(yb[m], ys[0], rtol=1e-4, atol=1e-4)


def test_prefill_through_host_entry_point(oracle):
    import laplace_b200 as lb
    t, M, K, N = GGMLType.Q4_K, 96, 512, 160
    w = synth.weights(t, K, N, seed=79, how="random")
    x = synth.normal_f32(80, (M, K))
    y = np.zeros((M, N), dtype=np.float32)
    lb.matmul_rows(x, lb.Tensor(t, w), y, M, K, N)
    check_close(y, oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), "matmul_rows prefill")


@pytest.mark.parametrize("t", [GGMLType.Q4_0, GGMLType.Q8_0, GGMLType.Q6_K])
@pytest.mark.parametrize("how", ["random", "ref", "affine"])
@pytest.mark.parametrize("M,K,N", [(20, 512, 40), (512, 4096, 4096), (130, 768, 129), (96, 2816, 200), (64, 14336, 136)])
def test_other_types_large_m(oracle, t, how, M, K, N):
    """Q4_0, Q8_0 and Q6_K (any K that is a multiple of 256) on the tensor cores: weight operand in two fp16 pieces."""
    if (M, K, N) == (512, 4096, 4096) and how != "affine":
        pytest.skip("one packing is enough at the large shape")
    w = synth.weights(t, K, N, seed=81, how=how)
    x = synth.normal_f32(82, (M, K))
    y, path = run_dev(t, x, w, M, K, N)
    assert path == 2, "the tensor-core kernel did not run"
    check_close(y, oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), f"{t.name} {how} M={M} K={K} N={N}")


@pytest.mark.parametrize("t", [GGMLType.Q4_0, GGMLType.Q8_0])
def test_block_quants_with_other_k_run_as_streaming_passes(oracle, t):
    """K that is not a multiple of 256 (legal for the 32-value block types) keeps the streaming kernel: still exact."""
    M, K, N = 20, 544, 40
    w = synth.weights(t, K, N, seed=83, how="affine")
    x = synth.normal_f32(84, (M, K))
    y, path = run_dev(t, x, w, M, K, N)
    assert path == 1
    check_close(y, oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), f"{t.name} K=544")


@pytest.mark.parametrize("how", ["random", "ref", "affine"])
@pytest.mark.parametrize("M,K,N", [(128, 2048, 128), (9, 2048, 8), (200, 4096, 200), (130, 6144, 129), (96, 14336, 256)])
def test_q6k_prefill(oracle, how, M, K, N):
    """Q6_K on the tensor cores (K a multiple of 2048): split fp16 operands, exact block sums."""
    t = GGMLType.Q6_K
    w = synth.weights(t, K, N, seed=90 + M, how=how)
    x = synth.normal_f32(91 + N, (M, K))
    y, path = run_dev(t, x, w, M, K, N)
    assert path == 2, "the tensor-core kernel did not run"
    ref = oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS)
    check_close(y, ref, f"Q6_K prefill {how} M={M} K={K} N={N}")


@pytest.mark.parametrize("ql,qh,sc", [(0x00, 0x00, -128), (0x00, 0x00, 127), (0xFF, 0xFF, -128), (0xFF, 0xFF, 127), (0x0F, 0xAA, -1)])
def test_q6k_prefill_extreme_blocks(oracle, ql, qh, sc):
    """Largest-magnitude weights (sc * (q6 - 32) = +-4096, -3968 ...) against full-scale activations:
    block sums reach 32 * 127 * 4096, just below 2^24, and must still be exact."""
    t, M, K, N = GGMLType.Q6_K, 16, 2048, 16
    blk = np.zeros(210, dtype=np.uint8)
    blk[0:128] = ql
    blk[128:192] = qh
    blk[192:208] = np.uint8(sc & 0xFF)
    blk[208:210] = np.frombuffer(np.float16(2.0 ** -12).tobytes(), dtype=np.uint8)
    w = np.tile(blk, (N, K // 256))
    x = np.full((M, K), 1.27, dtype=np.float32)
    x[1::2] *= -1.0
    x[:, ::7] *= 0.5
    y, path = run_dev(t, x, w, M, K, N)
    assert path == 2
    ref = oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS)
    assert np.allclose(y, ref, rtol=2e-5, atol=0.0), np.abs(y - ref).max()


@pytest.mark.parametrize("t,K", [(GGMLType.Q4_K, 512), (GGMLType.Q6_K, 2048)])
def test_prefill_special_rows(oracle, t, K):
    """Edge rows of a prefill call: an all-zero activation row (scale 0, result exactly 0), a row with one NaN
    (the block's scale becomes NaN as with NEON FMAX, so the whole output row is NaN), a row of a single
    large value; the other rows are unaffected."""
    M, N = 40, 128
    w = synth.weights(t, K, N, seed=95, how="random")
    x = synth.normal_f32(96, (M, K))
    x[3] = 0.0
    x[7, 33] = np.nan
    x[11] = 0.0
    x[11, K - 1] = 1.0e6
    y, path = run_dev(t, x, w, M, K, N)
    assert path == 2
    ref = oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS)
    assert np.isnan(ref[7]).all() and np.isnan(y[7]).all()
    assert not y[3].any() and not ref[3].any()
    keep = np.ones(M, dtype=bool)
    keep[7] = False
    check_close(y[keep], ref[keep], f"{t.name} prefill with special rows")
    assert np.allclose(y[11], ref[11], rtol=2e-6, atol=0.0)


def test_scratch_growth_is_refused_during_stream_capture(oracle):
    """A prefill call whose scratch would have to grow calls the allocator, which is illegal while the call's
    stream is being captured into a CUDA graph: the call is refused with LAPLACE_ERR_STATE, the capture stays
    valid, and the same call succeeds once made outside a capture (after which a capture of it works)."""
    import torch
    from laplace_b200 import device
    L = device.lib()
    t, M, K, N = GGMLType.Q4_K, 1536, 14336, 128            # needs far more scratch than any other test
    w = synth.weights(t, K, N, seed=97, how="random")
    x = synth.normal_f32(98, (M, K))
    xd, wd = torch.from_numpy(x).cuda(), device.upload_weights(w)
    y = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        g.capture_begin()
        rc = L.laplace_cuda_gemm_dev(xd.data_ptr(), wd.data_ptr(), int(t), y.data_ptr(), M, K, N, s.cuda_stream)
        g.capture_end()
    assert rc == -3 and b"captured" in L.laplace_cuda_last_error()
    with torch.cuda.stream(s):
        rc = L.laplace_cuda_gemm_dev(xd.data_ptr(), wd.data_ptr(), int(t), y.data_ptr(), M, K, N, s.cuda_stream)     # grows the scratch
        assert rc == 0, L.laplace_cuda_last_error()
        s.synchronize()
        y.zero_()
        g2 = torch.cuda.CUDAGraph()
        g2.capture_begin()
        rc = L.laplace_cuda_gemm_dev(xd.data_ptr(), wd.data_ptr(), int(t), y.data_ptr(), M, K, N, s.cuda_stream)
        g2.capture_end()
        assert rc == 0, L.laplace_cuda_last_error()
        g2.replay()
    device.sync()
    check_close(y.cpu().numpy(), oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), "captured prefill call")


def test_peer_store_form_on_one_gpu(oracle):
    """laplace_cuda_gemm_peers_dev with a world of one: the drain (and the fix-up of tiles the balanced split cut) writes
    into the rank's own peer buffer; the closing kernel advances and announces the step."""
    import torch
    from laplace_b200 import device
    from laplace_b200.shard import PeerGather, RowShards
    L = device.lib()
    # the last four: one GPU's slice of the k/v, q/o, gate/up and down projections when eight GPUs share a Llama-3-8B layer
    for t, M, K, N in ((GGMLType.Q4_K, 200, 1024, 1160), (GGMLType.Q6_K, 40, 2048, 136), (GGMLType.Q4_K, 512, 4096, 1024),
                       (GGMLType.Q4_K, 512, 4096, 128), (GGMLType.Q4_K, 512, 4096, 512), (GGMLType.Q4_K, 512, 4096, 1792),
                       (GGMLType.Q6_K, 512, 14336, 512)):
        w = synth.weights(t, K, N, seed=2300 + M, how="random")
        x = synth.normal_f32(2301 + M, (M, K))
        pg = PeerGather(L, RowShards(L, N, 0, 1), M)
        try:
            for rep in range(2):
                assert pg.gemm_peers(torch.from_numpy(x).cuda(), device.upload_weights(w), t, K, device._stream())
                pg.step_wait(device._stream())
                device.sync()
                check_close(pg.slot(0).cpu().numpy(), oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), f"peer-store GEMM {t.name} {M}x{K}x{N}")
        finally:
            pg.close()
