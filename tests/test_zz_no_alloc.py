"""The prefill entry point that allocates nothing (laplace_cuda_gemm_noalloc_dev).

It serves callers that cannot use the CUDA allocator while requests are in flight (their own
memory pools hold all HBM, or they cannot afford the allocator's locks and the device
synchronisation of a growing buffer): the quantized activations
go to an array built into the library instead of a cudaMalloc'd buffer. This file is named
to be collected last, so a run that stops at the first failure has already run everything
else; the test passes alone in a fresh process as well as after the other tests.
"""
import os

import numpy as np
import pytest

from tests import synth
from laplace_b200.ggml import GGMLType
from tests.parity import check_close

pytestmark = pytest.mark.gpu
THREADS = os.cpu_count() or 1


def _call(L, t, x, w, M, K, N):
    import torch
    from laplace_b200 import device
    xd = torch.from_numpy(x).cuda()
    wd = device.upload_weights(w)
    y_ref = device.gemm(xd, wd, t, M, K, N)                       # existing entry point (tensor-core path)
    assert L.laplace_cuda_last_path() == 2
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    rc = L.laplace_cuda_gemm_noalloc_dev(xd.data_ptr(), wd.data_ptr(), int(t), y.data_ptr(), M, K, N,
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.laplace_cuda_last_error()
    device.sync()
    return y.cpu().numpy(), y_ref.cpu().numpy()


def test_noalloc_matches_the_allocating_entry_point_twice(oracle):
    from laplace_b200 import device
    L = device.lib()
    # two calls in a row with different shapes and data: the shared array keeps the previous
    # call's contents, so the second call also checks that nothing stale leaks through
    for t, M, K, N, seed in ((GGMLType.Q4_K, 200, 1024, 136, 91), (GGMLType.Q4_K, 96, 2816, 256, 93)):
        w = synth.weights(t, K, N, seed=seed, how="random")
        x = synth.normal_f32(seed + 1, (M, K))
        a, b = _call(L, t, x, w, M, K, N)
        # same kernels on the same inputs: the tests' tolerance (1e-5 relative L2) is met with equality
        assert np.isfinite(a).all()
        assert np.linalg.norm(a.astype(np.float64) - b) <= 1e-5 * np.linalg.norm(b)
        assert np.array_equal(a, b)
        check_close(a, oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), f"noalloc vs oracle {M}x{K}x{N}")


@pytest.mark.parametrize("t,M,K,N", [(GGMLType.Q4_K, 512, 4096, 1024),      # the K-split's partial sums do not fit the array: runs unsplit
                                     (GGMLType.Q6_K, 72, 2048, 200),        # the other type the prefill kernels take
                                     (GGMLType.Q4_K, 500, 4096, 128)])      # scratch close to the array's size, K-split kept
def test_noalloc_other_plans_and_types(oracle, t, M, K, N):
    from laplace_b200 import device
    L = device.lib()
    w = synth.weights(t, K, N, seed=95, how="affine")
    x = synth.normal_f32(96, (M, K))
    a, b = _call(L, t, x, w, M, K, N)
    check_close(a, b.astype(np.float64), "noalloc vs the allocating entry point")
    check_close(a, oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), f"noalloc vs oracle {t.name} {M}x{K}x{N}")


def test_noalloc_rejects_what_it_cannot_serve():
    import torch
    from laplace_b200 import device
    L = device.lib()
    t = int(GGMLType.Q4_K)
    xd = torch.zeros(16, device="cuda")
    wd = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    # beyond the built-in array: 1024 x 8192 needs ~33 MiB
    rc = L.laplace_cuda_gemm_noalloc_dev(xd.data_ptr(), wd.data_ptr(), t, xd.data_ptr(), 1024, 8192, 128, None)
    assert rc == -5 and b"scratch" in L.laplace_cuda_last_error()
    # a decode shape is not served here (it needs no scratch in the first place)
    rc = L.laplace_cuda_gemm_noalloc_dev(xd.data_ptr(), wd.data_ptr(), t, xd.data_ptr(), 1, 256, 8, None)
    assert rc == -1
